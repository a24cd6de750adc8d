"""CPU tests of the C-ABI boundary: the shared library loads, exports exactly what
include/fa_sm100.h declares, the ctypes mirror of fa_params has the C layout, and
argument validation answers with error codes before any CUDA call is made."""
import ctypes
import os
import re
import subprocess

import pytest

from triton_flashattn_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "fa_sm100.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _cabi.load()
    declared = _declared_functions()
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in fa_sm100.h but not exported"
    assert sorted(_cabi.EXPORTED_SYMBOLS) == sorted(n for n in declared if n in _cabi.EXPORTED_SYMBOLS)


def test_version_and_status_strings():
    lib = _cabi.load()
    assert lib.fa_version() == 2
    assert _cabi.status_string(0) == "ok"
    for code in range(1, 10):
        assert _cabi.status_string(code) not in ("ok", "unknown error code")
    assert _cabi.status_string(12345) == "unknown error code"


def test_struct_layout_matches_the_header(tmp_path):
    src = tmp_path / "sz.c"
    src.write_text(
        '#include "fa_sm100.h"\n#include <stdio.h>\n#include <stddef.h>\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(fa_params), offsetof(fa_params, sm_scale),"
        " offsetof(fa_params, q), offsetof(fa_params, delta), offsetof(fa_params, dbias_stride),"
        " offsetof(fa_params, ds16), offsetof(fa_params, ds16_stride));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    c = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    P = _cabi.FaParams
    assert c == [ctypes.sizeof(P), P.sm_scale.offset, P.q.offset, P.delta.offset, P.dbias_stride.offset,
                 P.ds16.offset, P.ds16_stride.offset]


def _params(**kw):
    p = _cabi.FaParams()
    p.struct_size = ctypes.sizeof(_cabi.FaParams)
    p.B = p.H = 1
    p.M = p.N = 128
    p.D = 64
    p.dtype = _cabi.FA_BF16
    p.sm_scale = 0.125
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("entry", ["fa_fwd", "fa_bwd", "fa_bwd_pre", "fa_bwd_dkdv", "fa_bwd_dq"])
def test_validation_error_codes_without_a_gpu(entry):
    fn = getattr(_cabi.load(), entry)
    assert fn(None, None) == 2  # FA_ERR_NULL
    assert fn(ctypes.byref(_params(struct_size=8)), None) == 1  # FA_ERR_ABI
    assert fn(ctypes.byref(_params(M=0)), None) == 3  # FA_ERR_SHAPE
    assert fn(ctypes.byref(_params(D=48)), None) == 3
    assert fn(ctypes.byref(_params(D=256)), None) == 2  # a legal head dim: next complaint is the null pointers
    assert fn(ctypes.byref(_params(dtype=7)), None) == 4  # FA_ERR_DTYPE
    assert fn(ctypes.byref(_params(bias_kind=9)), None) == 4
    assert fn(ctypes.byref(_params()), None) == 2  # pointers are null
    assert fn(ctypes.byref(_params(B=70000)), None) in (2, 9)


def test_selftest_entry_validates_arguments():
    lib = _cabi.load()
    assert lib.fa_selftest_umma(0, 1, None, None, None, 0, None) == 2
    assert lib.fa_last_device_status(0, None) == 2


def test_public_api_rejects_cpu_tensors_loudly():
    import torch
    from triton_flashattn_b200 import flash_attention_fn

    q = torch.randn(1, 16, 1, 16, dtype=torch.float16)
    with pytest.raises(ValueError, match="no CPU path"):
        flash_attention_fn(q, q, q)
