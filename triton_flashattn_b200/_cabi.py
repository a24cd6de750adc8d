"""ctypes binding of libfa_sm100.so (declared in include/fa_sm100.h).

The library is the only compute path of this package: if it cannot be loaded the
import of the public API fails with a clear error instead of falling back to
anything else.
"""
from __future__ import annotations

import ctypes
import os

_LIB_NAME = "libfa_sm100.so"
_PKG_DIR = os.path.dirname(os.path.abspath(__file__))

FA_F16, FA_BF16 = 0, 1
FA_BIAS_NONE, FA_BIAS_SAME, FA_BIAS_BOOL, FA_BIAS_F32 = 0, 1, 2, 3
FA_OK = 0

_I64x3 = ctypes.c_int64 * 3


class FaParams(ctypes.Structure):
    """Mirror of `struct fa_params`; field order and types must match the header."""

    _fields_ = [
        ("struct_size", ctypes.c_uint32),
        ("device", ctypes.c_int32),
        ("B", ctypes.c_int32),
        ("H", ctypes.c_int32),
        ("M", ctypes.c_int32),
        ("N", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("bias_kind", ctypes.c_int32),
        ("causal", ctypes.c_int32),
        ("write_dbias", ctypes.c_int32),
        ("sm_scale", ctypes.c_float),
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("d_o", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("dbias", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("delta", ctypes.c_void_p),
        ("q_stride", _I64x3),
        ("k_stride", _I64x3),
        ("v_stride", _I64x3),
        ("o_stride", _I64x3),
        ("do_stride", _I64x3),
        ("dq_stride", _I64x3),
        ("dk_stride", _I64x3),
        ("dv_stride", _I64x3),
        ("bias_stride", _I64x3),
        ("dbias_stride", _I64x3),
        ("ds16", ctypes.c_void_p),
        ("ds16_stride", _I64x3),
    ]


EXPORTED_SYMBOLS = (
    "fa_version",
    "fa_launch_count",
    "fa_status_string",
    "fa_fwd",
    "fa_bwd",
    "fa_bwd_static_scratch",
    "fa_bwd_pre",
    "fa_bwd_dkdv",
    "fa_bwd_dq",
    "fa_last_device_status",
    "fa_reset_device_status",
    "fa_set_status_mirror",
    "fa_selftest_umma",
    "fa_selftest_wait_timeout",
)

_lib = None


def lib_path() -> str:
    return os.path.join(_PKG_DIR, _LIB_NAME)


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises ImportError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m triton_flashattn_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback path."
        )
    lib = ctypes.CDLL(path)
    P = ctypes.POINTER(FaParams)
    lib.fa_version.restype = ctypes.c_int
    lib.fa_launch_count.restype = ctypes.c_uint64
    lib.fa_status_string.restype = ctypes.c_char_p
    lib.fa_status_string.argtypes = [ctypes.c_int]
    for name in ("fa_fwd", "fa_bwd", "fa_bwd_static_scratch", "fa_bwd_pre", "fa_bwd_dkdv", "fa_bwd_dq"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int
        fn.argtypes = [P, ctypes.c_void_p]
    lib.fa_last_device_status.restype = ctypes.c_int
    lib.fa_last_device_status.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int32)]
    lib.fa_reset_device_status.restype = ctypes.c_int
    lib.fa_reset_device_status.argtypes = [ctypes.c_int]
    lib.fa_selftest_umma.restype = ctypes.c_int
    lib.fa_selftest_umma.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    lib.fa_set_status_mirror.restype = ctypes.c_int
    lib.fa_set_status_mirror.argtypes = [ctypes.c_int, ctypes.c_void_p]
    lib.fa_selftest_wait_timeout.restype = ctypes.c_int
    lib.fa_selftest_wait_timeout.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p]
    _lib = lib
    return lib


# Per device: (pinned torch tensor kept alive, ctypes view of its 8 words).  A kernel that
# abandons a bounded wait writes its record there, so every API call can check the health of
# the device with one host memory read instead of a synchronisation.
_mirrors: dict[int, tuple] = {}


def health_words(device: int):
    """ctypes int32[8] view of the host copy of `device`'s status word (registered on first use)."""
    m = _mirrors.get(device)
    if m is None:
        import torch

        t = torch.zeros(8, dtype=torch.int32).pin_memory()
        check(load().fa_set_status_mirror(device, t.data_ptr()), "fa_set_status_mirror")
        m = (t, (ctypes.c_int32 * 8).from_address(t.data_ptr()))
        _mirrors[device] = m
    return m[1]


def raise_if_unhealthy(device: int) -> None:
    """Raises when a kernel on `device` has abandoned a wait since the last reset: from then on
    every kernel of the library returns without doing any work, so results would be garbage."""
    w = health_words(device)
    if w[0] != 0:
        raise RuntimeError(
            f"a kernel on cuda:{device} abandoned a bounded wait (kernel {w[1]}, block {w[2]}, "
            f"site {w[4]}, iteration {w[5]}); later kernels do no work until "
            "_cabi.reset_device_status() is called")


def status_string(code: int) -> str:
    return load().fa_status_string(code).decode()


def check(code: int, what: str) -> None:
    if code != FA_OK:
        raise RuntimeError(f"{what} failed: {status_string(code)} (code {code})")


def device_status(device: int) -> list[int]:
    """Synchronises `device` and returns its 8-word kernel status (all zero = healthy)."""
    out = (ctypes.c_int32 * 8)()
    load().fa_last_device_status(device, out)
    return list(out)


def reset_device_status(device: int) -> None:
    check(load().fa_reset_device_status(device), "fa_reset_device_status")
