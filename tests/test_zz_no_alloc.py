"""GPU test of fa_bwd_static_scratch, the backward entry point for callers that have
no way to allocate device memory (plugins inside a runtime with a fixed memory plan,
real-time loops, bindings without an allocator): its scratch lives in a fixed device
array inside the library instead of a caller-provided `delta` tensor.

The test calls it through the C ABI and compares dq, dk, dv and dbias with what the
regular fa_bwd entry point (caller-allocated scratch) produces from the same inputs,
twice in a row with different problems, so that contents left in the shared array by
the first call cannot help or hurt the second.  The file name sorts last on purpose.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 2097152  # B * H * M limit stated in include/fa_sm100.h


def _backward_both_ways(B, M, N, H, D, dtype, causal, seed):
    from triton_flashattn_b200 import _cabi
    from triton_flashattn_b200 import flash_attention as fa

    lib = _cabi.load()
    g = torch.Generator().manual_seed(seed)
    q, k, v, do = (torch.randn(B, s, H, D, generator=g).to(dtype).cuda() for s in (M, N, N, M))
    bias = (0.5 * torch.randn(B, H, M, N, generator=g)).to(dtype).cuda()
    scale = D ** -0.5
    o, lse = fa._flash_attn_fwd(q, k, v, bias, causal, scale)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    results = []
    for entry, own_scratch in ((lib.fa_bwd, True), (lib.fa_bwd_static_scratch, False)):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbias = fa._empty_dbias(bias, dtype)
        bias_t, kind = fa._classify_bias(bias, q)
        p = fa._params(q, k, v, o, lse, bias_t, kind, causal, scale)
        p.d_o, p.do_stride = do.data_ptr(), fa._stride3(do)
        p.dq, p.dq_stride = dq.data_ptr(), fa._stride3(dq)
        p.dk, p.dk_stride = dk.data_ptr(), fa._stride3(dk)
        p.dv, p.dv_stride = dv.data_ptr(), fa._stride3(dv)
        p.write_dbias = 1
        p.dbias, p.dbias_stride = dbias.data_ptr(), fa._stride3(dbias)
        delta = torch.empty((B, H, M), device="cuda", dtype=torch.float32) if own_scratch else None
        p.delta = delta.data_ptr() if own_scratch else None  # the new entry point ignores it
        _cabi.check(entry(ctypes.byref(p), stream), "backward")
        torch.cuda.synchronize()
        results.append({"dq": dq, "dk": dk, "dv": dv, "dbias": dbias.clone()})
    assert _cabi.device_status(0)[0] == 0
    return results


def test_static_scratch_backward_matches_regular_backward_twice():
    tol = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
    for (B, M, N, H, D, dtype, causal, seed) in ((2, 384, 320, 2, 128, torch.bfloat16, True, 21),
                                                 (1, 200, 136, 3, 64, torch.float16, False, 22)):
        ref, new = _backward_both_ways(B, M, N, H, D, dtype, causal, seed)
        for name in ref:
            err = (ref[name].float() - new[name].float()).abs().max().item()
            assert err <= tol[dtype], f"{name}: {err}"


def test_static_scratch_refuses_problems_beyond_its_limit():
    from triton_flashattn_b200 import _cabi

    p = _cabi.FaParams()
    p.struct_size = ctypes.sizeof(_cabi.FaParams)
    p.B, p.H, p.M, p.N, p.D = 64, 64, 1024, 128, 64  # 4,194,304 rows > MAX_ROWS
    assert p.B * p.H * p.M > MAX_ROWS
    rc = _cabi.load().fa_bwd_static_scratch(ctypes.byref(p), None)
    assert rc == 9 and "limit" in _cabi.status_string(rc)
