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
    # both entry points run the same deterministic kernels on the same inputs, so the results
    # must agree bit for bit (tolerance 0), on two calls in a row with different problems
    for (B, M, N, H, D, dtype, causal, seed) in ((2, 384, 320, 2, 128, torch.bfloat16, True, 21),
                                                 (1, 200, 136, 3, 64, torch.float16, False, 22)):
        ref, new = _backward_both_ways(B, M, N, H, D, dtype, causal, seed)
        for name in ref:
            assert torch.equal(ref[name], new[name]), f"{name} differs between fa_bwd and fa_bwd_static_scratch"


def test_static_scratch_at_its_row_limit_allocates_nothing():
    """B * H * M exactly at the limit (2,097,152 rows; the long-sequence benchmark configuration
    has this many): accepted, bitwise equal to the regular entry point, and the amount of free
    device memory is the same before and after the call."""
    from triton_flashattn_b200 import _cabi
    from triton_flashattn_b200 import flash_attention as fa

    lib = _cabi.load()
    B, H, M, N, D, dtype = 8, 32, 8192, 128, 64, torch.bfloat16
    assert B * H * M == MAX_ROWS
    g = torch.Generator(device="cuda").manual_seed(23)
    rnd = lambda *shape: torch.randn(*shape, generator=g, device="cuda").to(dtype)
    q, k, v, do = rnd(B, M, H, D), rnd(B, N, H, D), rnd(B, N, H, D), rnd(B, M, H, D)
    bias = (0.5 * torch.randn(B, H, M, N, generator=g, device="cuda")).to(dtype)
    scale = D ** -0.5
    o, lse = fa._flash_attn_fwd(q, k, v, bias, False, scale)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for entry, own in ((lib.fa_bwd, True), (lib.fa_bwd_static_scratch, False)):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbias = fa._empty_dbias(bias, dtype)
        delta = torch.empty((B, H, M), device="cuda", dtype=torch.float32) if own else None
        bias_t, kind = fa._classify_bias(bias, q)
        p = fa._params(q, k, v, o, lse, bias_t, kind, False, scale)
        p.d_o, p.do_stride = do.data_ptr(), fa._stride3(do)
        p.dq, p.dq_stride = dq.data_ptr(), fa._stride3(dq)
        p.dk, p.dk_stride = dk.data_ptr(), fa._stride3(dk)
        p.dv, p.dv_stride = dv.data_ptr(), fa._stride3(dv)
        p.write_dbias = 1
        p.dbias, p.dbias_stride = dbias.data_ptr(), fa._stride3(dbias)
        p.delta = delta.data_ptr() if own else None
        if not own:
            # an earlier call has resolved the array's address; from here on the entry point
            # must not change the amount of free device memory
            _cabi.check(entry(ctypes.byref(p), stream), "warm-up call")
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
        _cabi.check(entry(ctypes.byref(p), stream), "backward")
        torch.cuda.synchronize()
        if not own:
            assert torch.cuda.mem_get_info()[0] == free_before, "device memory changed across the call"
        outs.append((dq, dk, dv, dbias))
    assert _cabi.device_status(0)[0] == 0
    for name, a, b in zip(("dq", "dk", "dv", "dbias"), *outs):
        assert torch.equal(a, b), name
    p.M += 1  # one row beyond the limit is refused
    assert lib.fa_bwd_static_scratch(ctypes.byref(p), stream) == 9


def test_static_scratch_refuses_problems_beyond_its_limit():
    from triton_flashattn_b200 import _cabi

    p = _cabi.FaParams()
    p.struct_size = ctypes.sizeof(_cabi.FaParams)
    p.B, p.H, p.M, p.N, p.D = 64, 64, 1024, 128, 64  # 4,194,304 rows > MAX_ROWS
    assert p.B * p.H * p.M > MAX_ROWS
    rc = _cabi.load().fa_bwd_static_scratch(ctypes.byref(p), None)
    assert rc == 9 and "limit" in _cabi.status_string(rc)
