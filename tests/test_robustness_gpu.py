"""GPU tests of what surrounds the arithmetic: the failure path of the bounded waits, stores
staying inside the tensors they belong to, and back-to-back calls without synchronisation.
Nothing here hangs, traps or faults a GPU: the one provoked failure is a wait with a short
limit on a barrier that nothing completes, after which the kernel returns normally."""
import ctypes

import pytest
import torch

from tests._util import make_inputs

pytestmark = pytest.mark.gpu

BF, HF = torch.bfloat16, torch.float16


def _bwd_params(fa, q, k, v, o, lse, bias, causal, scale, do, dq, dk, dv, dbias, delta):
    bias_t, kind = fa._classify_bias(bias, q)
    p = fa._params(q, k, v, o, lse, bias_t, kind, causal, scale)
    p.d_o, p.do_stride = do.data_ptr(), fa._stride3(do)
    p.dq, p.dq_stride = dq.data_ptr(), fa._stride3(dq)
    p.dk, p.dk_stride = dk.data_ptr(), fa._stride3(dk)
    p.dv, p.dv_stride = dv.data_ptr(), fa._stride3(dv)
    p.delta = delta.data_ptr() if delta is not None else None
    if dbias is not None:
        p.write_dbias = 1
        p.dbias, p.dbias_stride = dbias.data_ptr(), fa._stride3(dbias)
    return p, bias_t


def test_abandoned_wait_is_reported_and_service_resumes_after_reset():
    """A wait that runs out (1 ms limit, barrier nobody arms): the kernel returns, the status
    word names kernel and site, the host copy lets the next API call raise without a
    synchronisation, kernels launched meanwhile do no work, and a reset restores service."""
    from triton_flashattn_b200 import _cabi, flash_attention_fn

    lib = _cabi.load()
    words = _cabi.health_words(0)
    assert words[0] == 0
    q, k, v, _, _ = make_inputs(1, 128, 128, 1, 64, HF, None, 40)
    good = flash_attention_fn(q, k, v)
    torch.cuda.synchronize()
    try:
        _cabi.check(lib.fa_selftest_wait_timeout(0, 1000, None), "fa_selftest_wait_timeout")
        torch.cuda.synchronize()  # the kernel came back by itself
        st = _cabi.device_status(0)
        assert st[:6] == [1, 101, 0, 0, 7, 1000], st
        assert list(words[:6]) == st[:6]  # host copy, written by the kernel
        out32 = (ctypes.c_int32 * 8)()
        assert lib.fa_last_device_status(0, out32) == 7  # FA_ERR_DEVICE_WAIT
        # the public API refuses to hand out tensors nobody computed
        with pytest.raises(RuntimeError, match="abandoned a bounded wait"):
            flash_attention_fn(q, k, v)
        # through the C ABI a launch is still accepted, and documented to do no work
        from triton_flashattn_b200 import flash_attention as fa
        o = torch.full_like(q, 7.0)
        lse = torch.full((1, 1, 128), 7.0, device="cuda")
        p = fa._params(q, k, v, o, lse, None, _cabi.FA_BIAS_NONE, False, 0.125)
        assert lib.fa_fwd(ctypes.byref(p), None) == 0
        torch.cuda.synchronize()
        assert torch.all(o == 7.0) and torch.all(lse == 7.0)
    finally:
        _cabi.reset_device_status(0)
    assert _cabi.device_status(0)[0] == 0 and words[0] == 0
    again = flash_attention_fn(q, k, v)
    torch.cuda.synchronize()
    assert torch.equal(again, good)


SENT16 = 0x7B7B  # bit pattern written around every output (a large finite 16-bit float)


def _guarded(shape, dtype, pad_elems=4096):
    """A tensor of `shape` carved out of the middle of a sentinel-filled buffer; returns
    (view, whole buffer as int16/int32 words, slice of the payload)."""
    n = 1
    for s in shape:
        n *= s
    buf = torch.empty(n + 2 * pad_elems, dtype=dtype, device="cuda")
    raw = buf.view(torch.int16 if dtype.itemsize == 2 else torch.int32)
    raw.fill_(SENT16 if dtype.itemsize == 2 else 0x7B7B7B7B)
    return buf[pad_elems:pad_elems + n].view(shape), raw, slice(pad_elems, pad_elems + n)


def _guards_intact(raw, payload):
    sent = SENT16 if raw.dtype == torch.int16 else 0x7B7B7B7B
    return bool(torch.all(raw[:payload.start] == sent)) and bool(torch.all(raw[payload.stop:] == sent))


@pytest.mark.parametrize("M,N,D,causal,bias_kind", [(200, 136, 64, False, "float"), (300, 100, 128, True, "float"),
                                                    (129, 1, 64, False, "float"), (100, 300, 32, True, "bool"),
                                                    (384, 384, 128, True, "float"), (50, 70, 16, False, None)])
def test_stores_stay_inside_their_tensors(M, N, D, causal, bias_kind, device_ok):
    """o, lse, delta, dq, dk, dv and dbias are carved out of sentinel-filled buffers; after a
    forward and a backward through the C ABI the sentinels around them, and the pad columns of
    the dbias rows, are untouched and every payload element has been written."""
    from triton_flashattn_b200 import _cabi
    from triton_flashattn_b200 import flash_attention as fa

    lib = _cabi.load()
    B, H = 2, 2
    q, k, v, bias, do = make_inputs(B, M, N, H, D, BF, bias_kind, 50)
    scale = D ** -0.5
    o, o_raw, o_pl = _guarded((B, M, H, D), BF)
    lse, lse_raw, lse_pl = _guarded((B, H, M), torch.float32)
    delta, delta_raw, delta_pl = _guarded((B, H, M), torch.float32)
    dq, dq_raw, dq_pl = _guarded((B, M, H, D), BF)
    dk, dk_raw, dk_pl = _guarded((B, N, H, D), BF)
    dv, dv_raw, dv_pl = _guarded((B, N, H, D), BF)
    dbias = dbias_full = None
    if bias_kind == "float":
        n_pad = (N + 7) // 8 * 8 + 8  # always at least 8 pad columns per row
        dbias_full, db_raw, db_pl = _guarded((B, H, M, n_pad), BF)
        dbias = dbias_full[..., :N]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p, keep = _bwd_params(fa, q, k, v, o, lse, bias, causal, scale, do, dq, dk, dv, dbias, delta)
    _cabi.check(lib.fa_fwd(ctypes.byref(p), stream), "fa_fwd")
    _cabi.check(lib.fa_bwd(ctypes.byref(p), stream), "fa_bwd")
    torch.cuda.synchronize()
    for name, raw, pl in (("o", o_raw, o_pl), ("lse", lse_raw, lse_pl), ("delta", delta_raw, delta_pl),
                          ("dq", dq_raw, dq_pl), ("dk", dk_raw, dk_pl), ("dv", dv_raw, dv_pl)):
        assert _guards_intact(raw, pl), f"{name}: a store landed outside the tensor"
        sent = SENT16 if raw.dtype == torch.int16 else 0x7B7B7B7B
        assert not bool(torch.any(raw[pl] == sent)), f"{name}: an element was never written"
    if dbias is not None:
        assert _guards_intact(db_raw, db_pl), "dbias: a store landed outside the buffer"
        # A bulk tensor store is clipped at the tensor's extent N, but the hardware writes whole
        # 16-byte units: the bytes between element N and the next 16-byte boundary of a row may
        # be overwritten (with the zeros dS holds for keys >= N).  That is why a dbias row pitch
        # must be a multiple of 16 bytes.  Everything from that boundary on must be untouched.
        n16 = (N + 7) // 8 * 8
        tail = dbias_full[..., N:n16].contiguous().view(torch.int16)
        touched = int((tail != SENT16).sum().item())
        print(f"dbias N={N}: {touched} of {tail.numel()} elements between N and the 16-byte boundary were written",
              flush=True)
        # (+0 or -0: dS of a masked key is 0 * (dP - delta))
        assert bool(torch.all((tail == SENT16) | ((tail & 0x7FFF) == 0))), \
            "dbias: garbage between N and the 16-byte boundary"
        pads = dbias_full[..., n16:].contiguous().view(torch.int16)
        assert bool(torch.all(pads == SENT16)), "dbias: a store landed in the pad columns of a row"
        assert not bool(torch.any(dbias.contiguous().view(torch.int16) == SENT16)), "dbias: unwritten element"


@pytest.mark.parametrize("static_scratch", [False, True])
def test_back_to_back_steps_without_sync(static_scratch, device_ok):
    """Two different problems of the same shape enqueued one after the other on one stream with
    no synchronisation in between, re-using the very same scratch and output addresses (every
    kernel may start while its predecessor still runs).  The second step's results must be
    bitwise what that problem gives when run alone."""
    from triton_flashattn_b200 import _cabi
    from triton_flashattn_b200 import flash_attention as fa

    lib = _cabi.load()
    entry = lib.fa_bwd_static_scratch if static_scratch else lib.fa_bwd
    B, M, N, H, D, causal = 2, 640, 512, 4, 128, True
    scale = D ** -0.5
    X = make_inputs(B, M, N, H, D, BF, "float", 60)
    Y = make_inputs(B, M, N, H, D, BF, "float", 61)
    o, lse = torch.empty_like(X[0]), torch.empty((B, H, M), device="cuda", dtype=torch.float32)
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(X[0]), torch.empty_like(X[1]), torch.empty_like(X[2])
    dbias = fa._empty_dbias(X[3], BF)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def enqueue(inp):
        q, k, v, bias, do = inp
        p, keep = _bwd_params(fa, q, k, v, o, lse, bias, causal, scale, do, dq, dk, dv, dbias,
                              None if static_scratch else delta)
        _cabi.check(lib.fa_fwd(ctypes.byref(p), stream), "fa_fwd")
        _cabi.check(entry(ctypes.byref(p), stream), "backward")

    def snapshot():
        torch.cuda.synchronize()
        return [t.clone() for t in (o, lse, dq, dk, dv, dbias)]

    enqueue(Y)
    alone = snapshot()
    enqueue(X)
    enqueue(Y)  # no synchronisation between the two steps
    after = snapshot()
    for name, a, b in zip(("o", "lse", "dq", "dk", "dv", "dbias"), alone, after):
        assert torch.equal(a, b), f"{name} of the second step differs from the same step run alone"
