"""Flash attention with an optional trainable (B, H, M, N) bias for NVIDIA B200.

Drop-in for the public interface of the reference project's `flash_attention.py`
(cited below as FA:<line>): the same two functions, the same two
`torch.autograd.Function` classes, the same argument order, defaults, layouts and
return values.  The compute path is libfa_sm100.so (hand-written sm_100a CUDA
kernels behind a C ABI, see include/fa_sm100.h); there is no other path.

    flash_attention_fn(q, k, v, bias=None, causal=False, sm_scale=None)          FA:848
    flash_attention_qkvpacked_fn(qkv, bias=None, causal=False, sm_scale=None)    FA:852

    q       : (B, M, H, D)      k, v : (B, N, H, D)      qkv : (B, S, 3, H, D)
    bias    : (B, H, M, N)      bool  -> scores where bias is False are ignored
                                float -> added to q.k^T * sm_scale before the softmax
    returns : (B, M, H, D) in q's dtype

If a float bias has requires_grad, backward also returns its gradient at the full
(B, H, M, N) shape (dS, written by the dK/dV kernel).
"""
from __future__ import annotations

import ctypes

import torch

from . import _cabi

_DTYPES = {torch.float16: _cabi.FA_F16, torch.bfloat16: _cabi.FA_BF16}
_HEAD_DIMS = {16, 32, 64, 128, 256}


def _stride3(t: torch.Tensor):
    st = t.stride()
    return _cabi._I64x3(st[0], st[1], st[2])


def _tile_ready(t: torch.Tensor) -> torch.Tensor:
    """(B, S, H, D) operand as the kernels need it: unit inner stride, every other
    stride and the base address a multiple of 16 bytes.  Copies only when needed."""
    s0, s1, s2, s3 = t.stride()
    ok = (s3 == 1 and s0 > 0 and s1 > 0 and s2 > 0 and (s0 | s1 | s2) % 8 == 0
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def _bias_ready(bias: torch.Tensor, elem_bytes: int) -> torch.Tensor:
    """(B, H, M, N) bias / mask with unit inner stride and 16-byte aligned pitches.
    Expanded views (stride 0 over B or H) are passed through untouched.  A bias whose
    row pitch is not a multiple of 16 bytes is copied into a padded buffer."""
    B, H, M, N = bias.shape
    st = bias.stride()
    ok = (
        st[3] == 1
        and st[2] > 0
        and all((s * elem_bytes) % 16 == 0 for s in st[:3])
        and bias.data_ptr() % 16 == 0
    )
    if ok:
        return bias
    align = 32 // elem_bytes  # 32-byte pitch lets the kernels fetch whole sectors
    n_pad = (N + align - 1) // align * align
    buf = torch.empty((B, H, M, n_pad), dtype=bias.dtype, device=bias.device)
    out = buf[..., :N]
    out.copy_(bias)
    return out


def _classify_bias(bias, q):
    """Returns (kernel_bias_tensor_or_None, kind)."""
    if bias is None:
        return None, _cabi.FA_BIAS_NONE
    if bias.dtype == torch.bool:
        return _bias_ready(bias, 1), _cabi.FA_BIAS_BOOL
    if not bias.dtype.is_floating_point:
        raise TypeError(f"bias must be a bool or floating tensor, got {bias.dtype}")
    if bias.dtype != q.dtype:
        # Any other float dtype is streamed as fp32 (the reference also adds the bias in fp32,
        # FA:52, FA:292): nothing is rounded to 16 bits, the gradient comes back in fp32.
        if bias.dtype != torch.float32:
            bias = bias.float()
        return _bias_ready(bias, 4), _cabi.FA_BIAS_F32
    return _bias_ready(bias, 2), _cabi.FA_BIAS_SAME


def _check_inputs(q, k, v, bias):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be 4-D: (B, M, H, D) / (B, N, H, D)")
    B, M, H, D = q.shape
    Bk, N, Hk, Dk = k.shape
    assert D == Dk, "q and k must share the head dimension"
    assert D in _HEAD_DIMS, "head dimension must be one of 16, 32, 64, 128, 256"
    if v.shape != k.shape:
        raise ValueError("v must have the shape of k (value head dim == query/key head dim)")
    if (Bk, Hk) != (B, H):
        raise ValueError("q and k/v disagree on batch or heads")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k, v must share one dtype: torch.float16 or torch.bfloat16")
    if not (q.is_cuda and k.device == q.device and v.device == q.device):
        raise ValueError("q, k, v must live on the same CUDA device (there is no CPU path)")
    if bias is not None:
        if tuple(bias.shape) != (B, H, M, N):
            raise ValueError(f"bias must have shape (B, H, M, N) = {(B, H, M, N)}, got {tuple(bias.shape)}")
        if bias.device != q.device:
            raise ValueError("bias must live on q's device")
    return B, M, N, H, D


def _device_index(t: torch.Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


def _params(q, k, v, o, lse, bias_t, bias_kind, causal, sm_scale):
    B, M, H, D = q.shape
    N = k.shape[1]
    p = _cabi.FaParams()
    p.struct_size = ctypes.sizeof(_cabi.FaParams)
    p.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    p.B, p.H, p.M, p.N, p.D = B, H, M, N, D
    p.dtype = _DTYPES[q.dtype]
    p.bias_kind = bias_kind
    p.causal = 1 if causal else 0
    p.write_dbias = 0
    p.sm_scale = float(sm_scale)
    p.q, p.k, p.v, p.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    p.q_stride, p.k_stride, p.v_stride, p.o_stride = _stride3(q), _stride3(k), _stride3(v), _stride3(o)
    p.lse = lse.data_ptr()
    if bias_t is not None:
        p.bias = bias_t.data_ptr()
        p.bias_stride = _stride3(bias_t)
    return p


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: torch.Tensor):
    """Handle of the current CUDA stream of t's device (the raw getter is ~10x cheaper than
    building a torch.cuda.Stream object on every call)."""
    if _raw_stream is not None:
        idx = t.device.index
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device() if idx is None else idx))
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _flash_attn_fwd(q, k, v, bias, causal, sm_scale):
    """Host launcher of the forward kernel; returns (o, lse2).  Mirrors FA:649-685.
    lse2 is the log2-domain log-sum-exp, fp32, laid out (B, H, M)."""
    B, M, N, H, D = _check_inputs(q, k, v, bias)
    _cabi.raise_if_unhealthy(_device_index(q))
    q, k, v = _tile_ready(q), _tile_ready(k), _tile_ready(v)
    bias_t, kind = _classify_bias(bias, q)
    o = q.new_empty((B, M, H, D))
    lse = torch.empty((B, H, M), device=q.device, dtype=torch.float32)
    p = _params(q, k, v, o, lse, bias_t, kind, causal, sm_scale)
    _cabi.check(_cabi.load().fa_fwd(ctypes.byref(p), _stream(q)), "fa_fwd")
    return o, lse


def _flash_attn_bwd(do, q, k, v, o, bias, causal, sm_scale, lse, dq, dk, dv, dbias):
    """Host launcher of the backward kernels; fills dq, dk, dv (and dbias) in place.
    Mirrors FA:688-763.  dbias, when given, must be a (B, H, M, N) tensor whose row pitch is a
    multiple of 16 bytes (see `_empty_dbias`): in q's dtype for a bias in q's dtype, fp32 (and
    zero-filled when causal) for any other float bias."""
    B, M, N, H, D = _check_inputs(q, k, v, bias)
    _cabi.raise_if_unhealthy(_device_index(q))
    q, k, v, o, do = (_tile_ready(t) for t in (q, k, v, o, do))
    bias_t, kind = _classify_bias(bias, q)
    delta = torch.empty((B, H, M), device=q.device, dtype=torch.float32)
    p = _params(q, k, v, o, lse, bias_t, kind, causal, sm_scale)
    p.d_o, p.do_stride = do.data_ptr(), _stride3(do)
    p.dq, p.dq_stride = dq.data_ptr(), _stride3(dq)
    p.dk, p.dk_stride = dk.data_ptr(), _stride3(dk)
    p.dv, p.dv_stride = dv.data_ptr(), _stride3(dv)
    p.delta = delta.data_ptr()
    if dbias is not None:
        p.write_dbias = 1
        p.dbias, p.dbias_stride = dbias.data_ptr(), _stride3(dbias)
    if kind == _cabi.FA_BIAS_F32 or (D == 256 and not (dbias is not None and kind == _cabi.FA_BIAS_SAME)):
        # the dK/dV stage hands dS to the dQ stage through a 16-bit scratch tensor (fp32 bias; at
        # head dim 256 always, unless the 16-bit bias gradient itself is that tensor)
        ds16 = _pitched_empty((B, H, M, N), q.dtype, q.device)
        p.ds16, p.ds16_stride = ds16.data_ptr(), _stride3(ds16)
    _cabi.check(_cabi.load().fa_bwd(ctypes.byref(p), _stream(q)), "fa_bwd")


def _empty_dbias(bias: torch.Tensor, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
    """(B, H, M, N) gradient buffer with a 16-byte aligned row pitch: dense when N allows it,
    else a view of a padded buffer (the caller compacts it afterwards).  For a 16-bit bias no
    zero fill is needed: the dK/dV kernel writes every tile, including the causally skipped
    ones (the reference relies on zeros_like, FA:799).  `zero`: fp32 gradient of a causal
    problem, whose skipped tiles nobody writes."""
    return _pitched_empty(tuple(bias.shape), dtype, bias.device, zero)


def _pitched_empty(shape, dtype: torch.dtype, device, zero: bool = False) -> torch.Tensor:
    """(B, H, M, N) tensor whose row pitch is a multiple of 16 bytes (a view of a padded buffer
    when N needs it)."""
    B, H, M, N = shape
    per16 = 16 // dtype.itemsize
    n_pad = (N + per16 - 1) // per16 * per16
    make = torch.zeros if zero else torch.empty
    buf = make((B, H, M, n_pad), dtype=dtype, device=device)
    return buf[..., :N]


def _new_dbias(bias: torch.Tensor, q: torch.Tensor, causal: bool) -> torch.Tensor:
    """Gradient buffer for `bias` as the kernels write it: q's dtype when the bias has it, else
    fp32.  Zero-filled where the kernels skip the causally masked tiles without writing them
    (fp32 gradients; every gradient at head dim 256)."""
    if bias.dtype == q.dtype:
        return _empty_dbias(bias, q.dtype, zero=bool(causal) and q.shape[-1] == 256)
    return _empty_dbias(bias, torch.float32, zero=bool(causal))


def _finish_dbias(dbias, bias):
    """Gradient as the reference returns it (FA:799): dense, in the bias's own dtype."""
    if dbias is None:
        return None
    if dbias.dtype != bias.dtype:
        return dbias.to(bias.dtype)  # also compacts a padded buffer
    return dbias if dbias.is_contiguous() else dbias.contiguous()


def _grad_like(t: torch.Tensor) -> torch.Tensor:
    """empty_like (strides preserved, as FA:796-798) when the kernels can write through those
    strides, else a contiguous tensor."""
    g = torch.empty_like(t)
    s0, s1, s2, s3 = g.stride()
    ok = s3 == 1 and s0 > 0 and s1 > 0 and s2 > 0 and (s0 | s1 | s2) % 8 == 0 and g.data_ptr() % 16 == 0
    return g if ok else torch.empty(t.shape, dtype=t.dtype, device=t.device)


class FlashAttentionFn(torch.autograd.Function):
    """Separate q, k, v.  Mirrors FlashAttentionFn of the reference (FA:766-803)."""

    @staticmethod
    def forward(ctx, q, k, v, bias=None, causal=False, sm_scale=None):
        D = q.shape[-1]
        sm_scale = (D ** -0.5) if sm_scale is None else sm_scale
        is_bias = bias is not None
        is_bias_trainable = bool(is_bias and bias.requires_grad)
        if is_bias_trainable and bias.dtype == torch.bool:
            raise TypeError("a bool mask cannot require grad")
        o, lse = _flash_attn_fwd(q, k, v, bias, causal, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, bias)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.is_bias = is_bias
        ctx.is_bias_trainable = is_bias_trainable
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, bias = ctx.saved_tensors
        dq, dk, dv = _grad_like(q), _grad_like(k), _grad_like(v)
        dbias = _new_dbias(bias, q, ctx.causal) if ctx.is_bias_trainable else None
        _flash_attn_bwd(do, q, k, v, o, bias, ctx.causal, ctx.sm_scale, lse, dq, dk, dv, dbias)
        return dq, dk, dv, _finish_dbias(dbias, bias), None, None


class FlashAttentionQKVPackedFn(torch.autograd.Function):
    """Packed (B, S, 3, H, D) input; q, k, v are strided views and the three
    gradients are written into views of one dqkv tensor.  Mirrors FA:806-845."""

    @staticmethod
    def forward(ctx, qkv, bias=None, causal=False, sm_scale=None):
        if qkv.dim() != 5 or qkv.shape[2] != 3:
            raise ValueError("qkv must be (B, S, 3, H, D)")
        D = qkv.shape[-1]
        sm_scale = (D ** -0.5) if sm_scale is None else sm_scale
        is_bias = bias is not None
        is_bias_trainable = bool(is_bias and bias.requires_grad)
        if is_bias_trainable and bias.dtype == torch.bool:
            raise TypeError("a bool mask cannot require grad")
        o, lse = _flash_attn_fwd(qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], bias, causal, sm_scale)
        ctx.save_for_backward(qkv, o, lse, bias)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.is_bias = is_bias
        ctx.is_bias_trainable = is_bias_trainable
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, bias = ctx.saved_tensors
        dqkv = torch.empty_like(qkv)
        if not dqkv.is_contiguous():
            dqkv = torch.empty(qkv.shape, dtype=qkv.dtype, device=qkv.device)
        dbias = _new_dbias(bias, qkv, ctx.causal) if ctx.is_bias_trainable else None
        _flash_attn_bwd(
            do, qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], o, bias, ctx.causal, ctx.sm_scale, lse,
            dqkv[:, :, 0], dqkv[:, :, 1], dqkv[:, :, 2], dbias,
        )
        return dqkv, _finish_dbias(dbias, bias), None, None


def flash_attention_fn(q, k, v, bias=None, causal=False, sm_scale=None):
    return FlashAttentionFn.apply(q, k, v, bias, causal, sm_scale)


def flash_attention_qkvpacked_fn(qkv, bias=None, causal=False, sm_scale=None):
    return FlashAttentionQKVPackedFn.apply(qkv, bias, causal, sm_scale)
