"""Caller-side conveniences around the two attention launchers.

* ``torch.ops.triton_flashattn_b200.attn_fwd`` / ``attn_bwd``: the launchers registered as
  ``torch.library`` custom operators (with shape-only "fake" implementations and an autograd
  formula), so that graph capture (``torch.compile``, ``torch.export``) sees one opaque node
  per direction instead of tracing into ctypes.
* ``flash_attention_op``: same call signature and results as ``flash_attention_fn``, routed
  through those operators.
* ``FlashAttention``: an ``nn.Module`` holding ``causal`` / ``sm_scale``.

The reference project has no counterpart (it imports ``torch.nn`` but defines no module,
flash_attention.py line 6); the arithmetic is the one of ``flash_attention.py`` here.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from . import flash_attention as _fa

_NS = "triton_flashattn_b200"


@torch.library.custom_op(f"{_NS}::attn_fwd", mutates_args=(), device_types="cuda")
def attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, bias: Optional[torch.Tensor],
             causal: bool, sm_scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(out (B,M,H,D), lse2 (B,H,M) fp32) of the forward kernel."""
    return _fa._flash_attn_fwd(q, k, v, bias, causal, sm_scale)


@attn_fwd.register_fake
def _attn_fwd_fake(q, k, v, bias, causal, sm_scale):
    B, M, H, D = q.shape
    return q.new_empty((B, M, H, D)), q.new_empty((B, H, M), dtype=torch.float32)


@torch.library.custom_op(f"{_NS}::attn_bwd", mutates_args=(), device_types="cuda")
def attn_bwd(do: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor,
             lse: torch.Tensor, bias: Optional[torch.Tensor], causal: bool, sm_scale: float,
             need_dbias: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dq, dk, dv, dbias); dbias is an empty (0,) tensor unless `need_dbias`."""
    dq, dk, dv = _fa._grad_like(q), _fa._grad_like(k), _fa._grad_like(v)
    dbias = _fa._new_dbias(bias, q, causal) if need_dbias else None
    _fa._flash_attn_bwd(do, q, k, v, o, bias, causal, sm_scale, lse, dq, dk, dv, dbias)
    dbias = q.new_empty((0,)) if dbias is None else _fa._finish_dbias(dbias, bias)
    return dq, dk, dv, dbias


@attn_bwd.register_fake
def _attn_bwd_fake(do, q, k, v, o, lse, bias, causal, sm_scale, need_dbias):
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if not need_dbias:
        return dq, dk, dv, q.new_empty((0,))
    return dq, dk, dv, bias.new_empty(tuple(bias.shape))  # dense, in the bias's dtype


def _setup_context(ctx, inputs, output):
    q, k, v, bias, causal, sm_scale = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse, bias)
    ctx.causal, ctx.sm_scale = causal, sm_scale
    ctx.need_dbias = bool(bias is not None and bias.requires_grad)


def _backward(ctx, do, _dlse):
    q, k, v, o, lse, bias = ctx.saved_tensors
    dq, dk, dv, dbias = attn_bwd(do, q, k, v, o, lse, bias, ctx.causal, ctx.sm_scale, ctx.need_dbias)
    return dq, dk, dv, (dbias if ctx.need_dbias else None), None, None


attn_fwd.register_autograd(_backward, setup_context=_setup_context)


def flash_attention_op(q, k, v, bias=None, causal=False, sm_scale=None):
    """`flash_attention_fn` through the registered operators (graph-capture friendly)."""
    if bias is not None and bias.requires_grad and bias.dtype == torch.bool:
        raise TypeError("a bool mask cannot require grad")
    scale = float(q.shape[-1] ** -0.5 if sm_scale is None else sm_scale)
    out, _ = attn_fwd(q, k, v, bias, bool(causal), scale)
    return out


class FlashAttention(nn.Module):
    """Attention over (B, M, H, D) query / (B, N, H, D) key and value tensors with an optional
    (B, H, M, N) additive bias or bool mask.  No parameters; `causal` and `sm_scale` are fixed
    at construction (sm_scale None = 1/sqrt(D))."""

    def __init__(self, causal: bool = False, sm_scale: Optional[float] = None):
        super().__init__()
        self.causal = causal
        self.sm_scale = sm_scale

    def forward(self, q, k, v, bias=None):
        return flash_attention_op(q, k, v, bias, self.causal, self.sm_scale)

    def extra_repr(self) -> str:
        return f"causal={self.causal}, sm_scale={self.sm_scale}"
