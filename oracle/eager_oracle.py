"""CPU/GPU fp32 restatement of the reference's attention forward and backward.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module; it
is the checker that `tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` /
`--impl reference` legs of `bench.py` compare against or time.

What it restates (reference project file `flash_attention.py`, cited as FA:<line>):
  * scores  s = (q . k^T) * sm_scale                         FA:38-39, FA:149-150
  * bounds / causal / bool-mask handling: masked scores are removed from the
    softmax (the reference adds -1.0e6 in the log2 domain, FA:41-50, which equals
    -inf whenever a row keeps at least one key); causal is top-left aligned,
    key n visible to query m iff m >= n                      FA:45
  * float bias added to the scaled scores before the softmax FA:51-53
  * out = softmax(s) . v, log2-domain log-sum-exp saved      FA:55-70, FA:188-194
  * delta = rowsum(o * do), o being the saved 16-bit output  FA:197-233, FA:653
  * dv = p^T . do ; dp = do . v^T ; ds = p * (dp - delta)    FA:294-306
  * dbias = ds                                               FA:307-308
  * dk = sm_scale * ds^T . q                                 FA:310, FA:449
  * dq = sm_scale * ds . k                                   FA:520, FA:644

Parity pin: the reference ships no tests or golden vectors.  This oracle is pinned
against outputs of the reference's own Triton kernels executed on CPU by Triton's
interpreter (fp16 inputs; see tests/golden/make_golden.py and
tests/test_oracle_golden.py).  bf16 cannot run in that interpreter, so bf16 parity
rests on this fp32 restatement alone.

One deliberate divergence: a row whose keys are all masked yields an all-zero
output row and zero gradients here (the reference produces finite but meaningless
values, fp32 eager softmax produces NaN).
"""
from __future__ import annotations

import math

import torch

LOG2E = 1.4426950408889634


def _scores(q, k, bias, causal, sm_scale):
    """Masked fp32 scores of shape (B, H, M, N) and the boolean keep-mask."""
    qf = q.float().transpose(1, 2)  # (B, H, M, D)
    kf = k.float().transpose(1, 2)  # (B, H, N, D)
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sm_scale
    M, N = s.shape[-2:]
    keep = torch.ones(M, N, dtype=torch.bool, device=s.device)
    if causal:
        keep = torch.ones(M, N, dtype=torch.bool, device=s.device).tril()
    keep = keep.expand(s.shape)
    if bias is not None:
        if bias.dtype == torch.bool:
            keep = keep & bias
        else:
            s = s + bias.float()
    return s, keep


def attention_forward(q, k, v, bias=None, causal=False, sm_scale=None):
    """Returns (out fp32 (B,M,H,D), lse2 fp32 (B,H,M), p fp32 (B,H,M,N))."""
    D = q.shape[-1]
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    s, keep = _scores(q, k, bias, causal, sm_scale)
    s = s.masked_fill(~keep, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(s - m)
    l = e.sum(dim=-1, keepdim=True)
    p = torch.where(l > 0, e / l.clamp_min(1e-38), torch.zeros_like(e))
    lse2 = torch.where(l > 0, (m + torch.log(l.clamp_min(1e-38))) * LOG2E,
                       torch.full_like(l, float("inf"))).squeeze(-1)
    out = torch.matmul(p, v.float().transpose(1, 2)).transpose(1, 2)
    return out, lse2, p


def attention_backward(q, k, v, bias, causal, sm_scale, do, o_saved=None):
    """Closed-form fp32 backward; returns dict(out, dq, dk, dv, dbias, delta, lse2).

    `o_saved`: the 16-bit output tensor a forward pass actually saved.  The backward of
    the reference reads that tensor to form delta, so when the backward of another
    implementation is checked it should be given that implementation's own saved output
    (a one-unit-in-the-last-place difference in `o` moves delta by ~sqrt(D) units)."""
    D = q.shape[-1]
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    out, lse2, p = attention_forward(q, k, v, bias, causal, sm_scale)
    dof = do.float().transpose(1, 2)  # (B, H, M, D)
    vf = v.float().transpose(1, 2)
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2)
    # The reference saves `o` in q's dtype (FA:653) and its preprocess kernel reads that
    # tensor (FA:207-219), so delta is formed from the ROUNDED output.
    if o_saved is not None:
        o_saved = o_saved.float()
    else:
        o_saved = out.to(q.dtype).float() if q.dtype in (torch.float16, torch.bfloat16) else out
    delta = (o_saved.transpose(1, 2) * dof).sum(-1)  # (B, H, M)
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    ds = p * (dp - delta.unsqueeze(-1))
    dq = torch.matmul(ds, kf) * sm_scale
    dk = torch.matmul(ds.transpose(-1, -2), qf) * sm_scale
    res = {
        "out": out,
        "dq": dq.transpose(1, 2),
        "dk": dk.transpose(1, 2),
        "dv": dv.transpose(1, 2),
        "dbias": ds if (bias is not None and bias.dtype != torch.bool) else None,
        "delta": delta,
        "lse2": lse2,
    }
    return res


def attention_autograd(q, k, v, bias, causal, sm_scale, do):
    """Same quantities through torch.autograd on the plain eager expression
    softmax(q k^T * scale + bias) v in fp32 (the textbook reference for this
    operator).  Used to cross-check attention_backward."""
    D = q.shape[-1]
    sm_scale = D ** -0.5 if sm_scale is None else sm_scale
    qf = q.detach().float().requires_grad_()
    kf = k.detach().float().requires_grad_()
    vf = v.detach().float().requires_grad_()
    bf = None
    if bias is not None and bias.dtype != torch.bool:
        bf = bias.detach().float().requires_grad_()
    s = torch.matmul(qf.transpose(1, 2), kf.transpose(1, 2).transpose(-1, -2)) * sm_scale
    if bias is not None:
        s = s.masked_fill(~bias, float("-inf")) if bias.dtype == torch.bool else s + bf
    if causal:
        M, N = s.shape[-2:]
        s = s.masked_fill(~torch.ones(M, N, dtype=torch.bool, device=s.device).tril(), float("-inf"))
    out = torch.matmul(torch.softmax(s, dim=-1), vf.transpose(1, 2)).transpose(1, 2)
    out.backward(do.float())
    return {"out": out.detach(), "dq": qf.grad, "dk": kf.grad, "dv": vf.grad,
            "dbias": None if bf is None else bf.grad}


def flops(B, H, M, N, D, causal, which="fwd+bwd"):
    """Matmul FLOPs in the usual flash-attention convention (recompute not counted)."""
    c = 0.5 if causal else 1.0
    mult = {"fwd": 4, "bwd": 10, "fwd+bwd": 14}[which]
    return mult * B * H * M * N * D * c


def default_scale(D):
    return 1.0 / math.sqrt(D)
