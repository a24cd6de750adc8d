"""Shared helpers of the GPU parity tests: seeded inputs, oracle comparison."""
import torch

from oracle import eager_oracle as oracle

# max-abs tolerance against the fp32 oracle, per input dtype ...
TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
# ... on top of two units in the last place of the 16-bit dtype relative to the
# value (2^-8 for bf16, 2^-11 for fp16 per unit): one for rounding the result
# itself to 16 bits, one for the 16-bit rounding of P, dS and the saved output that
# feed the products (the reference rounds at the same points: flash_attention.py
# lines 66, 299, 309, 517 and the 16-bit `o` it saves).  Without this term no
# implementation returning 16-bit tensors can meet an absolute bound once
# |value| exceeds ~4, as gradients of short causal rows do.
ULP = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}


def make_inputs(B, M, N, H, D, dtype, bias_kind, seed, device="cuda", bias_scale=1.0, p_keep=0.9):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, M, H, D, generator=g).to(dtype).to(device)
    k = torch.randn(B, N, H, D, generator=g).to(dtype).to(device)
    v = torch.randn(B, N, H, D, generator=g).to(dtype).to(device)
    do = torch.randn(B, M, H, D, generator=g).to(dtype).to(device)
    bias = None
    if bias_kind == "float":
        bias = (bias_scale * torch.randn(B, H, M, N, generator=g)).to(dtype).to(device)
    elif bias_kind == "bool":
        bias = torch.rand(B, H, M, N, generator=g) < p_keep
        i = torch.arange(min(M, N))
        bias[:, :, i, i] = True
        bias = bias.to(device)
    return q, k, v, bias, do


def run_ours(q, k, v, bias, causal, sm_scale, do, trainable_bias=True):
    from triton_flashattn_b200 import flash_attention_fn

    q = q.detach().clone().requires_grad_()
    k = k.detach().clone().requires_grad_()
    v = v.detach().clone().requires_grad_()
    b = bias
    if bias is not None and bias.dtype != torch.bool and trainable_bias:
        b = bias.detach().clone().requires_grad_()
    out = flash_attention_fn(q, k, v, b, causal, sm_scale)
    out.backward(do)
    res = {"out": out.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad}
    if b is not None and b.requires_grad:
        res["dbias"] = b.grad
    return res


def errors(ours, ref, dtype=None):
    """Per tensor: (max-abs error, max-abs error in excess of the output rounding)."""
    errs = {}
    for name, t in ours.items():
        r = ref[name].float()
        assert torch.isfinite(t.float()).all(), f"{name} has non-finite values"
        d = (t.float() - r).abs()
        ulp = ULP.get(dtype if dtype is not None else t.dtype, 0.0)
        errs[name] = (d.max().item(), (d - ulp * r.abs()).max().item())
    return errs


def check_case(B, M, N, H, D, dtype, bias_kind, causal, seed=0, sm_scale=None, bias_scale=1.0,
               tol_mult=1.0, trainable_bias=True, verbose=True):
    q, k, v, bias, do = make_inputs(B, M, N, H, D, dtype, bias_kind, seed, bias_scale=bias_scale)
    ours = run_ours(q, k, v, bias, causal, sm_scale, do, trainable_bias)
    ref = oracle.attention_backward(q, k, v, bias, causal, sm_scale, do, o_saved=ours["out"])
    errs = errors(ours, ref, dtype)
    tol = TOL[dtype] * tol_mult
    if verbose:
        print(f"B{B} M{M} N{N} H{H} D{D} {dtype} bias={bias_kind} causal={causal}: "
              + " ".join(f"{n}={e[0]:.2e}" for n, e in errs.items()), flush=True)
    for name, (e_abs, e_excess) in errs.items():
        assert e_excess <= tol, f"{name}: max-abs error {e_abs:.3e} (beyond output rounding {e_excess:.3e}) > {tol:.1e}"
    return errs
