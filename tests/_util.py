"""Shared helpers of the GPU parity tests: seeded inputs, oracle comparison.

Acceptance rule, per output tensor (`accept`):
  1. raw max-abs error <= TOL[dtype] (2e-2 bf16, 5e-3 fp16 against the fp32 oracle): pass.
  2. otherwise every element over TOL must be explained by the 16-bit rounding of a LARGE
     value: |err| <= TOL + ULP[dtype] * |ref|.  Half a bf16 unit in the last place of a value
     of magnitude 4..8 is already 1.6e-2, so no implementation that returns 16-bit tensors can
     meet a purely absolute 2e-2 there.  The number of such elements, the smallest |ref| among
     them and the raw maximum are printed, never hidden.
The oracle's backward is fed ITS OWN forward output rounded to the input dtype (what a user
of the reference would get); the variant fed the device's saved output is reported beside it.
"""
import torch

from oracle import eager_oracle as oracle

TOL = {torch.bfloat16: 2e-2, torch.float16: 5e-3}
# two units in the last place of the 16-bit dtype, relative to the value: one for rounding the
# result itself, one for the 16-bit rounding of P, dS and the saved output that feed the
# products (the reference rounds at the same points: flash_attention.py lines 66, 299, 309, 517)
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


def account(t, r, dtype):
    """Error account of one tensor against its fp32 reference: raw max-abs, number of elements
    over the absolute tolerance, the smallest |ref| among those, and the worst excess over
    (tolerance + output rounding)."""
    r = r.float()
    assert torch.isfinite(t.float()).all(), "non-finite values"
    d = (t.float() - r).abs()
    tol = TOL[dtype]
    over = d > tol
    n_over = int(over.sum().item())
    return {
        "raw": d.max().item(),
        "n_over": n_over,
        "min_ref_over": r.abs()[over].min().item() if n_over else None,
        "excess": (d - ULP[dtype] * r.abs()).max().item(),
    }


def errors(ours, ref, dtype=None):
    """Per tensor: (raw max-abs error, max-abs error in excess of the output rounding)."""
    out = {}
    for name, t in ours.items():
        a = account(t, ref[name], dtype if dtype is not None else t.dtype)
        out[name] = (a["raw"], a["excess"])
    return out


def accept(name, a, dtype, tol_mult=1.0, label=""):
    """Applies the acceptance rule of the module docstring to one account."""
    tol = TOL[dtype] * tol_mult
    if a["raw"] <= tol:
        return
    assert a["excess"] <= tol, (
        f"{label}{name}: max-abs {a['raw']:.3e} > {tol:.1e} and not explained by 16-bit rounding "
        f"(excess {a['excess']:.3e}; {a['n_over']} elements over, smallest |ref| {a['min_ref_over']})")
    print(f"  note {label}{name}: raw max-abs {a['raw']:.3e} exceeds {tol:.1e} on {a['n_over']} "
          f"elements, all with |ref| >= {a['min_ref_over']:.2f} (16-bit rounding of large values)",
          flush=True)


def compare(ours, q, k, v, bias, causal, sm_scale, do, dtype, tol_mult=1.0, label="", verbose=True):
    """Checks `ours` against the oracle (backward fed the oracle's own rounded output) and
    reports the variant fed the device's saved output beside it.  Returns the accounts."""
    ref = oracle.attention_backward(q, k, v, bias, causal, sm_scale, do)
    ref_saved = oracle.attention_backward(q, k, v, bias, causal, sm_scale, do, o_saved=ours["out"])
    acc = {n: account(t, ref[n], dtype) for n, t in ours.items()}
    acc_saved = {n: account(t, ref_saved[n], dtype) for n, t in ours.items()}
    if verbose:
        print(label + " ".join(f"{n}={a['raw']:.2e}(saved-o {acc_saved[n]['raw']:.2e})" for n, a in acc.items()),
              flush=True)
    for n, a in acc.items():
        accept(n, a, dtype, tol_mult, label)
    return acc


def check_case(B, M, N, H, D, dtype, bias_kind, causal, seed=0, sm_scale=None, bias_scale=1.0,
               tol_mult=1.0, trainable_bias=True, verbose=True):
    q, k, v, bias, do = make_inputs(B, M, N, H, D, dtype, bias_kind, seed, bias_scale=bias_scale)
    ours = run_ours(q, k, v, bias, causal, sm_scale, do, trainable_bias)
    label = f"B{B} M{M} N{N} H{H} D{D} {dtype} bias={bias_kind} causal={causal}: "
    return compare(ours, q, k, v, bias, causal, sm_scale, do, dtype, tol_mult, label, verbose)
