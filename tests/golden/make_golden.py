"""Generates the golden fixtures in this directory from the REFERENCE implementation.

Run where the reference project is checked out (it is not needed to run the tests):

    REFERENCE_DIR=/path/to/triton_flashattn python tests/golden/make_golden.py

The reference's own Triton kernels are executed on CPU tensors by Triton's
interpreter (TRITON_INTERPRET=1).  `triton.autotune` needs a GPU to benchmark, so
the three autotuned kernels are called with their smallest listed configuration
(32x32 tiles) instead of being tuned; nothing else of the reference is altered.
The interpreter cannot run bf16, so every fixture is fp16.

Each fixture is an .npz holding the seeded inputs and the reference's outputs
(out, dq, dk, dv and, for a trainable bias, dbias; packed cases hold dqkv).
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

REF = os.environ["REFERENCE_DIR"]  # checkout of sukjunhwang/triton_flashattn
sys.path.insert(0, REF)
import flash_attention as ref  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


class _FixedConfig:
    """Stands in for a triton Autotuner: always launches configs[idx]."""

    def __init__(self, tuner, idx):
        self.fn, self.cfg = tuner.fn, tuner.configs[idx]

    def __getitem__(self, grid):
        def run(*a, **kw):
            kw = dict(kw)
            kw.update(self.cfg.kwargs)
            g = grid(kw) if callable(grid) else grid
            return self.fn[g](*a, **kw)

        return run


for _name in ("_attn_fwd", "_attn_bwd_dkdv", "_attn_bwd_dq"):
    setattr(ref, _name, _FixedConfig(getattr(ref, _name), 2))

CASES = [
    # name, B, M, N, H, D, bias kind, causal, sm_scale, seed, packed
    ("config1_fp16_floatbias", 2, 128, 128, 4, 64, "float", False, 1 / 8, 0, False),
    ("causal_floatbias", 1, 64, 64, 2, 32, "float", True, None, 1, False),
    ("causal_boolmask", 1, 64, 64, 2, 32, "bool", True, None, 2, False),
    ("ragged_floatbias", 1, 50, 70, 2, 32, "float", False, None, 3, False),
    ("causal_nobias_d64", 1, 96, 96, 2, 64, None, True, None, 4, False),
    ("packed_boolmask_causal", 1, 64, 64, 2, 32, "bool", True, None, 5, True),
    ("nobias_d16_cross", 1, 48, 80, 1, 16, None, False, 0.3, 6, False),
]


def make_case(name, B, M, N, H, D, bias_kind, causal, sm_scale, seed, packed):
    g = torch.Generator().manual_seed(seed)
    dt = torch.float16
    if packed:
        qkv = torch.randn(B, M, 3, H, D, generator=g).to(dt)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    else:
        q = torch.randn(B, M, H, D, generator=g).to(dt)
        k = torch.randn(B, N, H, D, generator=g).to(dt)
        v = torch.randn(B, N, H, D, generator=g).to(dt)
    do = torch.randn(B, M, H, D, generator=g).to(dt)
    bias = None
    if bias_kind == "float":
        bias = torch.randn(B, H, M, N, generator=g).to(dt)
    elif bias_kind == "bool":
        bias = torch.rand(B, H, M, N, generator=g) < 0.9
        i = torch.arange(min(M, N))
        bias[:, :, i, i] = True
    out = {}
    if packed:
        x = qkv.clone().requires_grad_()
        o = ref.flash_attention_qkvpacked_fn(x, bias, causal, sm_scale)
        o.backward(do)
        out.update(qkv=qkv.numpy(), dqkv=x.grad.numpy())
    else:
        qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
        bb = bias.clone().requires_grad_() if bias_kind == "float" else bias
        o = ref.flash_attention_fn(qq, kk, vv, bb, causal, sm_scale)
        o.backward(do)
        out.update(q=q.numpy(), k=k.numpy(), v=v.numpy(), dq=qq.grad.numpy(), dk=kk.grad.numpy(),
                   dv=vv.grad.numpy())
        if bias_kind == "float":
            out["dbias"] = bb.grad.numpy()
    out.update(do=do.numpy(), out=o.detach().numpy(), causal=np.array(causal),
               sm_scale=np.array(np.nan if sm_scale is None else sm_scale, dtype=np.float64))
    if bias is not None:
        out["bias"] = bias.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k_: getattr(v_, "shape", None) for k_, v_ in out.items()})


if __name__ == "__main__":
    import warnings

    warnings.filterwarnings("ignore")
    for c in CASES:
        make_case(*c)
