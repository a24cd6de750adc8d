"""CPU tests of the oracle: it must reproduce the golden vectors produced by the
reference's own Triton kernels (tests/golden/make_golden.py), its two formulations
must agree, and it must obey the properties the domain offers."""
import pytest
import torch

from oracle import eager_oracle as oracle
from tests import _golden

# The reference computes in fp16 with fp32 accumulation; its outputs are fp16.
REF_TOL = 5e-3


@pytest.mark.parametrize("name", _golden.names())
def test_oracle_matches_reference_vectors(name):
    g = _golden.load(name)
    bias = g.get("bias")
    res = oracle.attention_backward(g["q"], g["k"], g["v"], bias, g["causal"], g["sm_scale"], g["do"])
    assert (res["out"] - g["out"].float()).abs().max().item() <= REF_TOL
    if g["packed"]:
        for i, n in enumerate(("dq", "dk", "dv")):
            assert (res[n] - g["dqkv"][:, :, i].float()).abs().max().item() <= REF_TOL, n
    else:
        for n in ("dq", "dk", "dv"):
            assert (res[n] - g[n].float()).abs().max().item() <= REF_TOL, n
        if "dbias" in g:
            assert (res["dbias"] - g["dbias"].float()).abs().max().item() <= REF_TOL


def test_reference_dbias_is_zero_above_the_diagonal():
    g = _golden.load("causal_floatbias")
    assert torch.all(g["dbias"][0, 0].triu(1) == 0)
    res = oracle.attention_backward(g["q"], g["k"], g["v"], g["bias"], True, None, g["do"])
    assert torch.all(res["dbias"][0, 0].triu(1) == 0)


@pytest.mark.parametrize("bias_kind", [None, "float", "bool"])
@pytest.mark.parametrize("causal", [False, True])
def test_closed_form_backward_equals_autograd(bias_kind, causal):
    g = torch.Generator().manual_seed(7)
    B, M, N, H, D = 2, 40, 56, 3, 16
    q, k, v = (torch.randn(B, s, H, D, generator=g) for s in (M, N, N))
    do = torch.randn(B, M, H, D, generator=g)
    bias = None
    if bias_kind == "float":
        bias = torch.randn(B, H, M, N, generator=g)
    elif bias_kind == "bool":
        bias = torch.rand(B, H, M, N, generator=g) < 0.8
        bias[..., 0] = True  # every row keeps a key
    a = oracle.attention_backward(q, k, v, bias, causal, None, do)
    b = oracle.attention_autograd(q, k, v, bias, causal, None, do)
    for n in ("out", "dq", "dk", "dv"):
        assert (a[n] - b[n]).abs().max().item() < 1e-5, n
    if bias_kind == "float":
        assert (a["dbias"] - b["dbias"]).abs().max().item() < 1e-5


def test_lse_is_log2_domain_logsumexp():
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, 33, 2, 8, generator=g) for _ in range(3))
    _, lse2, p = oracle.attention_forward(q, k, v, None, False, 0.5)
    s = torch.einsum("bmhd,bnhd->bhmn", q, k) * 0.5
    assert (lse2 - torch.logsumexp(s, -1) * oracle.LOG2E).abs().max().item() < 1e-5
    assert (p.sum(-1) - 1).abs().max().item() < 1e-5


def test_fully_masked_row_gives_zero_output_and_zero_grads():
    g = torch.Generator().manual_seed(4)
    q, k, v = (torch.randn(1, 8, 1, 8, generator=g) for _ in range(3))
    do = torch.randn(1, 8, 1, 8, generator=g)
    mask = torch.ones(1, 1, 8, 8, dtype=torch.bool)
    mask[0, 0, 3] = False
    r = oracle.attention_backward(q, k, v, mask, False, None, do)
    assert torch.all(r["out"][0, 3] == 0) and torch.all(r["dq"][0, 3] == 0)
    assert all(torch.isfinite(t).all() for t in (r["out"], r["dq"], r["dk"], r["dv"]))


def test_linearity_in_v_and_do():
    """out is linear in v; dq, dk, dv, dbias are linear in do."""
    g = torch.Generator().manual_seed(5)
    q, k, v, v2 = (torch.randn(1, 24, 2, 8, generator=g) for _ in range(4))
    do, do2 = (torch.randn(1, 24, 2, 8, generator=g) for _ in range(2))
    bias = torch.randn(1, 2, 24, 24, generator=g)
    o1, _, _ = oracle.attention_forward(q, k, v, bias, True)
    o2, _, _ = oracle.attention_forward(q, k, v2, bias, True)
    o3, _, _ = oracle.attention_forward(q, k, 2 * v + v2, bias, True)
    assert (o3 - (2 * o1 + o2)).abs().max().item() < 1e-5
    a = oracle.attention_backward(q, k, v, bias, True, None, do)
    b = oracle.attention_backward(q, k, v, bias, True, None, do2)
    c = oracle.attention_backward(q, k, v, bias, True, None, do - 3 * do2)
    for n in ("dq", "dk", "dv", "dbias"):
        assert (c[n] - (a[n] - 3 * b[n])).abs().max().item() < 1e-4, n


def test_dbias_rows_sum_to_zero():
    """Each row of dS sums to zero (softmax Jacobian), masked entries are exactly zero."""
    g = torch.Generator().manual_seed(6)
    q, k, v, do = (torch.randn(2, 32, 2, 16, generator=g) for _ in range(4))
    bias = torch.randn(2, 2, 32, 32, generator=g)
    r = oracle.attention_backward(q, k, v, bias, True, None, do)
    assert r["dbias"].sum(-1).abs().max().item() < 1e-4


def test_flop_count_convention():
    assert oracle.flops(8, 16, 2048, 2048, 128, False, "fwd+bwd") == 14 * 8 * 16 * 2048 * 2048 * 128
    assert oracle.flops(1, 1, 128, 128, 64, True, "fwd") == 4 * 128 * 128 * 64 * 0.5
