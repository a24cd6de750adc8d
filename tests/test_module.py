"""nn.Module wrapper and torch.library operators around the attention launchers."""
import pytest
import torch

import triton_flashattn_b200 as fa


def test_operators_are_registered_with_shape_only_implementations():
    from torch._subclasses.fake_tensor import FakeTensorMode

    ops = torch.ops.triton_flashattn_b200
    assert hasattr(ops, "attn_fwd") and hasattr(ops, "attn_bwd")
    with FakeTensorMode():
        q = torch.empty(2, 100, 3, 64, dtype=torch.bfloat16, device="cuda")
        k = torch.empty(2, 70, 3, 64, dtype=torch.bfloat16, device="cuda")
        v = torch.empty_like(k)
        bias = torch.empty(2, 3, 100, 70, dtype=torch.bfloat16, device="cuda")
        o, lse = ops.attn_fwd(q, k, v, bias, False, 0.125)
        assert o.shape == q.shape and o.dtype == q.dtype
        assert lse.shape == (2, 3, 100) and lse.dtype == torch.float32
        dq, dk, dv, dbias = ops.attn_bwd(o, q, k, v, o, lse, bias, False, 0.125, True)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == v.shape
        assert dbias.shape == bias.shape and dbias.is_contiguous()  # dense, as the reference returns it
        assert ops.attn_bwd(o, q, k, v, o, lse, None, True, 0.125, False)[3].numel() == 0


def test_module_has_no_parameters_and_no_cpu_path():
    m = fa.FlashAttention(causal=True, sm_scale=0.5)
    assert "causal=True" in repr(m) and not list(m.parameters())
    q = torch.zeros(1, 4, 1, 16, dtype=torch.float16)
    with pytest.raises((NotImplementedError, RuntimeError, ValueError)):
        m(q, q, q)  # CPU tensors: the operators exist for CUDA only, nothing falls back


@pytest.mark.gpu
@pytest.mark.parametrize("bias_kind,causal", [("float", False), ("bool", True), (None, True)])
def test_operator_path_equals_autograd_function_bitwise(bias_kind, causal, device_ok):
    from tests._util import make_inputs

    q, k, v, bias, do = make_inputs(2, 200, 136, 2, 64, torch.bfloat16, bias_kind, 31)
    res = []
    for fn in (fa.flash_attention_fn, fa.FlashAttention(causal=causal)):
        qs, ks, vs = (t.detach().clone().requires_grad_() for t in (q, k, v))
        b = bias
        if bias_kind == "float":
            b = bias.detach().clone().requires_grad_()
        out = fn(qs, ks, vs, b, causal) if fn is fa.flash_attention_fn else fn(qs, ks, vs, b)
        out.backward(do)
        res.append((out, qs.grad, ks.grad, vs.grad, b.grad if bias_kind == "float" else None))
    for a, c in zip(*res):
        if a is not None:
            assert torch.equal(a, c)


@pytest.mark.gpu
def test_operator_is_captured_as_one_graph_node(device_ok):
    from tests._util import make_inputs

    q, k, v, bias, do = make_inputs(1, 128, 128, 2, 64, torch.float16, "float", 32)
    q.requires_grad_()
    seen = []

    def backend(gm, example_inputs):
        seen.append([n.target for n in gm.graph.nodes if n.op == "call_function"])
        return gm.forward

    fn = torch.compile(lambda a, b, c, d: fa.flash_attention_op(a, b, c, d, True), backend=backend,
                       fullgraph=True)
    out = fn(q, k, v, bias)
    ref = fa.flash_attention_fn(q, k, v, bias, True)
    assert torch.equal(out, ref)
    assert any(torch.ops.triton_flashattn_b200.attn_fwd.default in g for g in seen)
