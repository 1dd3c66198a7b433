"""Backward formulas of the layer mirror against gradients produced by the reference's own `backward` methods
(tests/golden/reference_backward_golden.npz, written by tests/golden/make_golden_backward.py).

The backward passes are dense torch ops (no CUDA kernel of this library is involved), so they are checked on
the CPU by handing each static `backward` a stand-in ctx with the tensors its `forward` saves. The sign-GEMMs
must agree bit for bit (the upstream gradients are multiples of 1/8, so every sum is exact); the shaping factors
are the same torch ops on the same device, so they agree exactly too.
"""
import types
from pathlib import Path

import numpy as np
import pytest
import torch

GOLD = np.load(Path(__file__).parent / "golden" / "reference_backward_golden.npz")


@pytest.fixture(scope="module")
def L():
    import bgemm_linear

    return bgemm_linear


def T(name):
    return torch.from_numpy(GOLD[name])


def ctx_of(saved, other=None):
    c = types.SimpleNamespace(saved_tensors=tuple(saved))
    if other is not None:
        c.other = other
    return c


@pytest.mark.parametrize("tag", ["lin2d", "lin3d"])
@pytest.mark.parametrize("kind", ["ste", "bireal"])
def test_straight_through_and_bireal_backward(L, tag, kind):
    fn = L.bgemm_linear if kind == "ste" else L.bgemm_linear_bireal
    gx, gw, none = fn.backward(ctx_of((T(f"{tag}_x"), T(f"{tag}_w"))), T(f"{tag}_go"))
    assert none is None and gx.dtype == torch.half and gw.dtype == torch.half
    assert torch.equal(gx.float(), T(f"{tag}_{kind}_gx"))
    assert torch.equal(gw.float(), T(f"{tag}_{kind}_gw"))
    if tag == "lin3d":
        assert gw.shape == (4, 48, 128)      # one slice per batch entry, as in the reference; autograd sums them into [M, K]


@pytest.mark.parametrize("tag", ["el2d", "el3d"])
def test_ternary_elastic_backward(L, tag):
    ctx = ctx_of((T(f"{tag}_qx"), T(f"{tag}_qw")), float(GOLD[f"{tag}_gs"]))
    gx, gw, gsa, gsw, none = L.nn_linear_elastic_signed.backward(ctx, T(f"{tag}_go"))
    assert none is None
    for got, name in ((gx, "gx"), (gw, "gw"), (gsa, "gsa"), (gsw, "gsw")):
        want = T(f"{tag}_nn_{name}")
        assert got.shape == want.shape, name
        assert torch.equal(got, want), name


@pytest.mark.parametrize("tag", ["el2d", "el3d"])
def test_binary_elastic_backward_from_its_pinned_parts(L, tag):
    """The reference's own method raises TypeError (three-argument call of a four-argument helper), so its parts
    are checked: sign-GEMMs as in bgemm_linear.backward, scale gradients by the helper with is_act=True, and
    2/cosh^2 shaping clipped at 4 (bgemm_linear.py:389-399, :441-451)."""
    qx, qw, go, gs = T(f"{tag}_qx"), T(f"{tag}_qw"), T(f"{tag}_go"), float(GOLD[f"{tag}_gs"])
    gx, gw, gsa, gsw, none = L.bgemm_linear_elastic_signed.backward(ctx_of((qx, qw), gs), go)
    ste_gx, ste_gw, _ = L.bgemm_linear.backward(ctx_of((qx, qw)), go)
    _, want_gsa = L.calculate_gradient_signed(qx, ste_gx, gs, True)
    _, want_gsw = L.calculate_gradient_signed(qw, ste_gw, gs, True)
    sech2 = lambda t: 2 / torch.cosh(t.abs().clamp(max=4)) ** 2      # noqa: E731
    assert torch.equal(gsa, want_gsa) and torch.equal(gsw, want_gsw)
    assert torch.allclose(gx, ste_gx * sech2(qx), rtol=1e-6, atol=0)
    assert torch.allclose(gw, ste_gw * sech2(qw), rtol=1e-6, atol=0)


@pytest.mark.parametrize("is_act", [True, False])
def test_scale_gradient_helper(L, is_act):
    gx, gs = L.calculate_gradient_signed(T("cgs_qx"), T("cgs_grad"), 0.125, is_act)
    assert torch.equal(gx, T(f"cgs_{int(is_act)}_gx"))
    assert torch.equal(gs, T(f"cgs_{int(is_act)}_gs"))


def test_attention_product_backward(L):
    g1, g2, none = L.bgemm_attn_matmul.backward(ctx_of((T("attn_a"), T("attn_v"))), T("attn_go"))
    assert none is None
    assert torch.equal(g1.float(), T("attn_g1"))
    assert torch.equal(g2.float(), T("attn_g2"))


def test_matmul_backward_is_the_gradient_of_a_times_b(L):
    """bgemm_matmul's forward is sign(A) @ sign(B). The reference's backward (bgemm_linear.py:28-42) multiplies the
    upstream gradient by B untransposed, which only type-checks for a square B and is then the gradient of A @ B.T;
    the mirror returns the straight-through gradient of the product it actually computes."""
    g = torch.Generator().manual_seed(7)
    a = torch.randn(24, 64, generator=g).half()
    b = torch.randn(64, 40, generator=g).half()
    go = (torch.randint(-8, 9, (24, 40), generator=g).float() / 8).half()
    ga, gb, none = L.bgemm_matmul.backward(ctx_of((a, b)), go)
    sa = a.sign().float().requires_grad_(True)
    sb = b.sign().float().requires_grad_(True)
    (sa @ sb).backward(go.float())
    assert none is None
    assert torch.equal(ga.float(), sa.grad) and torch.equal(gb.float(), sb.grad)


def test_dense_twin_layer_forward_and_backward(L):
    """BNNLinear is pure torch in the mirror as in the reference: whole-layer forward and autograd backward."""
    layer = L.BNNLinear(128, 64, False)
    with torch.no_grad():
        layer.weight.copy_(T("bnn_w"))
    x = T("bnn_x").clone().requires_grad_(True)
    y = layer(x)
    y.backward(T("bnn_go"))
    assert torch.allclose(y.detach(), T("bnn_y"), rtol=1e-6, atol=1e-7)
    for got, name in ((x.grad, "gx"), (layer.weight.grad, "gw"), (layer.sw.grad, "gsw")):
        assert torch.allclose(got, T(f"bnn_{name}"), rtol=1e-5, atol=1e-7), name
    assert abs(float(layer.sa.grad) - float(GOLD["bnn_gsa"])) <= 1e-5 * abs(float(GOLD["bnn_gsa"]))
