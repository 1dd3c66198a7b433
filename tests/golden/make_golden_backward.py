"""Regenerates reference_backward_golden.npz: gradients computed BY THE REFERENCE'S OWN backward formulas.

Needs a checkout of yifu-ding/BGEMM-CUDA (first argument; the default is the REF path below). The reference's
tests/python/bgemm_linear.py is imported with a stub `lowbit_kernel` (never called): every `backward` there is
a static method made of plain torch ops on `ctx.saved_tensors` / `ctx.other`, so it runs on the CPU when handed
a stand-in ctx that holds what the matching `forward` would have saved:

  bgemm_linear.backward                 bgemm_linear.py:149-165   saved (half(input), half(weight))
  bgemm_linear_bireal.backward          bgemm_linear.py:186-219   same, activation gradient x (2 - 2|x|)
  nn_linear_elastic_signed.backward     bgemm_linear.py:277-346   saved ((x - mean)/sa, w - mean), other = grad_scale
  bgemm_attn_matmul.backward            bgemm_linear.py:64-86     saved (half(attn), half(value))
  calculate_gradient_signed             bgemm_linear.py:519-535
  BNNLinear (whole layer, torch autograd over BinActive)          bgemm_linear.py:599-645
  NNLinear_elastic_signed (whole layer, forward + backward)       bgemm_linear.py:569-595

bgemm_linear_elastic_signed.backward (bgemm_linear.py:382-457) cannot be run: it calls
calculate_gradient_signed with three arguments (:398-399) while the function takes four (:519), so it raises
TypeError as soon as a model with that layer is trained. Its parts are pinned separately instead: the two
sign-GEMMs are bgemm_linear.backward's, the scale gradients are calculate_gradient_signed(..., is_act=True)
(the only reading under which the three-argument call makes sense), and the sech^2 shaping with clip 4 is
recomputed in the test.

Upstream gradients are multiples of 1/8 in [-1, 1], so every sign-GEMM in these formulas is exact in fp16
whatever the summation order; only the shaping factors (exp, cosh) round differently between devices.

Run:  python tests/golden/make_golden_backward.py [reference_root]
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from make_golden import load_reference_layers  # noqa: E402


def eighths(gen, *shape):
    return torch.randint(-8, 9, shape, generator=gen).float() / 8


def spread(gen, *shape, scale=1.5):
    """Values on both sides of the clip points 1 and 4, none of them zero."""
    t = torch.randn(*shape, generator=gen) * scale
    return torch.where(t == 0, torch.full_like(t, 0.25), t)


def ctx_of(saved, other=None):
    c = types.SimpleNamespace(saved_tensors=tuple(saved))
    if other is not None:
        c.other = other
    return c


def main():
    ref = load_reference_layers()
    out = {}
    g = torch.Generator().manual_seed(3001)

    # straight-through and Bi-Real: 2-D and batched 3-D activations
    for tag, xs, M in (("lin2d", (32, 128), 48), ("lin3d", (4, 32, 128), 48)):
        x = spread(g, *xs, scale=0.8).half()
        w = spread(g, M, xs[-1], scale=0.8).half()
        go = eighths(g, *xs[:-1], M).half()
        out[f"{tag}_x"], out[f"{tag}_w"], out[f"{tag}_go"] = x.numpy(), w.numpy(), go.numpy()
        for name, fn in (("ste", ref.bgemm_linear), ("bireal", ref.bgemm_linear_bireal)):
            gx, gw, _ = fn.backward(ctx_of((x, w)), go)
            out[f"{tag}_{name}_gx"], out[f"{tag}_{name}_gw"] = gx.float().numpy(), gw.float().numpy()

    # elastic signed quantisers: saved tensors are fp32 ((x - mean)/sa and w - mean), the product is scaled by sa*sw
    for tag, xs, M in (("el2d", (32, 128), 40), ("el3d", (3, 32, 128), 40)):
        qx = spread(g, *xs, scale=2.5)
        qw = spread(g, M, xs[-1], scale=0.9)
        go = eighths(g, *xs[:-1], M)
        gs = 1.0 / float(np.sqrt(qx.numel()))
        out[f"{tag}_qx"], out[f"{tag}_qw"], out[f"{tag}_go"], out[f"{tag}_gs"] = qx.numpy(), qw.numpy(), go.numpy(), np.float64(gs)
        gx, gw, gsa, gsw, _ = ref.nn_linear_elastic_signed.backward(ctx_of((qx, qw), gs), go)
        out[f"{tag}_nn_gx"], out[f"{tag}_nn_gw"] = gx.numpy(), gw.numpy()
        out[f"{tag}_nn_gsa"], out[f"{tag}_nn_gsw"] = gsa.numpy(), gsw.numpy()
        try:
            ref.bgemm_linear_elastic_signed.backward(ctx_of((qx, qw), gs), go)
            raise SystemExit("the reference's bgemm_linear_elastic_signed.backward ran: regenerate with it included")
        except TypeError:
            pass

    # scale-gradient helper on its own, both branches
    qx = spread(g, 16, 64, scale=1.2)
    gr = eighths(g, 16, 64)
    for is_act in (True, False):
        gx, gs_ = ref.calculate_gradient_signed(qx, gr, 0.125, is_act)
        out[f"cgs_{int(is_act)}_gx"], out[f"cgs_{int(is_act)}_gs"] = gx.numpy(), gs_.numpy()
    out["cgs_qx"], out["cgs_grad"] = qx.numpy(), gr.numpy()

    # attention product: attn [Sq, Sk] read as a {0,1} mask, value [Sk, d] as {-1,+1}
    attn = spread(g, 64, 128, scale=1.0).half()
    val = spread(g, 128, 32, scale=1.0).half()
    go = eighths(g, 64, 32).half()
    g1, g2, _ = ref.bgemm_attn_matmul.backward(ctx_of((attn, val)), go)
    out["attn_a"], out["attn_v"], out["attn_go"] = attn.numpy(), val.numpy(), go.numpy()
    out["attn_g1"], out["attn_g2"] = g1.float().numpy(), g2.float().numpy()

    # whole layer through torch autograd: the reference's dense twin, forward + backward. No bias: the twin adds it
    # before the scales (inside F.linear) and the kernel layers after them, so only the bias-free layers are twins.
    torch.manual_seed(3002)
    layer = ref.BNNLinear(128, 64, False)
    x = torch.randn(32, 128, requires_grad=True)
    y = layer(x)
    go = eighths(g, 32, 64)
    y.backward(go)
    out["bnn_x"], out["bnn_w"] = x.detach().numpy(), layer.weight.detach().numpy()
    out["bnn_go"], out["bnn_y"] = go.numpy(), y.detach().numpy()
    out["bnn_gx"], out["bnn_gw"] = x.grad.numpy(), layer.weight.grad.numpy()
    out["bnn_gsw"], out["bnn_gsa"] = layer.sw.grad.numpy(), np.float32(layer.sa.grad.item())

    # whole layer, binary/ternary weight x ternary activation: the reference runs it in dense torch, so its own
    # forward and backward can be taken end to end (two steps, so that the lazily created scales are exercised twice)
    torch.manual_seed(3003)
    layer = ref.NNLinear_elastic_signed(256, 48, True)
    x = torch.randn(64, 256, requires_grad=True)
    y = layer(x)
    go = eighths(g, 64, 48)
    y.backward(go)
    out["nnel_x"], out["nnel_w"], out["nnel_bias"] = x.detach().numpy(), layer.weight.detach().numpy(), layer.bias.detach().numpy()
    out["nnel_go"], out["nnel_y"] = go.numpy(), y.detach().numpy()
    out["nnel_gx"], out["nnel_gw"], out["nnel_gbias"] = x.grad.numpy(), layer.weight.grad.numpy(), layer.bias.grad.numpy()
    out["nnel_gsw"], out["nnel_gsa"] = layer.sw.grad.numpy(), layer.sa.grad.numpy()

    np.savez_compressed(HERE / "reference_backward_golden.npz", **out)
    print("wrote", HERE / "reference_backward_golden.npz", {k: getattr(v, "shape", ()) for k, v in out.items()})


if __name__ == "__main__":
    main()
