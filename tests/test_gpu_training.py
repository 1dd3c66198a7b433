"""Training-side parity on the GPU: whole layers (kernel forward + torch backward) against gradients taken from the
reference's own layers (tests/golden/reference_backward_golden.npz), and the demo MLP learning a synthetic task."""
import types
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "reference_backward_golden.npz")


@pytest.fixture(scope="module")
def L():
    import bgemm_linear

    return bgemm_linear


def T(name):
    return torch.from_numpy(GOLD[name])


def close(got, want, rel):
    """|got - want| within `rel` of the largest magnitude in `want` (gradients span orders of magnitude)."""
    got, want = got.detach().float().cpu(), want.float()
    assert got.shape == want.shape, (got.shape, want.shape)
    return float((got - want).abs().max()) <= rel * max(float(want.abs().max()), 1e-12)


def _loaded(layer, prefix):
    with torch.no_grad():
        layer.weight.copy_(T(f"{prefix}_w"))
        if layer.bias is not None:
            layer.bias.copy_(T(f"{prefix}_bias"))
    return layer.cuda()


def test_ternary_elastic_layer_forward_and_backward_match_the_reference_layer(L):
    """NNLinear_elastic_signed is dense torch in the reference, so its forward AND backward are golden end to end;
    here the forward is two 1-bit GEMMs on the GPU. The output is `half_product * sa * sw`: torch rounds the 0-dim
    fp32 scale to half before a CPU multiply and keeps it in fp32 inside a CUDA kernel, hence 1e-3 on y. The gradients
    are fp32 GEMMs and elementwise factors of the saved tensors: 1e-4."""
    layer = _loaded(L.NNLinear_elastic_signed(256, 48, True), "nnel")
    x = T("nnel_x").cuda().requires_grad_(True)
    y = layer(x)
    y.backward(T("nnel_go").cuda())
    assert close(y, T("nnel_y"), 1e-3)
    for got, name in ((x.grad, "gx"), (layer.weight.grad, "gw"), (layer.bias.grad, "gbias"), (layer.sw.grad, "gsw"), (layer.sa.grad, "gsa")):
        assert close(got, T(f"nnel_{name}"), 1e-4), name


@pytest.mark.parametrize("cls", ["BGEMMLinear", "BGEMMLinear_bireal"])
def test_binary_layers_backward_match_the_dense_twin(L, cls):
    """The reference's BNNLinear is the dense twin of both layers: same forward, identity (straight-through) gradient
    through the sign. BGEMMLinear's backward is that gradient computed in fp16 (its kernel output is fp16, so autograd
    hands it an fp16 upstream gradient, as in the reference): 2e-3 of the largest entry. Bi-Real multiplies the
    activation gradient by 2 - 2 min(|x - zpa|, 1) (bgemm_linear.py:205-213). Bias-free: the twin adds its bias before
    the scales, the kernel layers after them."""
    layer = _loaded(getattr(L, cls)(128, 64, False), "bnn")
    x = T("bnn_x").cuda().requires_grad_(True)
    y = layer(x)
    y.backward(T("bnn_go").cuda())
    assert close(y, T("bnn_y"), 1e-3)
    want_gx = T("bnn_gx")
    if cls == "BGEMMLinear_bireal":
        centred = (T("bnn_x") - T("bnn_x").mean()).half().float()
        want_gx = want_gx * (2 - 2 * centred.abs().clamp(max=1))
    assert close(x.grad, want_gx, 2e-3)
    assert close(layer.weight.grad, T("bnn_gw"), 2e-3)
    assert close(layer.sw.grad, T("bnn_gsw"), 1e-3)
    assert close(layer.sa.grad, torch.tensor(float(GOLD["bnn_gsa"])), 1e-3)


@pytest.mark.parametrize("shape", [(64, 128), (2, 32, 128)])
def test_binary_elastic_layer_backward_equals_its_formula_on_the_cpu(L, shape):
    """BGEMMLinear_elastic_signed on the GPU, then the same backward formula (pinned part by part on the CPU against
    the reference) evaluated on the CPU from the tensors the forward must have saved."""
    g = torch.Generator().manual_seed(11)
    layer = L.BGEMMLinear_elastic_signed(shape[-1], 40, True)
    x = torch.randn(*shape, generator=g) * 1.5
    go = torch.randint(-8, 9, (*shape[:-1], 40), generator=g).float() / 8
    w = layer.weight.detach().clone()
    layer = layer.cuda()
    xin = x.cuda().requires_grad_(True)
    y = layer(xin)
    y.backward(go.cuda())
    sa, sw = layer.sa.detach().cpu(), layer.sw.detach().cpu()
    qx, qw = (x - x.mean().item()) / sa, w - w.mean().item()
    want_y = (qx.sign() @ qw.sign().T) * sa * sw + layer.bias.detach().cpu()
    assert close(y, want_y, 1e-3)      # half rounding of product * sa, as above
    ctx = types.SimpleNamespace(saved_tensors=(qx, qw), other=layer.grad_scale)
    gx, gw, gsa, gsw, _ = L.bgemm_linear_elastic_signed.backward(ctx, go)
    assert close(xin.grad, gx, 1e-4)
    assert close(layer.weight.grad, gw.sum(0) if gw.dim() == 3 else gw, 1e-4)
    assert close(layer.sa.grad, gsa.sum(), 1e-4)
    assert close(layer.sw.grad, gsw.reshape(-1, 40).sum(0), 1e-4)


@pytest.mark.parametrize("model", ["bgemm", "bgemm_bireal", "bgemm_elastic", "nn_elastic"])
def test_demo_mlp_learns_the_synthetic_task(model):
    """The reference's demo network (512-128-128-128-1) with each binary layer class: the loss falls and the
    held-out accuracy beats chance clearly. The data are a seeded synthetic stand-in for the table the reference
    trains on, which it does not ship."""
    import train_demo as D

    torch.manual_seed(0)
    dev = torch.device("cuda")
    net = D.MLP(Linear=D.LAYERS[model], bias=True, dropout=0.1).to(dev)
    train = torch.utils.data.DataLoader(D.synthetic_dataset(8192, 1), batch_size=256, shuffle=True, drop_last=True,
                                        generator=torch.Generator().manual_seed(5))
    test = torch.utils.data.DataLoader(D.synthetic_dataset(2048, 2), batch_size=256)
    crit = torch.nn.BCEWithLogitsLoss()
    opt = D.make_optimizer(net)
    first = D.train_epoch(net, train, opt, crit, dev)
    for _ in range(4):
        last = D.train_epoch(net, train, opt, crit, dev)
    assert all(np.isfinite(first)) and all(np.isfinite(last))
    assert np.mean(last) < 0.8 * np.mean(first[:8]), (np.mean(first[:8]), np.mean(last))
    assert D.accuracy(net, test, dev) > 0.75
