"""Regenerates the golden fixtures in this directory FROM THE REFERENCE ITSELF.

Needs a checkout of yifu-ding/BGEMM-CUDA (first argument; the default is the REF path below) and, for the prepack vectors,
oracle/_ref/libref_prepack.so (built by `make -C oracle ref` from the reference's own header).
It imports the reference's tests/python/bgemm_linear.py with a stub `lowbit_kernel` module -- the
classes used here are the reference's pure-torch CPU paths and never call the extension:

  BNNLinear.forward                 bgemm_linear.py:633-645   dense twin of the binary linear layers
  NNLinear_elastic_signed.forward   bgemm_linear.py:585-595   binary/ternary weight x ternary activation
  mm.forward                        bgemm_linear.py:107-108   {0,1} x {-1,+1} attention product
  BinActive.forward, ternary        bgemm_linear.py:604-608, :222-241

Run:  python tests/golden/make_golden.py [reference_root]
"""
import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
# the reference checkout: argv[1], else $REFERENCE_ROOT, else a directory named `reference` beside this repository
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT", Path(__file__).resolve().parents[3] / "reference"))


def load_reference_layers():
    stub = types.ModuleType("lowbit_kernel")

    def _no_gpu(*a, **k):
        raise RuntimeError("the stub lowbit_kernel must not be called while generating golden vectors")

    stub.bgemm_linear_forward_cuda = _no_gpu
    sys.modules["lowbit_kernel"] = stub
    spec = importlib.util.spec_from_file_location("ref_bgemm_linear", REF / "tests" / "python" / "bgemm_linear.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    del sys.modules["lowbit_kernel"]
    return mod


def main():
    ref = load_reference_layers()
    out = {}

    # 1. BNNLinear: random float inputs, with and without bias
    torch.manual_seed(2001)
    for tag, (N, K, M, bias) in {"bnn_a": (32, 128, 32, False), "bnn_b": (48, 384, 96, True), "bnn_c": (7, 200, 10, False)}.items():
        layer = ref.BNNLinear(K, M, bias)
        x = torch.randn(N, K)
        with torch.no_grad():
            y = layer(x)
        out[f"{tag}_x"] = x.numpy()
        out[f"{tag}_w"] = layer.weight.detach().numpy()
        if bias:
            out[f"{tag}_bias"] = layer.bias.detach().numpy()
        out[f"{tag}_y"] = y.numpy()
        out[f"{tag}_sw"] = layer.sw.detach().numpy()
        out[f"{tag}_sa"] = np.float32(layer.sa.item())

    # 2. NNLinear_elastic_signed: (a) random floats, (b) integer-valued tensors with exactly zero mean,
    #    so that zeros survive the mean-centring and the ternary path is exercised on both operands
    torch.manual_seed(2002)
    layer = ref.NNLinear_elastic_signed(256, 64, True)
    x = torch.randn(32, 256)
    with torch.no_grad():
        y = layer(x)
    out["bwta_a_x"], out["bwta_a_w"], out["bwta_a_bias"], out["bwta_a_y"] = x.numpy(), layer.weight.detach().numpy(), layer.bias.detach().numpy(), y.numpy()

    g = torch.Generator().manual_seed(2003)
    N, K, M = 64, 512, 72      # the reference layer asserts N % 32 == 0

    def balanced_ternary(rows, cols):
        # each row: equal numbers of +1 and -1, the rest 0 -> global mean exactly 0
        t = torch.zeros(rows, cols)
        for r in range(rows):
            perm = torch.randperm(cols, generator=g)
            n = int(torch.randint(cols // 8, cols // 2 - 1, (1,), generator=g))
            t[r, perm[:n]] = 1.0
            t[r, perm[n:2 * n]] = -1.0
        return t

    layer = ref.NNLinear_elastic_signed(K, M, False)
    with torch.no_grad():
        layer.weight.copy_(balanced_ternary(M, K))
    x = balanced_ternary(N, K)
    with torch.no_grad():
        y = layer(x)
    assert float(x.mean()) == 0.0 and float(layer.weight.mean()) == 0.0
    out["bwta_b_x"], out["bwta_b_w"], out["bwta_b_y"] = x.numpy(), layer.weight.detach().numpy(), y.numpy()

    # 3. attention product through the reference's mm Function: {0,1} mask @ {-1,+1} values
    g = torch.Generator().manual_seed(2004)
    attn01 = torch.bernoulli(torch.full((96, 256), 0.5), generator=g)
    v = ref.BinActive.apply(torch.randn(256, 64, generator=g))
    out["attn_mask"], out["attn_v"] = attn01.numpy(), v.numpy()
    out["attn_y"] = ref.mm.apply(attn01, v).numpy()

    # 4. BinActive / ternary on edge values
    edge = torch.tensor([0.0, -0.0, 1e-4, -1e-4, 3.0, -2.5, float("inf"), float("-inf")])   # all exact-sign-preserving in fp16
    out["edge_in"] = edge.numpy()
    out["edge_binactive"] = ref.BinActive.apply(edge).numpy()
    out["edge_ternary"] = ref.ternary(edge, True).numpy()

    # 5. prepack words from the reference's own bin_matrix_prepacking_to_uint32
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle as O

    g = torch.Generator().manual_seed(2005)
    w = torch.randn(64, 256, generator=g).to(torch.float16)
    w[0, 0], w[0, 1], w[5, 31], w[5, 32] = 0.0, -0.0, -0.0, 0.0
    out["prepack_w_f16bits"] = w.numpy().view(np.uint16)
    out["prepack_words"] = O.ref_pack_rowmajor_msb(w)

    np.savez_compressed(HERE / "reference_golden.npz", **out)
    print("wrote", HERE / "reference_golden.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
