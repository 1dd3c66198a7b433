"""GPU parity at the five benchmark configurations, each at its full stated shape, through the C ABI.

  C1  BGEMM   W[4096, 4096] x X[64, 4096], both {-1,+1}: int32 accumulators and fp16 output
  C2  BWTA    W[4096, 4096] x ternary X[128, 4096], per-channel fp16 scale: int32 and scaled fp16
  C3  A x V   32 x 12 heads, A[512, 512] in {0,1}, V[512, 64] in {-1,+1}: int32, one batched call
  C4  MLP     1024 -> 4096 -> 4096 -> 10 at batch 256 (the last layer has M = 10, a shape the reference
              refuses: lowbit_kernel/csrc/fp6_linear.cu:288-290): logits and the three accumulators
  C5  LLM projection W[28672, 8192] x ternary X[N, 8192], N in {1, 16, 128, 1024, 4096}: one call, and
              the row-sharded form (2, 4, 8 shards computed one after another on this GPU)

Integer results are compared bit for bit with the CPU oracle (dense fp32 matmul on mapped tensors, exact below
2**24); scaled fp16 outputs within 1e-3 relative, and for equality (same fp32 multiply and rounding).
"""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu

RTOL = 1e-3


@pytest.fixture(scope="module")
def B():
    import bgemm_b200

    return bgemm_b200


def _prepared(B, w, x, op):
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[op])
    return plane, acts, colsum


def test_config1_bgemm_4096x4096x64(B):
    cfg = O.config1()                                      # seed 1001
    w, x = cfg["w"], cfg["x"]
    M, K = w.shape
    acc = O.ref_acc(w, x, O.OP_XOR)
    plane, acts, colsum = _prepared(B, w, x, O.OP_XOR)
    for split_k in (0, 1, 4):
        assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_XOR, B.OUT_I32, split_k=split_k).cpu(), acc), split_k
    want16 = O.ref_out(acc, O.OUT_F16)
    assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_XOR, B.OUT_F16).cpu(), want16)
    # the literal drop-in call on unpacked fp16 operands
    assert torch.equal(B.linear_forward(w.cuda(), x.cuda(), B.OP_XOR, out_kind=B.OUT_F16).cpu(), want16)
    assert B.lib.bgemm_device_status(1) == 0


def test_config2_bwta_4096x4096x128_scaled(B):
    cfg = O.config2()                                      # seed 1002
    w, x, alpha = cfg["w"], cfg["x"], cfg["alpha"]
    M, K = w.shape
    acc = O.ref_acc(w, x, O.OP_BWTA)
    want = O.ref_out(acc, O.OUT_F16_SCALED, alpha)
    plane, acts, colsum = _prepared(B, w, x, O.OP_BWTA)
    for split_k in (0, 1, 8):
        assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, B.OUT_I32, split_k=split_k).cpu(), acc), split_k
        got = B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, B.OUT_F16_SCALED, alpha=alpha.cuda(), split_k=split_k).cpu()
        assert torch.allclose(got.float(), want.float(), rtol=RTOL, atol=0)
        assert torch.equal(got, want)
    assert B.lib.bgemm_device_status(1) == 0


def test_config3_attention_384_heads_one_call(B):
    cfg = O.config3()                                      # seed 1003: 384 x (A[512,512], V[512,64])
    a, v = cfg["attn"], cfg["v"]
    H, S, d = v.shape
    want = O.ref_attn_heads(a, v)
    plane, _, _ = B.pack_weights((2 * a - 1).cuda(), B.WBIT_NONNEGATIVE)       # "1" = sign bit clear, as the reference encodes it
    acts, colsum = B.prepare_acts(v.cuda(), B.ACT_SIGN, transpose=True)
    got = B.gemm(plane, S, S, acts, colsum, B.OP_ATTN, B.OUT_I32, B.LAYOUT_MN).cpu()
    assert got.shape == (H, S, d) and torch.equal(got, want)
    import lowbit_kernel

    got2 = lowbit_kernel.bgemm_attn_matmul_batched((2 * a - 1).cuda(), v.cuda(), True).cpu()
    assert torch.equal(got2, want)
    assert B.lib.bgemm_device_status(1) == 0


def test_config4_mlp_1024_4096_4096_10_batch256(B):
    import bgemm_linear as L

    cfg = O.config4()                                      # seed 1004
    ws, x = cfg["ws"], cfg["x"]
    want, accs = O.ref_mlp(ws, x)
    alphas = [torch.from_numpy(O.c_rowmeanabs_f16(w).copy()) for w in ws]
    # the three accumulators, layer by layer through the C ABI (inputs of a layer = the oracle's previous output)
    h = x
    for w, a, acc in zip(ws, alphas, accs):
        M, K = w.shape
        plane, acts, colsum = _prepared(B, w, h, O.OP_XOR)
        assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_XOR, B.OUT_I32).cpu(), acc), (M, K)
        h = O.ref_out(acc, O.OUT_F16_SCALED, a)
    # the layer stack: fused epilogues, plain chain, CUDA-graph replay; bit-exact with the oracle's scales
    for kwargs in ({}, {"fused": False}, {"graph": True}):
        mlp = L.BinaryMLP([w.cuda() for w in ws], **kwargs)
        for layer, a in zip(mlp.layers, alphas):
            layer.alpha.copy_(a.cuda())
        got = mlp(x.cuda()).cpu()
        assert got.shape == (256, 10) and got.dtype == torch.float16
        assert torch.allclose(got.float(), want.float(), rtol=RTOL, atol=0), kwargs
        assert torch.equal(got, want), kwargs
    # with the library's own per-row scales (a mean of fp16 magnitudes accumulated in another order): 1e-3
    got = L.BinaryMLP([w.cuda() for w in ws])(x.cuda()).cpu()
    assert torch.allclose(got.float(), want.float(), rtol=2e-3, atol=1e-6)
    assert B.lib.bgemm_device_status(1) == 0


C5_N = (1, 16, 128, 1024, 4096)


@pytest.fixture(scope="module")
def c5(B):
    """W[28672, 8192], ternary X[4096, 8192] (smaller N use its first N rows), alpha; oracle accumulators for all rows."""
    cfg = O.config5(N=max(C5_N))                            # seed 1005
    w, x, alpha = cfg["w"], cfg["x"], cfg["alpha"]
    acc = O.ref_acc(w, x, O.OP_BWTA)                        # [4096, 28672] int32, one fp32 matmul on the host
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    return dict(w=w, x=x, alpha=alpha, acc=acc, plane=plane, alpha_dev=alpha.cuda())


@pytest.mark.parametrize("N", C5_N)
def test_config5_llm_projection_single_call(B, c5, N):
    M, K = c5["w"].shape
    acts, colsum = B.prepare_acts(c5["x"][:N].cuda(), B.ACT_TERNARY)
    acc = c5["acc"][:N]
    assert torch.equal(B.gemm(c5["plane"], M, K, acts, colsum, B.OP_BWTA, B.OUT_I32).cpu(), acc)
    want = O.ref_out(acc, O.OUT_F16_SCALED, c5["alpha"])
    got = B.gemm(c5["plane"], M, K, acts, colsum, B.OP_BWTA, B.OUT_F16_SCALED, alpha=c5["alpha_dev"]).cpu()
    assert torch.allclose(got.float(), want.float(), rtol=RTOL, atol=0)
    assert torch.equal(got, want)
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("N", C5_N)
@pytest.mark.parametrize("shards", (2, 4, 8))
def test_config5_row_shards_on_one_gpu(B, c5, N, shards):
    """The multi-GPU decomposition, computed shard after shard on this GPU: rank r owns a contiguous range of rows,
    i.e. a contiguous byte range of the tiled plane, and emits its [rows_r, N] slab; the slabs concatenate to the
    full result."""
    from sharded import row_shards

    M, K = c5["w"].shape
    kblocks = -(-K // 256)
    acts, colsum = B.prepare_acts(c5["x"][:N].cuda(), B.ACT_TERNARY)
    slabs = []
    for s, e in row_shards(M, shards):
        sub = c5["plane"][(s // 128) * kblocks * 4096: -(-e // 128) * kblocks * 4096]
        slabs.append(B.gemm(sub, e - s, K, acts, colsum, B.OP_BWTA, B.OUT_F16_SCALED, B.LAYOUT_MN, c5["alpha_dev"][s:e]))
    got = torch.cat(slabs, dim=0).t().cpu()
    want = O.ref_out(c5["acc"][:N], O.OUT_F16_SCALED, c5["alpha"])
    assert torch.equal(got, want)
    assert B.lib.bgemm_device_status(1) == 0
