"""CPU tests: the oracle against the golden vectors generated from the reference, and against itself."""
import numpy as np
import pytest
import torch

import oracle as O

GOLD = np.load(__import__("pathlib").Path(__file__).parent / "golden" / "reference_golden.npz")


def test_prepack_words_match_reference_output():
    w = torch.from_numpy(GOLD["prepack_w_f16bits"].view(np.float16).copy())
    assert np.array_equal(O.c_pack_rowmajor_msb(w), GOLD["prepack_words"])
    if O.reflib() is not None:                       # the reference's own code, when it was compiled here
        assert np.array_equal(O.ref_pack_rowmajor_msb(w), GOLD["prepack_words"])


def _bnn_from_oracle(x, w, sw, sa, bias=None):
    xc = torch.from_numpy(x) - torch.from_numpy(x).mean()
    wc = torch.from_numpy(w) - torch.from_numpy(w).mean()
    acc = O.ref_acc(wc, xc, O.OP_XOR).float()
    if bias is not None:
        acc = acc + torch.from_numpy(bias)
    return acc * torch.from_numpy(sw) * float(sa)


@pytest.mark.parametrize("tag", ["bnn_a", "bnn_b", "bnn_c"])
def test_bnn_linear_golden(tag):
    bias = GOLD[f"{tag}_bias"] if f"{tag}_bias" in GOLD.files else None
    y = _bnn_from_oracle(GOLD[f"{tag}_x"], GOLD[f"{tag}_w"], GOLD[f"{tag}_sw"], GOLD[f"{tag}_sa"], bias)
    if bias is None:
        assert torch.equal(y, torch.from_numpy(GOLD[f"{tag}_y"]))
    else:   # F.linear folds the bias into the fp32 GEMM accumulation, so only the bias term may differ by rounding
        assert torch.allclose(y, torch.from_numpy(GOLD[f"{tag}_y"]), rtol=1e-5, atol=1e-7)
    # and the C restatement gives the same integers as the torch matmul
    xc = torch.from_numpy(GOLD[f"{tag}_x"]) - torch.from_numpy(GOLD[f"{tag}_x"]).mean()
    wc = torch.from_numpy(GOLD[f"{tag}_w"]) - torch.from_numpy(GOLD[f"{tag}_w"]).mean()
    assert np.array_equal(O.c_bgemm_dense(wc, xc, O.OP_XOR), O.ref_acc(wc, xc, O.OP_XOR).numpy())


def _bwta_layer(x, w, bias):
    x, w = torch.from_numpy(x), torch.from_numpy(w)
    sw = w.norm(1, 1) / w.nelement()
    sa = 2 * x.abs().mean()
    xq = (x - x.mean().item()) / sa
    wq = w - w.mean().item()
    acc = (torch.sign(xq.half().float()) @ torch.sign(wq.half().float()).T)
    # the reference multiplies a HALF product by the 0-dim fp32 scale first (stays half), then by the fp32 row scales
    y = acc.half() * sa * sw
    return y if bias is None else y + torch.from_numpy(bias)


def test_bwta_layer_golden_random():
    y = _bwta_layer(GOLD["bwta_a_x"], GOLD["bwta_a_w"], GOLD["bwta_a_bias"])
    assert torch.equal(y, torch.from_numpy(GOLD["bwta_a_y"]))


def test_bwta_layer_golden_exact_zeros():
    """Integer-valued operands with zero mean: zeros on BOTH sides must contribute nothing."""
    x, w = torch.from_numpy(GOLD["bwta_b_x"]), torch.from_numpy(GOLD["bwta_b_w"])
    assert (x == 0).any() and (w == 0).any()
    y = _bwta_layer(GOLD["bwta_b_x"], GOLD["bwta_b_w"], None)
    assert torch.equal(y, torch.from_numpy(GOLD["bwta_b_y"]))
    # two-plane decomposition used on the GPU: sum_{w != 0} sgn(w) t(x) = D_nz - 2 D_neg
    t = torch.sign(x)
    d_nz = (t @ (w != 0).float().T)
    d_neg = (t @ (w < 0).float().T)
    assert torch.equal(d_nz - 2 * d_neg, t @ torch.sign(w).T)
    # binary-weight BWTA of the oracle agrees wherever the weight row has no zero
    acc = O.ref_acc(torch.where(w == 0, torch.ones_like(w), w), x, O.OP_BWTA)
    assert np.array_equal(acc.numpy(), O.c_bgemm_dense(torch.where(w == 0, torch.ones_like(w), w), x, O.OP_BWTA))


def test_attention_product_golden():
    mask, v = torch.from_numpy(GOLD["attn_mask"]), torch.from_numpy(GOLD["attn_v"])
    want = torch.from_numpy(GOLD["attn_y"]).to(torch.int32)
    assert torch.equal(O.ref_attn_heads(mask[None], v[None])[0], want)
    # the extension encodes the mask in the sign bit: "1" = sign bit clear
    acc = O.ref_acc(2 * mask - 1, v.T.contiguous(), O.OP_ATTN)      # [d, Sq]
    assert torch.equal(acc.T, want)
    assert np.array_equal(O.c_bgemm_dense(2 * mask - 1, v.T.contiguous(), O.OP_ATTN).T, want.numpy())


def test_edge_values_of_the_reference_quantisers():
    edge = torch.from_numpy(GOLD["edge_in"])
    # torch.sign semantics of the ternary path
    assert np.array_equal(O.map_act(edge, O.OP_BWTA).numpy(), GOLD["edge_ternary"])
    # The dense twin (BinActive) sends -0.0 to +1; the reference's CUDA kernel -- which this library
    # follows -- reads the sign BIT, so -0.0 is -1 there. Everything else agrees.
    got = O.map_act(edge, O.OP_XOR).numpy()
    want = GOLD["edge_binactive"].copy()
    neg_zero = np.signbit(GOLD["edge_in"]) & (GOLD["edge_in"] == 0)
    assert np.array_equal(got[~neg_zero], want[~neg_zero])
    assert np.all(got[neg_zero] == -1) and np.all(want[neg_zero] == 1)


@pytest.mark.parametrize("op", [0, 1, 2])
def test_packed_ptx_restatement_equals_dense_definition(op):
    g = O._gen(op)
    w = torch.randn(96, 384, generator=g).half()
    x = torch.randn(40, 384, generator=g).half()
    x[0, :4] = torch.tensor([0.0, -0.0, 1.0, -1.0]).half()
    bits = O.c_bgemm_bits(O.c_pack_rowmajor_msb(w), O.c_pack_rowmajor_msb(x), 384, op)
    assert np.array_equal(bits, O.c_bgemm_dense(w, x, op))
    assert np.array_equal(bits, O.ref_acc(w, x, op).numpy())


@pytest.mark.parametrize("split_k", [1, 2, 3, 5])
def test_reference_split_k_semantics_equal_direct(split_k):
    """fp32 slabs summed then rounded (kernel_reduction.cuh) == rounding the exact integer sum."""
    g = O._gen(split_k)
    w = O.rand_pm1((64, 1280), g)
    x = O.rand_pm1((32, 1280), g)
    direct = O.ref_out(O.ref_acc(w, x, O.OP_XOR), O.OUT_F16).numpy()
    assert np.array_equal(O.c_splitk_f16(w, x, O.OP_XOR, split_k).view(np.uint16), direct.view(np.uint16))


def test_store_conversions():
    acc = torch.arange(-9000, 9000, 7, dtype=torch.int32).reshape(1, -1).repeat(3, 1).contiguous()
    alpha = (0.01 + 0.09 * torch.rand(acc.shape[1], generator=O._gen(9))).half()
    assert np.array_equal(O.c_store_f16(acc.numpy()).view(np.uint16), O.ref_out(acc, O.OUT_F16).numpy().view(np.uint16))
    assert np.array_equal(O.c_store_f16_scaled(acc.numpy(), alpha.numpy()).view(np.uint16),
                          O.ref_out(acc, O.OUT_F16_SCALED, alpha).numpy().view(np.uint16))


def test_fp16_conversion_against_numpy():
    lib = O.clib()
    rs = np.random.RandomState(0)
    vals = np.concatenate([np.arange(-70000, 70000, 13, dtype=np.float32),
                           (rs.randn(20000) * 10.0 ** rs.randint(-9, 6, 20000)).astype(np.float32),
                           np.array([0.0, -0.0, 65504, 65519.99, 65520, 2 ** -24, 2 ** -25, 1.5 * 2 ** -25, np.inf, -np.inf], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)
    halves = np.arange(0, 65536, 17, dtype=np.uint16)
    halves = halves[~np.isnan(halves.view(np.float16))]          # NaN payload handling is not part of the path
    back = np.array([lib.oracle_f16_to_f32(int(h)) for h in halves], dtype=np.float32)
    assert np.array_equal(back.view(np.uint32), halves.view(np.float16).astype(np.float32).view(np.uint32))


def test_layout_restatement_roundtrip():
    g = O._gen(4)
    M, K = 200, 700
    w = torch.randn(M, K, generator=g).half()
    plane, pop = O.np_pack_weights(w, 0)
    assert plane.size == O.plane_bytes(M, K)
    words = plane.view(np.uint32).reshape(-(-M // 128), -(-K // 256), 2, 128, 4)
    s = torch.signbit(w).numpy()
    for (m, k) in [(0, 0), (199, 699), (130, 300), (5, 255), (128, 256)]:
        kb, kk = divmod(k, 256)
        j, c, b = kk // 32, (kk % 32) // 4, kk % 4
        bit = (words[m // 128, kb, c // 4, m % 128, c % 4] >> (8 * b + j)) & 1
        assert bit == int(s[m, k])
    assert pop.sum() == s.sum()
    a, c = O.np_prepare_acts(w, O.ACT_TERNARY)
    assert a.shape == (M, O.act_ld(K)) and np.array_equal(c, torch.sign(w.float()).sum(1).int().numpy())


def test_mlp_reference_shapes():
    cfg = O.config4(batch=8, dims=(64, 128, 128, 10))
    y, accs = O.ref_mlp(cfg["ws"], cfg["x"])
    assert y.shape == (8, 10) and y.dtype == torch.float16 and len(accs) == 3
