"""GPU parity tests: every result of libbgemm_b200.so (called through its C ABI) against the CPU oracle.

Integer results are compared bit for bit; fp16-scaled results within 1e-3 relative (they are in fact
produced by the same fp32-multiply + round-to-nearest-even and are also checked for exact equality).
"""
import numpy as np
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def B():
    import bgemm_b200

    return bgemm_b200


def _rand_w(M, K, g, kind="pm1"):
    if kind == "pm1":
        return O.rand_pm1((M, K), g)
    return torch.randn(M, K, generator=g).to(torch.float16)


def _acts_for(op, N, K, g):
    if op == O.OP_BWTA:
        return O.rand_ternary((N, K), g)
    x = torch.randn(N, K, generator=g).to(torch.float16)
    x[0, 0] = 0.0          # +0 -> +1
    if K > 1:
        x[0, 1] = -0.0     # -0 -> -1 (sign bit)
    return x


def _run(B, w, x, op, split_k=0, out_kind=O.OUT_I32, layout=0, alpha=None):
    wd, xd = w.cuda(), x.cuda()
    plane, _, _ = B.pack_weights(wd, B.WBIT_OF_OP[op])
    acts, colsum = B.prepare_acts(xd, B.ACT_MODE_OF_OP[op])
    return B.gemm(plane, w.shape[0], w.shape[1], acts, colsum, op, out_kind, layout,
                  None if alpha is None else alpha.cuda(), split_k).cpu()


@pytest.mark.parametrize("M,K", [(128, 256), (200, 300), (10, 4096), (257, 1000), (1024, 1024)])
@pytest.mark.parametrize("mode", [0, 1])
def test_pack_weights_matches_layout_definition(B, M, K, mode):
    g = O._gen(M * 7 + K)
    w = torch.randn(M, K, generator=g).to(torch.float16)
    w[0, 0] = 0.0
    w[M - 1, K - 1] = -0.0
    plane, rowpop, alpha = B.pack_weights(w.cuda(), mode, want_rowpop=True, want_alpha=True)
    ref_plane, ref_pop = O.np_pack_weights(w, mode)
    assert plane.numel() == O.plane_bytes(M, K)
    assert np.array_equal(plane.cpu().numpy(), ref_plane)
    assert np.array_equal(rowpop.cpu().numpy(), ref_pop)
    ref_alpha = O.c_rowmeanabs_f16(w).astype(np.float32)
    got = alpha.cpu().float().numpy()
    assert np.all(np.abs(got - ref_alpha) <= 1e-3 * np.abs(ref_alpha) + 1e-7)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32, torch.int8])
def test_pack_weights_dtypes_and_host_twin(B, dtype):
    import ctypes

    g = O._gen(5)
    M, K = 130, 520
    base = torch.randint(-3, 4, (M, K), generator=g)
    w = base.to(dtype)
    plane, rowpop, _ = B.pack_weights(w.cuda(), 0, want_rowpop=True)
    ref_plane, ref_pop = O.np_pack_weights(base.float() - 0.0, 0)   # zero -> +0 -> bit 0, like int8 0
    assert np.array_equal(plane.cpu().numpy(), ref_plane)
    assert np.array_equal(rowpop.cpu().numpy(), ref_pop)
    # CPU twin writes the same bytes
    host_plane = np.zeros(O.plane_bytes(M, K), dtype=np.uint8)
    host_pop = np.zeros(M, dtype=np.int32)
    wc = w.contiguous()
    rc = B.lib.bgemm_pack_weights_host(wc.data_ptr(), B.dtype_code(wc), M, K, K, 0, host_plane.ctypes.data, host_pop.ctypes.data, None)
    assert rc == 0
    assert np.array_equal(host_plane, ref_plane) and np.array_equal(host_pop, ref_pop)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32, torch.int8])
@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("M,K,offset", [(130, 520, 0), (70, 515, 0), (300, 1024, 0), (200, 768, 1)])
def test_pack_weights_every_mode_dtype_and_alignment(B, dtype, mode, M, K, offset):
    """Vector and element-wise paths of the packing kernel (whole and ragged K blocks, rows that start off a 16-byte
    boundary) for every source type and weight-bit mode, with row sums and scales."""
    g = O._gen(M + K + mode)
    base = torch.randint(-3, 4, (M, K + 8), generator=g)
    wide = base.to(dtype).cuda()
    w = wide[:, offset:offset + K]                       # a view: row pitch K + 8, rows misaligned when offset is odd
    plane, rowpop, alpha = B.pack_weights(w, mode, want_rowpop=True, want_alpha=True)
    ref = base[:, offset:offset + K].float() - 0.0      # zero -> +0 -> sign bit clear, like int8 0
    ref_plane, ref_pop = O.np_pack_weights(ref, mode)
    assert np.array_equal(plane.cpu().numpy(), ref_plane)
    assert np.array_equal(rowpop.cpu().numpy(), ref_pop)
    want_alpha = ref.abs().mean(dim=1).numpy()
    assert np.all(np.abs(alpha.cpu().float().numpy() - want_alpha) <= 1e-3 * want_alpha + 1e-7)


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("N,K", [(1, 256), (5, 300), (64, 4096), (33, 1000), (300, 4096)])
def test_prepare_acts(B, mode, N, K):
    g = O._gen(N + K + mode)
    x = O.rand_ternary((N, K), g) if mode == 1 else torch.randn(N, K, generator=g).to(torch.float16)
    x[0, 0] = -0.0
    acts, colsum = B.prepare_acts(x.cuda(), mode)
    ref_a, ref_c = O.np_prepare_acts(x, mode)
    assert np.array_equal(acts.cpu().numpy(), ref_a)
    assert np.array_equal(colsum.cpu().numpy(), ref_c)
    # transposed source gives the same result
    acts_t, colsum_t = B.prepare_acts(x.t().contiguous().cuda(), mode, transpose=True)
    assert np.array_equal(acts_t.cpu().numpy(), ref_a)
    assert np.array_equal(colsum_t.cpu().numpy(), ref_c)


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("N,K,pad", [(3, 4096, 0), (40, 8192, 0), (5, 2500, 0), (7, 4096, 4), (2, 300, 0), (1100, 2304, 0)])
def test_prepare_acts_from_int8_sources(B, mode, N, K, pad):
    """int8 activations (ternary values already stored as bytes, or general int8 for W1A8) through every mode: rows long
    enough for the 8-byte vector path, ragged tails, rows that are not 8-byte aligned (pitch K + 4)."""
    g = O._gen(N + K + mode)
    full = torch.randint(-128, 128, (N, K + pad), generator=g, dtype=torch.int8)
    full[:, ::7] = 0
    x = full[:, :K]
    acts, colsum = B.prepare_acts(full.cuda()[:, :K], mode)
    ref_a, ref_c = O.np_prepare_acts(x, mode)
    assert np.array_equal(acts.cpu().numpy(), ref_a)
    assert np.array_equal(colsum.cpu().numpy(), ref_c)


def test_rowmajor_msb_prepack_matches_reference_format(B):
    g = O._gen(11)
    M, K = 96, 512
    w = torch.randn(M, K, generator=g).to(torch.float16)
    w[3, 5] = -0.0
    dst = torch.empty((M, K // 32), dtype=torch.int32, device="cuda")
    B.check(B.lib.bgemm_pack_rowmajor_msb(None, w.cuda().data_ptr(), B.DT_F16, M, K, K, dst.data_ptr()), "pack_rowmajor")
    torch.cuda.synchronize()
    got = dst.cpu().numpy().view(np.uint32)
    assert np.array_equal(got, O.c_pack_rowmajor_msb(w))
    if O.reflib() is not None:
        assert np.array_equal(got, O.ref_pack_rowmajor_msb(w))
    # retiling the reference format gives the same plane as packing directly
    plane = torch.empty(O.plane_bytes(M, K), dtype=torch.uint8, device="cuda")
    B.check(B.lib.bgemm_retile_rowmajor_msb(None, dst.data_ptr(), M, K, 0, plane.data_ptr()), "retile")
    direct, _, _ = B.pack_weights(w.cuda(), 0)
    assert torch.equal(plane, direct)


OPS = [O.OP_AND, O.OP_XOR, O.OP_ATTN, O.OP_BWTA]


@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("N", [1, 7, 16, 17, 32, 33, 64, 100, 128, 200, 256, 300, 520])
def test_gemm_all_tile_widths(B, op, N):
    g = O._gen(100 + N + op)
    M, K = 256, 512
    w = _rand_w(M, K, g, "randn")
    x = _acts_for(op, N, K, g)
    got = _run(B, w, x, op, split_k=1)
    assert torch.equal(got, O.ref_acc(w, x, op))


@pytest.mark.parametrize("M,K,N", [(19200, 512, 24), (19300, 768, 32), (38400, 300, 17)])
def test_few_columns_on_more_row_tiles_than_sms(B, M, K, N):
    """17-32 activation rows with more 128-row tiles than SMs run on 64-column tiles (half of them padding): two CTAs per
    SM, or the persistent kernel beyond two tiles per SM."""
    g = O._gen(M + K + N)
    for op in (O.OP_XOR, O.OP_BWTA):
        w = _rand_w(M, K, g, "randn")
        x = _acts_for(op, N, K, g)
        assert torch.equal(_run(B, w, x, op, split_k=1), O.ref_acc(w, x, op)), (op, M, K, N)
        assert torch.equal(_run(B, w, x, op, split_k=0), O.ref_acc(w, x, op)), (op, M, K, N)


@pytest.mark.parametrize("M,K", [(128, 256), (130, 384), (10, 4096), (257, 1000), (640, 129), (1, 1), (300, 8192)])
@pytest.mark.parametrize("N", [3, 24, 64, 130])
@pytest.mark.parametrize("split_k", [1, 0, 3, 8, 12])
def test_gemm_ragged_shapes_and_split_k(B, M, K, N, split_k):
    g = O._gen(M + K + N)
    for op in (O.OP_XOR, O.OP_BWTA):
        w = _rand_w(M, K, g, "randn")
        x = _acts_for(op, N, K, g)
        got = _run(B, w, x, op, split_k=split_k)
        assert torch.equal(got, O.ref_acc(w, x, op)), (op, M, K, N, split_k)


def test_gemm_known_answers(B):
    M, N, K = 128, 16, 512
    ones = torch.ones(M, K, dtype=torch.float16)
    xs = torch.ones(N, K, dtype=torch.float16)
    assert torch.all(_run(B, ones, xs, O.OP_XOR) == K)
    assert torch.all(_run(B, -ones, xs, O.OP_XOR) == -K)
    assert torch.all(_run(B, -ones, -xs, O.OP_AND) == K)
    assert torch.all(_run(B, ones, -xs, O.OP_AND) == 0)
    assert torch.all(_run(B, ones, -xs, O.OP_ATTN) == -K)        # mask all ones, values all -1
    assert torch.all(_run(B, -ones, xs, O.OP_ATTN) == 0)         # mask all zeros
    assert torch.all(_run(B, ones, torch.zeros(N, K, dtype=torch.float16), O.OP_BWTA) == 0)
    alt = torch.ones(M, K, dtype=torch.float16)
    alt[:, 1::2] = -1
    assert torch.all(_run(B, alt, xs, O.OP_XOR) == 0)
    # single element set: only column k0 of x is non-zero -> result is sign(w[:, k0])
    e = torch.zeros(N, K, dtype=torch.float16)
    e[:, 77] = 1
    g = O._gen(3)
    w = O.rand_pm1((M, K), g)
    got = _run(B, w, e, O.OP_BWTA)
    assert torch.equal(got, w[:, 77].to(torch.int32).unsqueeze(0).expand(N, M))


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("split_k", [1, 4, 5, 8])
def test_output_kinds(B, layout, split_k):
    cfg = O.config2(M=384, K=2048, N=40)
    w, x, alpha = cfg["w"], cfg["x"], cfg["alpha"]
    acc = O.ref_acc(w, x, O.OP_BWTA)
    want = {O.OUT_I32: acc, O.OUT_F16: O.ref_out(acc, O.OUT_F16), O.OUT_F16_SCALED: O.ref_out(acc, O.OUT_F16_SCALED, alpha)}
    for kind in (O.OUT_I32, O.OUT_F16, O.OUT_F16_SCALED):
        got = _run(B, w, x, O.OP_BWTA, split_k=split_k, out_kind=kind, layout=layout, alpha=alpha)
        ref = want[kind] if layout == 0 else want[kind].t()
        assert got.shape == ref.shape
        if kind == O.OUT_I32:
            assert torch.equal(got, ref)
        else:
            assert torch.allclose(got.float(), ref.float(), rtol=1e-3, atol=0)
            assert torch.equal(got, ref)          # same arithmetic -> same bits
    # C restatement of the store conversions agrees too
    assert np.array_equal(O.c_store_f16_scaled(acc.numpy(), alpha.numpy()).view(np.uint16), want[O.OUT_F16_SCALED].numpy().view(np.uint16))


def test_f16_rounding_above_2048(B):
    """|acc| > 2048 is not representable in fp16: the store must round to nearest even like __int2half_rn."""
    M, N, K = 128, 16, 8192
    w = torch.ones(M, K, dtype=torch.float16)
    x = torch.ones(N, K, dtype=torch.float16)
    x[:, :5] = -1                                     # acc = 8192 - 10 = 8182: a tie between 8180 and 8184 -> even
    got = _run(B, w, x, O.OP_XOR, out_kind=O.OUT_F16)
    assert torch.all(got == O.ref_out(O.ref_acc(w, x, O.OP_XOR), O.OUT_F16))
    assert float(got[0, 0]) == 8184.0


@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("M,N,K", [(256, 32, 512), (100, 5, 300), (512, 96, 1280)])
def test_linear_forward_dropin(B, op, M, N, K):
    g = O._gen(op + M)
    w = _rand_w(M, K, g, "randn")
    x = _acts_for(op, N, K, g)
    got = B.linear_forward(w.cuda(), x.cuda(), op, out_kind=B.OUT_F16).cpu()
    assert torch.equal(got, O.ref_out(O.ref_acc(w, x, op), O.OUT_F16))
    got32 = B.linear_forward(w.cuda(), x.cuda(), op, out_kind=B.OUT_I32, split_k=2).cpu()
    assert torch.equal(got32, O.ref_acc(w, x, op))
    if K % 128 == 0:
        # packed-bit restatement of the reference PTX agrees with the dense definition
        if op != O.OP_BWTA:
            bits = O.c_bgemm_bits(O.c_pack_rowmajor_msb(w), O.c_pack_rowmajor_msb(x), K, op)
            assert np.array_equal(bits, got32.numpy())


def test_shared_workspace_survives_calls_of_different_shapes(B):
    """One scratch buffer serves calls whose layouts differ; the arrival counters must stay usable."""
    g = O._gen(91)
    for (M, N, K, sk) in [(256, 32, 8192, 16), (1024, 200, 4096, 12), (128, 16, 8192, 32), (256, 32, 8192, 16), (640, 64, 2560, 9)]:
        w, x = _rand_w(M, K, g, "randn"), _acts_for(O.OP_BWTA, N, K, g)
        assert torch.equal(_run(B, w, x, O.OP_BWTA, split_k=sk), O.ref_acc(w, x, O.OP_BWTA)), (M, N, K, sk)
        got = B.linear_forward(w.cuda(), x.cuda(), O.OP_BWTA, out_kind=B.OUT_I32, split_k=sk).cpu()
        assert torch.equal(got, O.ref_acc(w, x, O.OP_BWTA)), (M, N, K, sk)


def test_batched_attention_heads(B):
    cfg = O.config3(heads=6, S=256, d=64)
    a, v = cfg["attn"], cfg["v"]
    H, S, d = v.shape
    # the reference encodes the {0,1} mask in the sign bit: "1" = sign bit clear
    plane, _, _ = B.pack_weights((2 * a - 1).cuda(), B.WBIT_NONNEGATIVE)
    acts, colsum = B.prepare_acts(v.cuda(), B.ACT_SIGN, transpose=True)       # V^T: [H, d, S]
    got = B.gemm(plane, S, S, acts, colsum, B.OP_ATTN, B.OUT_I32, B.LAYOUT_MN).cpu()
    assert got.shape == (H, S, d)
    assert torch.equal(got, O.ref_attn_heads(a, v))


def test_late_waves_mn_int32_every_run(B):
    """More tiles than the GPU holds at once, [M, N] int32 output (the slowest epilogue), repeated: tiles of the
    later waves run next to CTAs that are storing, which once let a weight stage be refilled before a stalled warp
    had read it (32 rows of a tile wrong in ~45 % of the runs). Every run must equal the oracle bit for bit."""
    M, K, N = 4096, 2048, 2048
    g = O._gen(4242)
    w = O.rand_pm1((M, K), g)
    x = O.rand_ternary((N, K), g)
    ref = O.ref_acc(w, x, O.OP_BWTA).t().contiguous()
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[O.OP_BWTA])
    for rep in range(12):
        got = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, 1, None, 1).cpu()
        assert torch.equal(got, ref), f"run {rep}: {int((got != ref).sum())} elements differ"
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,batch,layout", [(512, 2048, 128, 80, 0), (384, 2304, 104, 110, 1), (1000, 2048, 100, 40, 0),
                                                (256, 4096, 64, 200, 0), (128, 2304, 64, 333, 1), (100, 2048, 40, 310, 0),
                                                (512, 512, 64, 100, 1), (256, 768, 64, 200, 0), (384, 1024, 128, 100, 0)])
def test_pools_on_the_persistent_kernel(B, M, K, N, batch, layout):
    """Pools of narrow problems in one launch (more tiles than two per SM, one tile across N) take the persistent kernel:
    odd K-block counts (short odd ones fall back to the tile-per-CTA kernel), two-K-block attention-like tiles,
    ragged M and N, both layouts, all three output kinds."""
    g = O._gen(M + K + N + batch)
    w = O.rand_pm1((batch, M, K), g)
    x = O.rand_ternary((batch, N, K), g)
    alpha = (torch.rand(batch, M, generator=g) + 0.5).to(torch.float16)
    acc = O.ref_acc(w, x, O.OP_BWTA)                                   # [batch, N, M]
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[O.OP_BWTA])
    for kind in (O.OUT_I32, O.OUT_F16, O.OUT_F16_SCALED):
        want = O.ref_out(acc, kind, alpha.unsqueeze(1))
        if layout == 1:
            want = want.transpose(1, 2)
        got = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, kind, layout, alpha.cuda(), 1).cpu()
        assert got.shape == want.shape
        if kind != O.OUT_I32:
            assert torch.allclose(got.float(), want.float(), rtol=1e-3, atol=0)
        assert torch.equal(got, want), (kind, int((got != want).sum()))
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,batch", [(12800, 3072, 300, 1), (1024, 3328, 256, 20)])
def test_persistent_kernel_with_several_tiles_across_n(B, M, K, N, batch):
    """More than two tiles per SM, 12 or more K blocks per tile, two or three tiles across N (the last one ragged)."""
    g = O._gen(M + K + N + batch)
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = O.rand_pm1(shape_w, g)
    x = O.rand_ternary(shape_x, g)
    acc = O.ref_acc(w, x, O.OP_BWTA)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[O.OP_BWTA])
    for layout in (0, 1):
        want = acc if layout == 0 else acc.transpose(-1, -2)
        got = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, layout, None, 1).cpu()
        assert torch.equal(got, want), (layout, int((got != want).sum()))
    assert B.lib.bgemm_device_status(1) == 0


def test_persistent_kernel_under_graph_replay(B):
    """The persistent kernel's barrier rings across many tiles, replayed back to back from a CUDA graph."""
    M, K, N, batch = 1024, 2304, 128, 60
    g = O._gen(77)
    w = O.rand_pm1((batch, M, K), g)
    x = O.rand_ternary((batch, N, K), g)
    ref = O.ref_acc(w, x, O.OP_BWTA)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[O.OP_BWTA])
    out = torch.empty((batch, N, M), dtype=torch.int32, device="cuda")
    B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, 0, None, 1, out=out)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            for _ in range(10):
                B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, 0, None, 1, out=out)
    for _ in range(3):
        out.fill_(-1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), ref)
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,batch,split_k", [(384, 1024, 40, 1, 1), (1000, 2048, 100, 1, 0), (300, 4096, 17, 3, 4), (256, 8192, 64, 1, 12),
                                                  (512, 2048, 128, 80, 1)])
@pytest.mark.parametrize("next_mode", [0, 1, 2])
def test_gemm_to_acts_equals_gemm_then_prepare(B, M, K, N, batch, split_k, next_mode):
    """The fused activation producer writes exactly what the fp16 output followed by prepare_acts gives (ragged M:
    zero padding up to the 256-column pitch; every K partitioning; the persistent kernel for the pool case)."""
    g = O._gen(M + K + N + batch + next_mode)
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = O.rand_pm1(shape_w, g)
    x = O.rand_ternary(shape_x, g)
    alpha = (torch.rand((batch, M) if batch > 1 else (M,), generator=g) * 0.5).to(torch.float16)
    alpha.view(-1)[3] = 0.0                                               # a dead row: results +-0, sign bit decides
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[O.OP_BWTA])
    for a in (alpha.cuda(), None):
        y = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_F16_SCALED if a is not None else O.OUT_F16, 0, a, split_k)
        want_acts, want_cs = B.prepare_acts(y, next_mode)
        got_acts, got_cs = B.gemm_to_acts(plane, M, K, acts, colsum, O.OP_BWTA, next_mode, a, split_k)
        assert got_acts.shape == want_acts.shape
        assert torch.equal(got_acts, want_acts)
        assert torch.equal(got_cs, want_cs)
        # row sums added to an array the caller has zeroed (no memset by the library)
        sums = torch.zeros(want_cs.numel(), dtype=torch.int32, device="cuda")
        got_acts, got_cs = B.gemm_to_acts(plane, M, K, acts, colsum, O.OP_BWTA, next_mode, a, split_k, sums=sums)
        assert torch.equal(got_acts, want_acts) and torch.equal(got_cs, want_cs) and got_cs.data_ptr() == sums.data_ptr()
    # and against the oracle's definition of the activation mapping
    acc = O.ref_acc(w, x, O.OP_BWTA)
    yref = O.ref_out(acc, O.OUT_F16_SCALED, alpha.unsqueeze(-2) if batch > 1 else alpha)
    np_acts, np_cs = O.np_prepare_acts(yref.reshape(-1, M), next_mode)
    got_acts, got_cs = B.gemm_to_acts(plane, M, K, acts, colsum, O.OP_BWTA, next_mode, alpha.cuda(), split_k)
    assert np.array_equal(got_acts.cpu().numpy().reshape(-1, got_acts.shape[-1]), np_acts)
    assert np.array_equal(got_cs.cpu().numpy().reshape(-1), np_cs)


@pytest.mark.parametrize("M,K,N,batch,layout", [(20000, 2304, 9, 1, 1), (1000, 4096, 16, 25, 0), (28672, 2048, 1, 1, 0), (19000, 2560, 16, 1, 0)])
def test_weight_streaming_shapes(B, M, K, N, batch, layout):
    """N <= 16 with more row tiles than SMs (the weight-streaming regime of the N = 1 / 16 sweep points): odd and
    even K-block counts, ragged M, batches, all output kinds, automatic and forced K partitioning, repeated."""
    g = O._gen(M + K + N + batch)
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = O.rand_pm1(shape_w, g)
    x = O.rand_ternary(shape_x, g)
    alpha = (torch.rand((batch, M) if batch > 1 else (M,), generator=g) + 0.5).to(torch.float16)
    acc = O.ref_acc(w, x, O.OP_BWTA)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[O.OP_BWTA])
    for kind in (O.OUT_I32, O.OUT_F16_SCALED, O.OUT_I32):
        want = O.ref_out(acc, kind, alpha.unsqueeze(-2) if batch > 1 else alpha)
        if layout == 1:
            want = want.transpose(-1, -2)
        got = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, kind, layout, alpha.cuda(), 0).cpu()
        assert torch.equal(got, want), (kind, int((got != want).sum()))
        assert torch.equal(B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, kind, layout, alpha.cuda(), 1).cpu(), want)
    na, ncs = B.gemm_to_acts(plane, M, K, acts, colsum, O.OP_BWTA, 1, alpha.cuda(), 0)
    ra, rcs = O.np_prepare_acts(O.ref_out(acc, O.OUT_F16_SCALED, alpha.unsqueeze(-2) if batch > 1 else alpha).reshape(-1, M), 1)
    assert np.array_equal(na.cpu().numpy().reshape(-1, na.shape[-1]), ra) and np.array_equal(ncs.cpu().numpy().reshape(-1), rcs)
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,split_k", [(256, 512, 33, 1), (1000, 4096, 128, 0), (4096, 2048, 16, 4), (130, 300, 7, 0)])
def test_binary_weight_int8_activation(B, M, K, N, split_k):
    """W1A8: int8 activations go through prepare_acts unchanged (BGEMM_ACT_INT8) and op BWTA gives
    sum_k sign(w) * x exactly (|acc| <= 127 K)."""
    g = O._gen(M + K + N)
    w = torch.randn(M, K, generator=g).to(torch.float16)
    x = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    want = (x.to(torch.float64) @ O.map_weight(w, O.OP_BWTA).to(torch.float64).t()).to(torch.int32)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_INT8)
    ra, rcs = O.np_prepare_acts(x, O.ACT_INT8)
    assert np.array_equal(acts.cpu().numpy(), ra) and np.array_equal(colsum.cpu().numpy(), rcs)
    got = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, 0, None, split_k).cpu()
    assert torch.equal(got, want)
    # fp16 activations are refused for this mode before anything is launched
    xh = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
    dst = torch.empty(4, 256, dtype=torch.int8, device="cuda")
    cs = torch.empty(4, dtype=torch.int32, device="cuda")
    assert B.lib.bgemm_prepare_acts(None, xh.data_ptr(), 0, 4, 256, 256, B.ACT_INT8, 0, dst.data_ptr(), cs.data_ptr(), 1, 0) == -6


def test_seeded_random_shapes(B):
    """Sixty seeded random problems over every knob of bgemm_gemm (op, shape, batch, K partitioning, output kind and
    layout) and of bgemm_gemm_to_acts, each against the oracle."""
    rng = np.random.default_rng(20240611)
    for case in range(60):
        op = int(rng.choice(OPS))
        M = int(rng.choice([1, 37, 128, 129, 300, 512, 1000]))
        K = int(rng.choice([1, 100, 256, 257, 768, 1024, 2304, 4096]))
        N = int(rng.choice([1, 5, 16, 40, 64, 65, 128, 130, 300]))
        batch = int(rng.choice([1, 1, 1, 3, 40, 170]))
        if batch * M * K > (1 << 26) or batch * M * N > (1 << 24):
            batch = 1
        split_k = int(rng.choice([0, 1, 1, 2, 5, 8, 11]))
        layout = int(rng.integers(0, 2))
        kind = int(rng.choice([O.OUT_I32, O.OUT_F16, O.OUT_F16_SCALED]))
        g = O._gen(1000 + case)
        shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
        w = torch.randn(shape_w, generator=g).to(torch.float16)
        x = O.rand_ternary(shape_x, g) if op == O.OP_BWTA else torch.randn(shape_x, generator=g).to(torch.float16)
        alpha = (torch.rand((batch, M) if batch > 1 else (M,), generator=g) + 0.25).to(torch.float16)
        acc = O.ref_acc(w, x, op)
        plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
        acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[op])
        got = B.gemm(plane, M, K, acts, colsum, op, kind, layout, alpha.cuda(), split_k).cpu()
        want = O.ref_out(acc, kind, alpha.unsqueeze(-2) if batch > 1 else alpha)
        if layout == 1:
            want = want.transpose(-1, -2)
        tag = (case, op, M, K, N, batch, split_k, layout, kind)
        assert got.shape == want.shape, tag
        assert torch.equal(got, want), tag
        if case % 3 == 0:
            mode = int(rng.integers(0, 3))
            na, ncs = B.gemm_to_acts(plane, M, K, acts, colsum, op, mode, alpha.cuda(), split_k)
            y = O.ref_out(acc, O.OUT_F16_SCALED, alpha.unsqueeze(-2) if batch > 1 else alpha)
            ra, rcs = O.np_prepare_acts(y.reshape(-1, M), mode)
            assert np.array_equal(na.cpu().numpy().reshape(-1, na.shape[-1]), ra), tag
            assert np.array_equal(ncs.cpu().numpy().reshape(-1), rcs), tag
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,layout,kind", [(384, 1024, 200, 0, O.OUT_F16_SCALED), (300, 2048, 130, 1, O.OUT_I32), (512, 4096, 9, 0, O.OUT_F16_SCALED),
                                                (256, 512, 64, 0, O.OUT_I32), (1000, 768, 1, 0, O.OUT_F16_SCALED), (128, 8192, 40, 1, O.OUT_F16)])
def test_multi_destination_epilogue_with_pitch(B, M, K, N, layout, kind):
    """bgemm_gemm_multi_out: the slab of a row shard written into three wider matrices at a column (row) offset -- the
    fused all-gather of the row-sharded layer, here with all destinations on this GPU. Everything outside the slab
    must stay untouched."""
    g = O._gen(M + K + N)
    w, x = O.rand_pm1((M, K), g), O.rand_ternary((N, K), g)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    want = O.ref_out(O.ref_acc(w, x, O.OP_BWTA), kind, alpha)                    # [N, M]
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_TERNARY)
    dt = torch.int32 if kind == O.OUT_I32 else torch.float16
    esz = 4 if kind == O.OUT_I32 else 2
    if layout == 0:       # [N, M_total], this shard's columns start at `off`
        total, off = M + 640, 256
        bufs = [torch.full((N, total), -7, dtype=dt, device="cuda") for _ in range(3)]
        ptrs = [b.data_ptr() + esz * off for b in bufs]
        ref = torch.full((N, total), -7, dtype=dt)
        ref[:, off:off + M] = want
    else:                 # [M_total, N] with a wider row pitch, this shard's rows start at `off`
        pitch, off = N + 24, 16
        bufs = [torch.full((M + 32, pitch), -7, dtype=dt, device="cuda") for _ in range(3)]
        ptrs = [b.data_ptr() + esz * off * pitch for b in bufs]
        total = pitch
        ref = torch.full((M + 32, pitch), -7, dtype=dt)
        ref[off:off + M, :N] = want.t()
    B.gemm_multi_out(plane, M, K, acts, colsum, B.OP_BWTA, ptrs, total, kind, layout, alpha.cuda() if kind == O.OUT_F16_SCALED else None)
    for b in bufs:
        assert torch.equal(b.cpu(), ref)
    assert B.lib.bgemm_device_status(1) == 0


def test_argument_errors(B):
    x = torch.zeros(4, 256, dtype=torch.float16, device="cuda")
    assert B.lib.bgemm_pack_weights(None, None, 0, 4, 256, 256, 0, x.data_ptr(), None, None, 1, 0) == -1
    assert B.lib.bgemm_pack_weights(None, x.data_ptr(), 9, 4, 256, 256, 0, x.data_ptr(), None, None, 1, 0) == -4
    assert B.lib.bgemm_pack_weights(None, x.data_ptr(), 0, 0, 256, 256, 0, x.data_ptr(), None, None, 1, 0) == -2
    assert B.lib.bgemm_gemm(None, x.data_ptr(), 4, 256, x.data_ptr(), x.data_ptr(), 4, 1, x.data_ptr(), 2, 0, None, 1, None, 0, 1) == -1
    # split-K without a workspace is refused before anything is launched
    assert B.lib.bgemm_gemm(None, x.data_ptr(), 4, 8192, x.data_ptr(), x.data_ptr(), 4, 1, x.data_ptr(), 0, 0, None, 16, None, 0, 1) == -5
    assert b"workspace" in B.lib.bgemm_status_string(-5)
    with pytest.raises(ValueError):
        B.pack_weights(torch.zeros(4, 256, dtype=torch.float16))
