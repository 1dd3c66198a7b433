"""GPU tests of the binary-weight x fp16-activation product (bgemm_w1a16_gemm; "W1A16", a to-do item of the reference's
README.md:29): the oracle is the CPU fp32 matmul of the fp16 activations with the sign-mapped weights. The kernel sums
fp32 partial results in an order of its own, so results are compared within 1e-3 relative (of the largest magnitude of
the row's result, which bounds cancellation), not bit for bit; with small integer activations every partial sum is
exactly representable and the comparison is exact."""
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
RTOL = 1e-3


@pytest.fixture(scope="module")
def B():
    import bgemm_b200

    return bgemm_b200


def _close(got, want):
    scale = want.abs().amax().clamp_min(1e-6)
    return bool(((got.float() - want).abs() <= RTOL * want.abs() + RTOL * scale).all())


@pytest.mark.parametrize("M,K,N", [(128, 256, 1), (300, 1000, 3), (4096, 4096, 8), (1000, 8192, 5), (513, 4100, 20), (64, 128, 9),
                                   (37, 1, 2), (2048, 11008, 4), (8192, 8192, 1), (28672, 2048, 16), (256, 40000, 2)])
def test_against_fp32_matmul(B, M, K, N):
    g = O._gen(M + K + N)
    w = torch.randn(M, K, generator=g).to(torch.float16)
    x = torch.randn(N, K, generator=g).to(torch.float16)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    want = O.ref_w1a16(w, x)
    for layout in (0, 1):
        got = B.w1a16_gemm(plane, M, K, x.cuda(), B.OUT_F32, layout).cpu()
        assert got.dtype == torch.float32 and _close(got if layout == 0 else got.t(), want), (M, K, N, layout)
    want_s = O.ref_w1a16(w, x, alpha)
    got16 = B.w1a16_gemm(plane, M, K, x.cuda(), B.OUT_F16, 0, alpha.cuda()).cpu()
    assert got16.dtype == torch.float16 and _close(got16, want_s.to(torch.float16).float())
    assert B.lib.bgemm_device_status(1) == 0


def test_small_integer_activations_are_exact(B):
    """Activations in {-4 .. 4}: every product and every partial sum is an integer far below 2**24, so the order of the
    fp32 additions cannot matter and the result must equal the oracle exactly -- also from an activation matrix whose
    rows are not 16-byte aligned (row pitch 1003 elements)."""
    M, K, N = 640, 1000, 11
    g = O._gen(3)
    w = torch.randn(M, K, generator=g).to(torch.float16)
    xw = torch.randint(-4, 5, (N, 1003), generator=g).to(torch.float16)
    x = xw[:, :K]
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    got = B.w1a16_gemm(plane, M, K, xw.cuda()[:, :K], B.OUT_F32, 0).cpu()
    assert torch.equal(got, O.ref_w1a16(w, x))
    # ternary activations: the same numbers as the integer BWTA path
    xt = O.rand_ternary((N, K), g)
    acts, colsum = B.prepare_acts(xt.cuda(), B.ACT_TERNARY)
    acc = B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, B.OUT_I32).cpu()
    assert torch.equal(B.w1a16_gemm(plane, M, K, xt.cuda(), B.OUT_F32, 0).cpu(), acc.float())


def test_extension_op_and_argument_errors(B):
    import lowbit_kernel

    g = O._gen(8)
    M, K, N = 512, 2048, 6
    w = torch.randn(M, K, generator=g).half()
    x = torch.randn(N, K, generator=g).half()
    plane = lowbit_kernel.binary_weight_prepacking_cuda(w.cuda(), 0)
    y = lowbit_kernel.w1a16_linear_forward(x.cuda(), plane, M, K, None, True, False)
    assert y.shape == (N, M) and y.dtype == torch.float32 and _close(y.cpu(), O.ref_w1a16(w, x))
    z = torch.zeros(8, device="cuda")
    assert B.lib.bgemm_w1a16_gemm(None, None, 8, 8, z.data_ptr(), 8, 1, z.data_ptr(), 3, 0, None, 0) == -1
    assert B.lib.bgemm_w1a16_gemm(None, z.data_ptr(), 8, 8, z.data_ptr(), 8, 1, z.data_ptr(), 0, 0, None, 0) == -4     # int32 output is not offered
    assert B.lib.bgemm_w1a16_gemm(None, z.data_ptr(), 8, 8, z.data_ptr(), 4, 1, z.data_ptr(), 3, 0, None, 0) == -2     # row pitch below K
    assert B.lib.bgemm_w1a16_gemm(None, z.data_ptr(), 8, 200000, z.data_ptr(), 200000, 1, z.data_ptr(), 3, 0, None, 0) == -6
