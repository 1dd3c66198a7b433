"""The wait-expiry path of the tensor-core kernels, exercised without faulting or hanging anything.

Every wait inside the kernels is bounded; when one runs out the CTA sets an abort flag, drains its copies, waits for the
UMMAs it issued, frees its tensor memory, records which barrier was missed and exits normally. The test hook
bgemm_debug_set_wait_test shortens the budget to 0.1 ms of SM clock and makes the weight producer withhold one
K block, so the unpack warps' wait on that stage runs out. Checked: the launch returns, bgemm_device_status reports
the code of the missed barrier, and the next normal launch is bit-exact again.
"""
import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture()
def B():
    import bgemm_b200

    yield bgemm_b200
    bgemm_b200.lib.bgemm_debug_set_wait_test(0, -1)          # never leave the hook armed


def _case(M, K, N, batch, seed):
    g = O._gen(seed)
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    return O.rand_pm1(shape_w, g), O.rand_ternary(shape_x, g)


@pytest.mark.parametrize("M,K,N,batch,codes", [(128, 4096, 64, 1, range(11, 19)),       # one CTA of the tile-per-CTA kernel
                                               (256, 2048, 128, 160, range(21, 30))])   # persistent kernel, every CTA
def test_withheld_weight_tile_makes_the_wait_run_out_and_the_kernel_return(B, M, K, N, batch, codes):
    w, x = _case(M, K, N, batch, 5)
    ref = O.ref_acc(w, x, O.OP_BWTA)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_TERNARY)
    assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, B.OUT_I32, split_k=1).cpu(), ref)
    assert B.lib.bgemm_device_status(1) == 0
    B.lib.bgemm_debug_set_wait_test(200_000, 5)              # 0.1 ms budget; K block 5 of every CTA never arrives
    B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, B.OUT_I32, split_k=1)
    torch.cuda.synchronize()                                 # the launch ends by itself
    status = B.lib.bgemm_device_status(1)
    assert status in codes, status
    assert B.lib.bgemm_device_status(0) == 0                 # reading with reset cleared the word
    B.lib.bgemm_debug_set_wait_test(0, -1)
    for _ in range(2):                                       # the context is intact: normal launches are exact again
        assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, B.OUT_I32, split_k=1).cpu(), ref)
    assert B.lib.bgemm_device_status(1) == 0
