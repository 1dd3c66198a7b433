"""Two-GPU tests of the row-sharded layer (skipped on a single-GPU box): one process per GPU over NCCL.

  * `ShardedRows` with the C-ABI GEMM as its shard arithmetic and the NCCL all-gather of the [rows_r, N] slabs;
  * `FusedGatherRows`: the all-gather fused into the GEMM epilogue (every rank stores its slab straight into every
    rank's result through peer-mapped memory), twice in a row with different activations.

Both must reproduce the CPU oracle's full [N, M] result bit for bit on every rank. NVLink multicast / NVLS stay off:
the peers exchange data through plain loads and stores only.
"""
import os
import socket

import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, K, Ns, result_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    import torch.distributed as dist

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import bgemm_b200 as B
        from sharded import FusedGatherRows, ShardedRows, make_gpu_shard, row_shards

        cfg = O.config5(M=M, K=K, N=max(Ns) + len(Ns), seed=1005)      # same seed on every rank: replicated inputs
        w, alpha = cfg["w"], cfg["alpha"]
        s, e = row_shards(M, world)[rank]
        plain = ShardedRows(M, make_gpu_shard(w[s:e].to(dev), B.OP_BWTA, alpha[s:e].to(dev), B.OUT_F16_SCALED))
        fused = FusedGatherRows(lambda a, b: w[a:b].to(dev), M, K, max(Ns), B.OP_BWTA, alpha.to(dev))
        for i, N in enumerate(Ns):
            x = cfg["x"][i:i + N]                                       # different activations for every call
            want = O.ref_out(O.ref_acc(w, x, O.OP_BWTA), O.OUT_F16_SCALED, alpha)
            got = plain.forward(x.to(dev), gather=True)
            assert got.shape == (N, M) and torch.equal(got.cpu(), want), f"rank {rank}: NCCL gather differs at N={N}"
            got2 = fused.forward(x.to(dev))
            torch.cuda.synchronize()
            assert got2.shape == (N, M) and torch.equal(got2.cpu(), want), f"rank {rank}: fused gather differs at N={N}"
            dist.barrier()                                              # everybody has read its result before the next call overwrites it
        assert B.lib.bgemm_device_status(1) == 0
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("M,K,Ns", [(1024, 2048, (200, 8, 1)), (4096, 1024, (64, 130))])
def test_row_sharded_layer_on_two_gpus(tmp_path, M, K, Ns):
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), M, K, Ns, str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
