"""CPU tests of the row-sharding plumbing, including a world_size-2 run over gloo."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle as O
from sharded import ShardedRows, row_shards, shard_pitch


def test_row_shards_cover_and_align():
    for M in [1, 10, 128, 129, 4096, 28672, 1000]:
        for ws in [1, 2, 3, 4, 8]:
            sh = row_shards(M, ws)
            assert len(sh) == ws and sh[0][0] == 0 and sh[-1][1] == M
            for (s0, e0), (s1, e1) in zip(sh, sh[1:]):
                assert e0 == s1 and s0 <= e0
            assert all(s % 128 == 0 or s == M for s, _ in sh)
            assert shard_pitch(M, ws) == max(e - s for s, e in sh)
    assert row_shards(28672, 8) == [(i * 3584, (i + 1) * 3584) for i in range(8)]
    with pytest.raises(ValueError):
        row_shards(0, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = O.config2(M=M, K=K, N=N, seed=77)             # same seed on every rank: replicated inputs
        w, x, alpha = cfg["w"], cfg["x"], cfg["alpha"]
        s, e = row_shards(M, world)[rank]

        def compute(xx):                                     # stand-in for the GPU shard arithmetic
            acc = O.ref_acc(w[s:e], xx, O.OP_BWTA)           # [N, rows]
            return O.ref_out(acc, O.OUT_F16_SCALED, alpha[s:e]).t().contiguous()   # [rows, N]

        layer = ShardedRows(M, compute)
        local = layer.forward(x)
        assert local.shape == (e - s, N)
        full = layer.forward(x, gather=True)
        want = O.ref_out(O.ref_acc(w, x, O.OP_BWTA), O.OUT_F16_SCALED, alpha)
        assert full.shape == (N, M) and torch.equal(full, want)
        if rank == 0:
            torch.save(full.clone(), out_path)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [512, 300])        # even shards / ragged last shard
def test_sharded_rows_world_size_2_gloo(tmp_path, M):
    out = tmp_path / "full.pt"
    mp.spawn(_worker, args=(2, _free_port(), M, 24, 256, str(out)), nprocs=2, join=True)
    assert out.exists()


def test_single_rank_needs_no_process_group():
    cfg = O.config1(M=256, K=256, N=8)
    layer = ShardedRows(256, lambda xx: O.ref_acc(cfg["w"], xx, O.OP_XOR).t().contiguous(), rank=0, world_size=1)
    assert torch.equal(layer.forward(cfg["x"], gather=True), O.ref_acc(cfg["w"], cfg["x"], O.OP_XOR))
