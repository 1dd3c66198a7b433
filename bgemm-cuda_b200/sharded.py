"""Row-sharded binary linear layer: one process per GPU, output rows split across ranks.

The reference has no multi-GPU path. Output rows of a linear layer are independent, so rank r keeps
the packed planes (and scales) of a contiguous block of rows and computes its own [rows_r, N] slab
with the same kernels as the single-GPU path; activations are replicated. There is no data-path
collective unless the caller asks for the full output, in which case the slabs -- emitted row-major
[rows_r, N] so that they concatenate along the row axis -- are all-gathered (NCCL over NVLink on GPUs,
any torch.distributed backend otherwise).

The arithmetic of a shard is injected (`compute`), which keeps this file free of device code: the GPU
product path passes the C-ABI GEMM, CPU tests of the plumbing pass a stand-in.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import torch
import torch.distributed as dist

ROW_ALIGN = 128        # rows per packed tile: shards start on tile boundaries


def row_shards(M: int, world_size: int, align: int = ROW_ALIGN) -> list[tuple[int, int]]:
    """Contiguous [start, end) row ranges, one per rank, starting on multiples of `align`.

    Tiles are dealt out as evenly as possible (the first `tiles % world_size` ranks get one more); ranks
    beyond the number of tiles get an empty range.
    """
    if M < 1 or world_size < 1:
        raise ValueError("M and world_size must be positive")
    tiles = -(-M // align)
    base, extra = divmod(tiles, world_size)
    out, t = [], 0
    for r in range(world_size):
        n = base + (1 if r < extra else 0)
        start, end = min(t * align, M), min((t + n) * align, M)
        out.append((start, end))
        t += n
    return out


def shard_pitch(M: int, world_size: int, align: int = ROW_ALIGN) -> int:
    """Rows each rank contributes to an equal-size all-gather (the largest shard, padded)."""
    return max(e - s for s, e in row_shards(M, world_size, align)) if M > 0 else 0


class ShardedRows:
    """Plumbing of a row-sharded product y[N, M] = f(W[M, K], x[N, K]).

    `compute(x) -> Tensor[rows_local, N]` evaluates this rank's slab. `forward(x)` returns the local slab;
    `forward(x, gather=True)` returns the full [N, M] result on every rank (a transposed view of the
    gathered [M, N] buffer, so no extra copy is made).
    """

    def __init__(self, M: int, compute: Callable[[torch.Tensor], torch.Tensor], group: Optional[dist.ProcessGroup] = None,
                 rank: Optional[int] = None, world_size: Optional[int] = None):
        self.M = M
        self.group = group
        self.world_size = world_size if world_size is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.shards = row_shards(M, self.world_size)
        self.start, self.end = self.shards[self.rank]
        self.pitch = shard_pitch(M, self.world_size)
        self.compute = compute

    @property
    def rows_local(self) -> int:
        return self.end - self.start

    def forward(self, x: torch.Tensor, gather: bool = False) -> torch.Tensor:
        local = self.compute(x)
        if local.shape[0] != self.rows_local:
            raise RuntimeError(f"shard compute returned {local.shape[0]} rows, expected {self.rows_local}")
        if not gather:
            return local
        return self.gather(local)

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        """All-gather [rows_r, N] slabs into the full result and return it as [N, M]."""
        N = local.shape[1]
        if self.world_size == 1:
            return local.t()
        even = all(e - s == self.pitch for s, e in self.shards)
        if even:
            full = torch.empty((self.M, N), dtype=local.dtype, device=local.device)
            dist.all_gather_into_tensor(full, local.contiguous(), group=self.group)
            return full.t()
        padded = torch.zeros((self.pitch, N), dtype=local.dtype, device=local.device)
        padded[: self.rows_local] = local
        buf = torch.empty((self.world_size * self.pitch, N), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(buf, padded, group=self.group)
        parts = [buf[r * self.pitch: r * self.pitch + (e - s)] for r, (s, e) in enumerate(self.shards)]
        return torch.cat(parts, dim=0).t()


def make_gpu_shard(weight_rows: torch.Tensor, op: int, alpha_rows: Optional[torch.Tensor], out_kind: int,
                   act_mode: Optional[int] = None) -> Callable[[torch.Tensor], torch.Tensor]:
    """Shard arithmetic on the GPU: prepack this rank's rows once, then one GEMM per call ([rows, N] out)."""
    import bgemm_b200 as B

    rows, K = weight_rows.shape
    plane, _, _ = B.pack_weights(weight_rows, B.WBIT_OF_OP[op])
    alpha = None if alpha_rows is None else alpha_rows.to(torch.float16).contiguous()
    mode = B.ACT_MODE_OF_OP[op] if act_mode is None else act_mode

    def compute(x: torch.Tensor) -> torch.Tensor:
        acts, colsum = B.prepare_acts(x, mode)
        return B.gemm(plane, rows, K, acts, colsum, op, out_kind, B.LAYOUT_MN, alpha)

    return compute


class FusedGatherRows:
    """Row-sharded layer whose all-gather is fused into the GEMM epilogue (GPUs of one node, NVLink / NVSwitch).

    Every rank owns a full [N_max, M] fp16 result buffer in symmetric memory (torch.distributed._symmetric_memory:
    device memory that every rank of the group maps, used here for allocation and address exchange only). Rank r's
    GEMM stores its [N, rows_r] slab at column start_r of EVERY rank's buffer (bgemm_gemm_multi_out: ordinary 16-byte
    global stores from the epilogue, remote ones over NVLink, no TMA, no multicast), a cross-rank barrier on the stream
    follows, and `forward` returns this rank's buffer, which now holds the whole [N, M] result. The transfer overlaps the
    tensor-core work tile by tile instead of following it as a separate collective.

    Successive calls reuse the buffer: the caller must be done with the previous result before the next forward
    (the leading barrier of `forward` makes sure no peer overwrites a result another rank is still reading only
    together with that rule).
    """

    def __init__(self, weight_rows_of: Callable[[int, int], torch.Tensor], M: int, K: int, n_max: int, op: int,
                 alpha: Optional[torch.Tensor], group: Optional[dist.ProcessGroup] = None):
        import os

        import bgemm_b200 as B
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")      # plain peer mappings only
        self.B, self.M, self.K, self.op, self.n_max = B, M, K, op, n_max
        self.group = group if group is not None else dist.group.WORLD
        self.world_size, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.shards = row_shards(M, self.world_size)
        self.start, self.end = self.shards[self.rank]
        w = weight_rows_of(self.start, self.end)                             # this rank's rows [rows_r, K]
        dev = w.device
        self.plane, _, _ = B.pack_weights(w, B.WBIT_OF_OP[op])
        self.alpha = None if alpha is None else alpha[self.start:self.end].to(torch.float16).contiguous()
        self.full = symm.empty((n_max, M), dtype=torch.float16, device=dev)
        self.handle = symm.rendezvous(self.full, self.group)
        # destination q = rank q's buffer + this rank's first column; the local one first
        order = [self.rank] + [q for q in range(self.world_size) if q != self.rank]
        self.out_ptrs = [int(self.handle.buffer_ptrs[q]) + 2 * self.start for q in order]
        torch.cuda.current_stream(dev).synchronize()                         # weights are static from here on

    @property
    def rows_local(self) -> int:
        return self.end - self.start

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B = self.B
        N = x.shape[0]
        assert N <= self.n_max
        acts, colsum = B.prepare_acts(x, B.ACT_MODE_OF_OP[self.op])
        return self.forward_prepared(acts, colsum)

    def forward_prepared(self, acts: torch.Tensor, colsum: torch.Tensor) -> torch.Tensor:
        B = self.B
        N = acts.shape[0]
        self.handle.barrier(channel=0)            # every rank is done reading the previous result
        if self.rows_local > 0:
            B.gemm_multi_out(self.plane, self.rows_local, self.K, acts, colsum, self.op, self.out_ptrs, self.M,
                             B.OUT_F16_SCALED if self.alpha is not None else B.OUT_F16, B.LAYOUT_NM, self.alpha, 0, static_weights=True)
        self.handle.barrier(channel=1)            # every rank's slab has landed everywhere
        return self.full[:N]


def shard_sizes(shards: Sequence[tuple[int, int]]) -> list[int]:
    return [e - s for s, e in shards]
