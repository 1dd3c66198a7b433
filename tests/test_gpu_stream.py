"""GPU parity tests of the weight-streaming kernel for N <= 16 (gemm_stream.cu: register-fed mma.sync int8): every N,
every op, ragged shapes, batches in grid.y, ranges of more groups than a CTA sums at once, general int8 activations,
the static-weights entry point, and replay from a CUDA graph. Every result is compared bit for bit with the CPU oracle.
The kernels behind it (CUDA-core streaming kernel, tensor-memory kernels) keep their coverage through a child process
that switches this one off."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def B():
    import bgemm_b200

    return bgemm_b200


def _inputs(op, batch, M, K, N, g):
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = torch.randn(shape_w, generator=g).to(torch.float16)
    x = O.rand_ternary(shape_x, g) if op == O.OP_BWTA else torch.randn(shape_x, generator=g).to(torch.float16)
    return w, x


def _check(B, w, x, op, batch, layouts=(0, 1), kinds=(O.OUT_I32, O.OUT_F16, O.OUT_F16_SCALED), static=False, acc=None, act_mode=None):
    M, K = w.shape[-2:]
    g = O._gen(M + K)
    alpha = (0.01 + 0.09 * torch.rand((batch, M) if batch > 1 else (M,), generator=g)).to(torch.float16)
    acc = O.ref_acc(w, x, op) if acc is None else acc
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[op] if act_mode is None else act_mode)
    torch.cuda.synchronize()                       # the plane is complete before any later launch: the static-weights promise holds
    for layout in layouts:
        for kind in kinds:
            a = alpha if kind == O.OUT_F16_SCALED else None
            got = B.gemm(plane, M, K, acts, colsum, op, kind, layout, None if a is None else a.cuda(), 0, static_weights=static).cpu()
            want = O.ref_out(acc, kind, None if a is None else (a.unsqueeze(-2) if batch > 1 else a))
            if layout == 1:
                want = want.transpose(-1, -2)
            assert got.shape == want.shape and torch.equal(got, want), (op, M, K, x.shape, layout, kind, int((got != want).sum()))


@pytest.mark.parametrize("N", list(range(1, 17)))
@pytest.mark.parametrize("op", [O.OP_XOR, O.OP_BWTA, O.OP_AND, O.OP_ATTN])
def test_every_n_and_op(B, N, op):
    g = O._gen(31 * N + op)
    w, x = _inputs(op, 1, 640, 1536, N, g)
    _check(B, w, x, op, 1, layouts=(N % 2,), static=bool(N & 2))
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,batch", [
    (128, 256, 5, 1), (300, 1000, 7, 1), (4096, 4096, 8, 1), (4096, 4096, 16, 2), (1000, 8192, 12, 3), (513, 4100, 9, 1),
    (64, 128, 16, 5), (37, 1, 6, 1), (2048, 11008, 8, 1), (256, 1024, 11, 170), (8192, 8192, 16, 1), (28672, 2048, 13, 1),
    (20000, 512, 8, 40), (20000, 768, 3, 40), (1, 300, 16, 1), (33, 65536, 2, 1)])
def test_shapes_batches_and_long_ranges(B, M, K, N, batch):
    """Ragged M / K / N, batches (fewer CTAs per problem, so a CTA walks over several passes of eight groups: the two
    20000-row cases give every CTA ~78 groups), K at the limit of the exact range, both column-tile counts."""
    g = O._gen(7 * M + K + N + batch)
    for op in (O.OP_BWTA, O.OP_XOR):
        w, x = _inputs(op, batch, M, K, N, g)
        _check(B, w, x, op, batch, kinds=(O.OUT_I32, O.OUT_F16_SCALED))
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("M,K,N,batch", [(256, 512, 1, 1), (1000, 4096, 6, 2), (300, 2304, 16, 1), (4096, 2048, 9, 1), (130, 300, 4, 3)])
@pytest.mark.parametrize("op_name", ["BWTA", "W1A8"])
def test_general_int8_activations(B, M, K, N, batch, op_name):
    """Binary weight x int8 activation (all of -128 .. 127): sum_k sign(w) x, exact."""
    g = O._gen(M + 3 * K + N)
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = torch.randn(shape_w, generator=g).to(torch.float16)
    x = torch.randint(-128, 128, shape_x, generator=g, dtype=torch.int8)
    x.view(-1)[:8] = -128                                                # the extreme value in every bit slice of a row
    acc = (x.to(torch.float64) @ O.map_weight(w, O.OP_BWTA).to(torch.float64).transpose(-1, -2)).to(torch.int32)
    _check(B, w, x, getattr(B, "OP_" + op_name), batch, acc=acc, act_mode=B.ACT_INT8, kinds=(O.OUT_I32, O.OUT_F16_SCALED))


def test_extreme_activations_at_the_longest_exact_k(B):
    """All activations -128 against all-negative weights at K = 65536: accumulator 7 of the one-tile variant reaches
    128 * 128 * 65536 / 8 per slice, the int32 result 2**23 -- exact."""
    M, K = 64, 65536
    w = -torch.ones(M, K, dtype=torch.float16)
    for N in (2, 3):
        x = torch.full((N, K), -128, dtype=torch.int8)
        x[N - 1, ::2] = 127
        acc = (x.to(torch.float64) @ O.map_weight(w, O.OP_BWTA).to(torch.float64).t()).to(torch.int32)
        _check(B, w, x, B.OP_W1A8, 1, acc=acc, act_mode=B.ACT_INT8, kinds=(O.OUT_I32,), layouts=(0,))


def test_graph_replay_with_static_weights(B):
    """Back-to-back launches replayed from a CUDA graph, weights fetched ahead of the dependency wait: the output of a
    launch must not depend on what the launch before it was doing."""
    M, K = 4096, 4096
    g = O._gen(5)
    planes, accs, prepared = [], [], []
    for N in (1, 8, 16, 4):
        w, x = _inputs(O.OP_BWTA, 1, M, K, N, g)
        planes.append(B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)[0])
        prepared.append(B.prepare_acts(x.cuda(), B.ACT_TERNARY))
        accs.append(O.ref_acc(w, x, O.OP_BWTA))
    outs = [torch.empty(a.shape, dtype=torch.int32, device="cuda") for a in accs]
    torch.cuda.synchronize()
    st = torch.cuda.Stream()

    def run():
        for pl, (ac, cs), out in zip(planes, prepared, outs):
            B.gemm(pl, M, K, ac, cs, O.OP_BWTA, O.OUT_I32, 0, None, 0, out=out, static_weights=True)

    with torch.cuda.stream(st):
        run()
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for _ in range(3):
                run()
        for o in outs:
            o.zero_()
        for _ in range(3):
            graph.replay()
        st.synchronize()
    for o, a in zip(outs, accs):
        assert torch.equal(o.cpu(), a)
    assert B.lib.bgemm_device_status(1) == 0


_OTHER_KERNELS_SNIPPET = r"""
import sys
sys.path[:0] = [r"%(root)s/bgemm-cuda_b200", r"%(root)s/oracle"]
import torch
import oracle as O
import bgemm_b200 as B
for (M, K, N, sk) in [(128, 256, 1, 0), (300, 1000, 3, 0), (4096, 4096, 4, 4), (1000, 8192, 2, 16), (256, 8192, 1, 32), (640, 2048, 12, 0), (28672, 1024, 16, 0)]:
    for op in (O.OP_XOR, O.OP_BWTA, O.OP_AND):
        g = O._gen(M + K + N)
        w = torch.randn(M, K, generator=g).to(torch.float16)
        x = O.rand_ternary((N, K), g) if op == O.OP_BWTA else torch.randn(N, K, generator=g).to(torch.float16)
        plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
        acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[op])
        got = B.gemm(plane, M, K, acts, colsum, op, O.OUT_I32, 0, None, sk).cpu()
        assert torch.equal(got, O.ref_acc(w, x, op)), (M, K, N, sk, op)
assert B.lib.bgemm_device_status(1) == 0
print("other kernels ok")
"""


@pytest.mark.parametrize("env", [{"BGEMM_STREAM_MAX_N": "0"},                                   # CUDA-core kernel for N <= 4, tensor memory above
                                 {"BGEMM_STREAM_MAX_N": "0", "BGEMM_SKINNY_MAX_N": "0"}])      # tensor-memory kernels for every N
def test_kernels_behind_the_streaming_kernel_still_serve_few_rows(env):
    """The dispatch limits are read once per process, hence the child process."""
    r = subprocess.run([sys.executable, "-c", _OTHER_KERNELS_SNIPPET % {"root": str(ROOT)}], env=dict(os.environ, **env),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "other kernels ok" in r.stdout, r.stdout + r.stderr
