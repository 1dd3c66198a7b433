"""GPU parity tests at N <= 4. The dispatcher gives a single ternary activation row to the CUDA-core weight-streaming
kernel (gemm_skinny.cu: bit planes + popcount) and the other shapes here to the register-fed streaming kernel
(gemm_stream.cu), falling back to gemm_skinny.cu where that one does not apply (K beyond 65536); tests/test_gpu_stream.py
runs a child process with the register-fed kernel switched off, which keeps the CUDA-core kernel's dp4a path and its
fallback for non-ternary activations covered, and the child process below switches both off to cover the tensor-core
kernels on the same small shapes. Every result is compared bit for bit with the CPU oracle."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
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
    if op == O.OP_BWTA:
        x = O.rand_ternary(shape_x, g)
    else:
        x = torch.randn(shape_x, generator=g).to(torch.float16)
    return w, x


def _check_all_outputs(B, plane, M, K, acts, colsum, op, acc, alpha, batch):
    for layout in (0, 1):
        for kind in (O.OUT_I32, O.OUT_F16, O.OUT_F16_SCALED):
            a = alpha if kind == O.OUT_F16_SCALED else None
            got = B.gemm(plane, M, K, acts, colsum, op, kind, layout, None if a is None else a.cuda(), 0).cpu()
            want = O.ref_out(acc, kind, None if a is None else (a.unsqueeze(-2) if batch > 1 else a))
            if layout == 1:
                want = want.transpose(-1, -2)
            assert torch.equal(got, want), (op, M, K, acts.shape, layout, kind)


@pytest.mark.parametrize("op", [O.OP_XOR, O.OP_BWTA, O.OP_AND, O.OP_ATTN])
@pytest.mark.parametrize("M,K,N,batch", [
    (128, 256, 1, 1), (300, 1000, 3, 1), (4096, 4096, 1, 1), (4096, 4096, 4, 2), (1000, 8192, 2, 3), (513, 4100, 4, 1),
    (64, 128, 1, 5), (37, 1, 2, 1), (2048, 11008, 4, 1), (256, 1024, 3, 170), (8192, 8192, 1, 1), (256, 40000, 2, 1),
    (256, 40000, 4, 1)])
def test_few_activation_rows(B, op, M, K, N, batch):
    g = O._gen(7 * M + K + N + batch)
    w, x = _inputs(op, batch, M, K, N, g)
    acc = O.ref_acc(w, x, op)
    alpha = (0.01 + 0.09 * torch.rand((batch, M) if batch > 1 else (M,), generator=g)).to(torch.float16)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[op])
    _check_all_outputs(B, plane, M, K, acts, colsum, op, acc, alpha, batch)
    assert B.lib.bgemm_device_status(1) == 0


@pytest.mark.parametrize("op_name", ["BWTA", "W1A8"])
@pytest.mark.parametrize("M,K,N,batch", [(256, 512, 1, 1), (1000, 4096, 2, 2), (300, 2304, 3, 1), (4096, 2048, 4, 1), (130, 300, 4, 3),
                                         (512, 11008, 4, 1)])
def test_int8_activations_at_few_rows(B, op_name, M, K, N, batch):
    """General int8 activations: op BWTA sends N = 3, 4 to the streaming kernel, which finds that they are not ternary
    and takes its dp4a route; op W1A8 keeps those N on the tensor-core kernel. Both must return sum_k sign(w) x."""
    op = getattr(B, "OP_" + op_name)
    g = O._gen(M + 3 * K + N)
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = torch.randn(shape_w, generator=g).to(torch.float16)
    x = torch.randint(-128, 128, shape_x, generator=g, dtype=torch.int8)
    acc = (x.to(torch.float64) @ O.map_weight(w, O.OP_BWTA).to(torch.float64).transpose(-1, -2)).to(torch.int32)
    alpha = (0.01 + 0.09 * torch.rand((batch, M) if batch > 1 else (M,), generator=g)).to(torch.float16)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_INT8)
    _check_all_outputs(B, plane, M, K, acts, colsum, op, acc, alpha, batch)
    assert B.lib.bgemm_device_status(1) == 0


def test_one_stray_value_leaves_the_popcount_route(B):
    """A single activation outside {-1, 0, +1}, in the last column of the last row, must switch the whole launch to
    exact int8 arithmetic."""
    M, K, N = 384, 3000, 4
    g = O._gen(99)
    w = torch.randn(M, K, generator=g).to(torch.float16)
    x = O.rand_ternary((N, K), g).to(torch.int8)
    x[N - 1, K - 1] = 2
    want = (x.to(torch.float64) @ O.map_weight(w, O.OP_BWTA).to(torch.float64).t()).to(torch.int32)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_INT8)
    assert torch.equal(B.gemm(plane, M, K, acts, colsum, B.OP_BWTA, O.OUT_I32, 0, None, 0).cpu(), want)


def test_streaming_kernel_under_graph_replay(B):
    M, K, N = 4096, 4096, 1
    g = O._gen(5)
    w, x = _inputs(O.OP_BWTA, 1, M, K, N, g)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_TERNARY)
    out = torch.empty((N, M), dtype=torch.int32, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, 0, None, 0, out=out)
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for _ in range(4):
                B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, O.OUT_I32, 0, None, 0, out=out)
        out.zero_()
        for _ in range(3):
            graph.replay()
        st.synchronize()
    assert torch.equal(out.cpu(), O.ref_acc(w, x, O.OP_BWTA))


_TENSOR_PATH_SNIPPET = r"""
import sys
sys.path[:0] = [r"%(root)s/bgemm-cuda_b200", r"%(root)s/oracle"]
import torch
import oracle as O
import bgemm_b200 as B
for (M, K, N, sk) in [(128, 256, 1, 0), (300, 1000, 3, 0), (4096, 4096, 4, 4), (1000, 8192, 2, 16), (256, 8192, 1, 32)]:
    for op in (O.OP_XOR, O.OP_BWTA, O.OP_AND):
        g = O._gen(M + K + N)
        w = torch.randn(M, K, generator=g).to(torch.float16)
        x = O.rand_ternary((N, K), g) if op == O.OP_BWTA else torch.randn(N, K, generator=g).to(torch.float16)
        plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
        acts, colsum = B.prepare_acts(x.cuda(), B.ACT_MODE_OF_OP[op])
        got = B.gemm(plane, M, K, acts, colsum, op, O.OUT_I32, 0, None, sk).cpu()
        assert torch.equal(got, O.ref_acc(w, x, op)), (M, K, N, sk, op)
assert B.lib.bgemm_device_status(1) == 0
print("tensor path ok")
"""


def test_tensor_core_kernels_still_serve_few_rows_when_asked():
    """BGEMM_SKINNY_MAX_N=0 (read once per process, hence the child process) switches the streaming kernel off: the
    same small-N problems then run on the tensor-core kernels, K partitions in clusters and through the workspace
    included."""
    env = dict(os.environ, BGEMM_SKINNY_MAX_N="0")
    r = subprocess.run([sys.executable, "-c", _TENSOR_PATH_SNIPPET % {"root": str(ROOT)}], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "tensor path ok" in r.stdout, r.stdout + r.stderr
