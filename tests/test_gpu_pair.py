"""GPU parity tests of the CTA-pair kernel (gemm_pair.cu: tcgen05.mma.cta_group::2, 256 x 256 tiles, wide activation
matrices): whole-tile and exact work splits (tiles accumulated in parts by several clusters and summed through the
workspace, including tiles cut into many parts), both output layouts, every output kind, every op, ragged M / N / K,
batches, general int8 activations (accumulators beyond 16 bits take the int32 path of its epilogue), several
destinations, repeated calls on one workspace, and replay from a CUDA graph. Every result is compared bit for bit with
the CPU oracle. The module switches the dispatcher to "the pair kernel wherever the shape allows it"
(bgemm_debug_set_pair_kernel), since its own rule keeps short K and few tiles on other kernels; a child process does the
same through the environment."""
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

    bgemm_b200.lib.bgemm_debug_set_pair_kernel(1)
    yield bgemm_b200
    bgemm_b200.lib.bgemm_debug_set_pair_kernel(-1)           # back to the library's own rule


def _inputs(op, batch, M, K, N, g, wide=False):
    shape_w, shape_x = ((batch, M, K), (batch, N, K)) if batch > 1 else ((M, K), (N, K))
    w = torch.randn(shape_w, generator=g).to(torch.float16)
    if wide:
        x = torch.randint(-128, 128, shape_x, generator=g, dtype=torch.int8)
    elif op == O.OP_BWTA:
        x = O.rand_ternary(shape_x, g)
    else:
        x = torch.randn(shape_x, generator=g).to(torch.float16)
    return w, x


def _reference(w, x, op, wide):
    if not wide:
        return O.ref_acc(w, x, op)
    sw = torch.where(torch.signbit(w.float()), -1.0, 1.0)
    return torch.matmul(x.double(), sw.double().transpose(-1, -2)).to(torch.int32)      # sum_k sign(w) * x, exact


def _run(B, M, K, N, op=O.OP_BWTA, batch=1, layouts=(0, 1), kinds=(O.OUT_I32, O.OUT_F16_SCALED), wide=False, use_ws=True, seed=0):
    g = O._gen(13 * M + 7 * K + N + batch + seed)
    w, x = _inputs(op, batch, M, K, N, g, wide)
    acc = _reference(w, x, op, wide)
    alpha = (0.01 + 0.09 * torch.rand((batch, M) if batch > 1 else (M,), generator=g)).to(torch.float16)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[op])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_INT8 if wide else B.ACT_MODE_OF_OP[op])
    for layout in layouts:
        for kind in kinds:
            a = alpha if kind == O.OUT_F16_SCALED else None
            want = O.ref_out(acc, kind, None if a is None else (a.unsqueeze(-2) if batch > 1 else a))
            if layout == 1:
                want = want.transpose(-1, -2)
            for rep in range(2):                    # the second call finds the workspace as the first one left it
                got = B.gemm(plane, M, K, acts, colsum, op, kind, layout, None if a is None else a.cuda(), 0, balance=use_ws).cpu()
                assert got.shape == want.shape and torch.equal(got, want), (op, M, K, N, batch, layout, kind, rep, int((got != want).sum()))
    assert B.lib.bgemm_device_status(1) == 0


def test_pair_kernel_is_what_runs(B):
    """Forced, every shape the kernel can take reports its workspace; by the library's own rule only long K, three or
    more tiles across N without a mostly empty last one, and enough tiles for every SM pair do."""
    ws = B.lib.bgemm_gemm_balance_workspace_bytes
    assert ws(2560, 2048, 1024, 0, 1) > 0
    assert ws(2560, 128, 1024, 0, 1) == 0            # narrow: other kernels
    assert ws(2432, 2048, 1024, 0, 1) == 0           # odd number of 128-row tiles
    B.lib.bgemm_debug_set_pair_kernel(-1)
    try:
        assert ws(28672, 1024, 8192, 0, 1) > 0 and ws(7168, 1024, 8192, 0, 1) > 0 and ws(28672, 768, 2560, 0, 1) > 0
        assert ws(2560, 2048, 1024, 0, 1) == 0       # 4 K blocks
        assert ws(28672, 512, 8192, 0, 1) == 0       # two tiles across N
        assert ws(28672, 640, 8192, 0, 1) == 0       # the third tile would be half empty
        assert ws(3584, 1024, 8192, 0, 1) == 0       # 56 tiles on 74 SM pairs
    finally:
        B.lib.bgemm_debug_set_pair_kernel(1)


@pytest.mark.parametrize("M,K,N", [(2560, 1024, 2048),      # 80 tiles x 4 K blocks on 74 pairs: every tile boundary is cut
                                   (2560, 1280, 2048),      # odd number of K blocks per tile
                                   (9472, 512, 512),        # exactly one tile per pair: nothing to cut
                                   (2500, 2048, 2000),      # ragged rows and columns
                                   (19200, 300, 256)])      # ragged K, one tile across N
def test_shapes_exact_and_whole_tile_split(B, M, K, N):
    _run(B, M, K, N)
    _run(B, M, K, N, use_ws=False, layouts=(0,), kinds=(O.OUT_I32,))


@pytest.mark.parametrize("op", [O.OP_XOR, O.OP_AND, O.OP_ATTN])
def test_ops(B, op):
    _run(B, 2560, 1024, 2048, op=op, kinds=(O.OUT_I32, O.OUT_F16))


def test_batches(B):
    _run(B, 1280, 512, 1280, batch=3)               # 5 pairs x 5 tiles x 3 problems
    _run(B, 768, 1024, 300, batch=13, layouts=(0,))  # ragged N inside every problem


def test_general_int8_activations_leave_16_bits(B):
    """|sum| reaches 127 K: the epilogue's int16 staging does not fit and it converts from tensor memory instead; with
    the exact split the parts are summed on that path too."""
    _run(B, 2560, 2048, 2048, wide=True, kinds=(O.OUT_I32,))
    _run(B, 2560, 2048, 2048, wide=True, kinds=(O.OUT_I32,), use_ws=False, layouts=(1,))


def test_several_destinations_with_pitch(B):
    M, K, N, lead = 2560, 512, 2048, 2560 + 512
    g = O._gen(99)
    w, x = _inputs(O.OP_BWTA, 1, M, K, N, g)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    want = O.ref_out(O.ref_acc(w, x, O.OP_BWTA), O.OUT_F16_SCALED, alpha)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_TERNARY)
    outs = [torch.zeros((N, lead), dtype=torch.float16, device="cuda") for _ in range(3)]
    B.gemm_multi_out(plane, M, K, acts, colsum, O.OP_BWTA, [o.data_ptr() + 2 * 256 for o in outs], lead, B.OUT_F16_SCALED, B.LAYOUT_NM, alpha.cuda())
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o[:, 256:256 + M].cpu(), want)
        assert not o[:, :256].any() and not o[:, 256 + M:].any()
    assert B.lib.bgemm_device_status(1) == 0


def test_graph_replay(B):
    M, K, N = 2560, 1024, 2048
    g = O._gen(5)
    w, x = _inputs(O.OP_BWTA, 1, M, K, N, g)
    want = O.ref_out(O.ref_acc(w, x, O.OP_BWTA), O.OUT_I32, None)
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_OF_OP[O.OP_BWTA])
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_TERNARY)
    out = torch.zeros((N, M), dtype=torch.int32, device="cuda")
    ws = torch.zeros(B.lib.bgemm_gemm_balance_workspace_bytes(M, N, K, 0, 1), dtype=torch.uint8, device="cuda")
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, out=out, ws=ws)
        st.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=st):
            for _ in range(3):
                B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, out=out, ws=ws)
        for _ in range(3):
            out.zero_()
            graph.replay()
            st.synchronize()
            assert torch.equal(out.cpu(), want)
    assert not ws[:65536].any()                     # the flags are back at zero
    assert B.lib.bgemm_device_status(1) == 0


def test_forced_on_small_shapes_and_many_parts():
    """BGEMM_PAIR=1 sends every eligible shape to the pair kernel, however few tiles it has: a 512 x 40960 x 256 problem
    is two tiles of 160 K blocks cut into ~37 parts each."""
    code = r"""
import sys
sys.path[:0] = [r"%s", r"%s"]
import torch, oracle as O, bgemm_b200 as B
for (M, K, N, layout, kind) in [(256, 512, 256, 0, O.OUT_I32), (512, 40960, 256, 0, O.OUT_I32), (512, 40960, 256, 1, O.OUT_F16),
                                (768, 2560, 520, 0, O.OUT_F16_SCALED), (2048, 8192, 768, 1, O.OUT_F16_SCALED)]:
    g = O._gen(M + K + N)
    w = torch.randn((M, K), generator=g).to(torch.float16); x = O.rand_ternary((N, K), g)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    want = O.ref_out(O.ref_acc(w, x, O.OP_BWTA), kind, alpha if kind == O.OUT_F16_SCALED else None)
    want = want.t() if layout == 1 else want
    plane, _, _ = B.pack_weights(w.cuda(), B.WBIT_NEGATIVE)
    acts, colsum = B.prepare_acts(x.cuda(), B.ACT_TERNARY)
    for rep in range(2):
        got = B.gemm(plane, M, K, acts, colsum, O.OP_BWTA, kind, layout, alpha.cuda() if kind == O.OUT_F16_SCALED else None, 0).cpu()
        assert torch.equal(got, want), (M, K, N, layout, kind, rep, int((got != want).sum()))
assert B.lib.bgemm_device_status(1) == 0
print("ok")
""" % (ROOT / "bgemm-cuda_b200", ROOT / "oracle")
    env = dict(os.environ, BGEMM_PAIR="1")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
