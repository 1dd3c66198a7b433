"""GPU test of bgemm_linear_forward_noalloc, the entry point for callers that cannot hand the library a workspace
(for instance a serving loop that owns all device memory in its own pools, or a C plug-in without access to its
host's allocator). Collected last on purpose: a run that stops at the first failure has then already run every
other test.

The entry point is called through the C ABI and must give, on two calls in a row (of different shapes, so that
the second call finds the first one's leftovers in the shared scratch array), exactly what bgemm_linear_forward
gives with a caller-provided workspace: bit-exact int32 accumulators and identical fp16 outputs (the tolerance
of the other GPU tests, 1e-3 relative, is checked as well).
"""
import ctypes

import pytest
import torch

import oracle as O

pytestmark = pytest.mark.gpu


def _bind(B):
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    B.lib.bgemm_linear_forward_noalloc.argtypes = [vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp]
    B.lib.bgemm_linear_forward_noalloc.restype = ci
    return B.lib.bgemm_linear_forward_noalloc


def _noalloc(B, fn, w, x, op, out_kind, alpha=None):
    M, K = w.shape
    N = x.shape[0]
    out = torch.empty((N, M), dtype=torch.int32 if out_kind == B.OUT_I32 else torch.float16, device="cuda")
    rc = fn(torch.cuda.current_stream().cuda_stream, w.data_ptr(), x.data_ptr(), out.data_ptr(), M, N, K, op, out_kind, B.LAYOUT_NM,
            None if alpha is None else alpha.data_ptr())
    assert rc == 0, B.lib.bgemm_status_string(rc)
    return out


def test_noalloc_entry_point_matches_workspace_entry_point_twice_in_a_row():
    import bgemm_b200 as B

    fn = _bind(B)
    cases = [(O.config2(M=1024, K=2048, N=96, seed=41), O.OP_BWTA),      # first call
             (O.config1(M=384, K=1000, N=33, seed=42), O.OP_XOR)]        # second call: other shape, ragged K and N
    for cfg, op in cases:
        w, x = cfg["w"].cuda(), cfg["x"].cuda()
        alpha = cfg.get("alpha", torch.full((w.shape[0],), 0.5, dtype=torch.float16)).cuda()
        for kind in (B.OUT_I32, B.OUT_F16_SCALED):
            a = alpha if kind == B.OUT_F16_SCALED else None
            got = _noalloc(B, fn, w, x, op, kind, a)
            want = B.linear_forward(w, x, op, out_kind=kind, alpha=a)
            torch.cuda.synchronize()
            if kind == B.OUT_I32:
                assert torch.equal(got, want)
                assert torch.equal(got.cpu(), O.ref_acc(cfg["w"], cfg["x"], op))
            else:
                assert torch.allclose(got.float(), want.float(), rtol=1e-3, atol=0)
                assert torch.equal(got, want)
    assert B.lib.bgemm_device_status(0) == 0


def test_noalloc_rejects_problems_beyond_its_fixed_scratch():
    import bgemm_b200 as B

    fn = _bind(B)
    x = torch.zeros(16, dtype=torch.float16, device="cuda")
    # 8192 x 16384 binary weights alone are 16 MiB packed: over the 8 MiB array -> refused before anything is launched
    rc = fn(None, x.data_ptr(), x.data_ptr(), x.data_ptr(), 8192, 8, 16384, 1, 1, 0, None)
    assert rc == -8 and b"capacity" in B.lib.bgemm_status_string(rc)
    assert fn(None, None, x.data_ptr(), x.data_ptr(), 8, 8, 8, 1, 1, 0, None) == -1
