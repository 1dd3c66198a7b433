"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every declared symbol,
refuses bad arguments before touching the device, and its host twins compute the documented formats."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle as O

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "bgemm-cuda_b200" / "libbgemm_b200.so"


@pytest.fixture(scope="module")
def lib():
    if not LIB.exists():
        import subprocess
        subprocess.run(["make", "-C", str(LIB.parent), "-j4", "libbgemm_b200.so"], check=True, capture_output=True)
    return ctypes.CDLL(str(LIB))


def declared_functions():
    text = (ROOT / "include" / "bgemm_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bgemm_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/bgemm_b200.h but not exported"


def test_geometry_helpers(lib):
    lib.bgemm_plane_bytes.restype = ctypes.c_size_t
    lib.bgemm_plane_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
    lib.bgemm_act_ld.restype = ctypes.c_int64
    lib.bgemm_act_ld.argtypes = [ctypes.c_int64]
    for M, K in [(1, 1), (128, 256), (129, 257), (4096, 4096), (28672, 8192), (10, 4096)]:
        assert lib.bgemm_plane_bytes(M, K) == O.plane_bytes(M, K)
        assert lib.bgemm_act_ld(K) == O.act_ld(K)
    assert lib.bgemm_plane_bytes(0, 5) == 0
    lib.bgemm_status_string.restype = ctypes.c_char_p
    assert lib.bgemm_status_string(0) == b"ok"
    assert lib.bgemm_version() >= 100


def test_arguments_are_validated_before_any_launch(lib):
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.bgemm_pack_weights.argtypes = [vp, vp, ci, i64, i64, i64, ci, vp, vp, vp, i64, i64]
    lib.bgemm_gemm.argtypes = [vp, vp, i64, i64, vp, vp, i64, ci, vp, ci, ci, vp, ci, vp, ctypes.c_size_t, i64]
    lib.bgemm_linear_forward.argtypes = [vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp, ci, vp, ctypes.c_size_t]
    lib.bgemm_prepare_acts.argtypes = [vp, vp, ci, i64, i64, i64, ci, ci, vp, vp, i64, i64]
    fake = 0x1000          # never dereferenced: every call below must fail validation first
    assert lib.bgemm_pack_weights(None, None, 0, 4, 4, 4, 0, fake, None, None, 1, 0) == -1
    assert lib.bgemm_pack_weights(None, fake, 7, 4, 4, 4, 0, fake, None, None, 1, 0) == -4
    assert lib.bgemm_pack_weights(None, fake, 0, 4, 4, 4, 9, fake, None, None, 1, 0) == -4
    assert lib.bgemm_pack_weights(None, fake, 0, 4, 8, 4, 0, fake, None, None, 1, 0) == -2      # ld < K
    assert lib.bgemm_pack_weights(None, fake, 0, 4, 4, 4, 0, fake + 4, None, None, 1, 0) == -3  # plane alignment
    assert lib.bgemm_prepare_acts(None, fake, 0, 4, 4, 4, 5, 0, fake, fake, 1, 0) == -4
    assert lib.bgemm_gemm(None, fake, 4, 4, fake, fake, 4, 9, fake, 0, 0, None, 1, None, 0, 1) == -4
    assert lib.bgemm_gemm(None, fake, 4, 4, fake, fake, 4, 1, fake, 2, 0, None, 1, None, 0, 1) == -1   # scaled without alpha
    assert lib.bgemm_gemm(None, fake, 4, 8192, fake, fake, 4, 1, fake, 0, 0, None, 16, None, 0, 1) == -5  # wide split-K without workspace
    assert lib.bgemm_gemm(None, fake, 0, 4, fake, fake, 4, 1, fake, 0, 0, None, 1, None, 0, 1) == -2
    assert lib.bgemm_linear_forward(None, fake, fake, fake, 4, 4, 4, 1, 1, 0, None, 1, None, 0) == -5
    assert lib.bgemm_linear_forward(None, None, fake, fake, 4, 4, 4, 1, 1, 0, None, 1, fake, 1 << 20) == -1


def test_a_refused_call_enqueues_nothing(lib):
    """Every argument error is found before the first launch or memset: the launch counter does not move, also for
    errors that only the last stage of a composite entry point (pack, prepare, GEMM) would notice."""
    vp, i64, ci, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    lib.bgemm_linear_forward.argtypes = [vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, vp, ci, vp, sz]
    lib.bgemm_gemm_to_acts.argtypes = [vp, vp, i64, i64, vp, vp, i64, ci, vp, ci, vp, vp, ci, vp, sz, i64]
    lib.bgemm_gemm.argtypes = [vp, vp, i64, i64, vp, vp, i64, ci, vp, ci, ci, vp, ci, vp, sz, i64]
    lib.bgemm_launch_count.restype = ctypes.c_uint64
    fake, big = 0x10000, 1 << 30
    before = lib.bgemm_launch_count()
    assert lib.bgemm_linear_forward(None, fake, fake, fake, 64, 8, 256, 1, 7, 0, None, 1, fake, big) == -4      # out_kind
    assert lib.bgemm_linear_forward(None, fake, fake, fake, 64, 8, 256, 1, 1, 3, None, 1, fake, big) == -4      # out_layout
    assert lib.bgemm_linear_forward(None, fake, fake, fake, 64, 8, 256, 1, 2, 0, None, 1, fake, big) == -1      # scaled, no alpha
    assert lib.bgemm_linear_forward(None, fake, fake, fake + 2, 64, 8, 256, 1, 0, 0, None, 1, fake, big) == -3  # int32 out misaligned
    assert lib.bgemm_linear_forward(None, fake, fake, fake, 64, 8, 256, 1, 1, 0, None, 1, fake + 8, big) == -3  # workspace misaligned
    assert lib.bgemm_gemm_to_acts(None, fake, 64, 8192, fake, fake, 8, 1, None, 0, fake, fake, 16, None, 0, 1) == -5   # needs a workspace
    lib.bgemm_gemm_to_acts_ex.argtypes = [vp, vp, i64, i64, vp, vp, i64, ci, vp, ci, vp, vp, ci, vp, sz, i64, ci]
    assert lib.bgemm_gemm_to_acts_ex(None, fake, 64, 8192, fake, fake, 8, 1, None, 0, fake, fake, 1, None, 0, 1, 8) == -4     # unknown flag
    assert lib.bgemm_gemm_to_acts_ex(None, fake, 64, 8192, fake, fake, 8, 1, None, 0, fake, fake, 16, None, 0, 1, 4) == -5    # needs a workspace
    assert lib.bgemm_gemm_to_acts(None, fake, 64, 8192, fake, fake, 8, 1, None, 0, fake, fake, 16, fake + 16, big, 1) == -3
    # general int8 activations on narrow tiles beyond the exact range
    assert lib.bgemm_gemm(None, fake, 128, 70000, fake, fake, 16, 4, fake, 0, 0, None, 1, None, 0, 1) == -6
    # flags of bgemm_gemm_ex: unknown bits; a balance workspace that a wide problem would use but that is missing, too small
    # or misaligned (2 = BGEMM_FLAG_BALANCE_WORKSPACE)
    lib.bgemm_gemm_ex.argtypes = [vp, vp, i64, i64, vp, vp, i64, ci, vp, ci, ci, vp, ci, vp, sz, i64, ci]
    lib.bgemm_gemm_balance_workspace_bytes.restype = sz
    lib.bgemm_gemm_balance_workspace_bytes.argtypes = [i64, i64, i64, ci, i64]
    assert lib.bgemm_gemm_ex(None, fake, 128, 512, fake, fake, 32, 1, fake, 0, 0, None, 1, None, 0, 1, 4) == -4
    want = lib.bgemm_gemm_balance_workspace_bytes(28672, 1024, 8192, 0, 1)
    assert want > 65536 and lib.bgemm_gemm_balance_workspace_bytes(28672, 128, 8192, 0, 1) == 0
    assert lib.bgemm_gemm_ex(None, fake, 28672, 8192, fake, fake, 1024, 3, fake, 1, 0, None, 0, None, 0, 1, 2) == -5
    assert lib.bgemm_gemm_ex(None, fake, 28672, 8192, fake, fake, 1024, 3, fake, 1, 0, None, 0, fake, want - 1, 1, 2) == -5
    assert lib.bgemm_gemm_ex(None, fake, 28672, 8192, fake, fake, 1024, 3, fake, 1, 0, None, 0, fake + 16, want, 1, 2) == -3
    assert lib.bgemm_launch_count() == before


def test_bundle_header_round_trip(lib):
    vp, i64, ci, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    lib.bgemm_bundle_bytes.restype = sz
    lib.bgemm_bundle_bytes.argtypes = [i64, i64]
    lib.bgemm_bundle_header_host.argtypes = [vp, i64, i64, ci]
    lib.bgemm_bundle_parse_host.argtypes = [vp, sz, vp, vp, vp, vp, vp, vp]
    total = lib.bgemm_bundle_bytes(300, 1000)
    assert total >= 256 + O.plane_bytes(300, 1000) + 300 * 6 and total % 256 == 0
    assert lib.bgemm_bundle_bytes(0, 5) == 0
    head = np.zeros(64, dtype=np.uint8)
    assert lib.bgemm_bundle_header_host(head.ctypes.data, 300, 1000, 1) == 0
    assert head[:4].tobytes() == b"BGPK" and int(head[4:8].view(np.uint32)[0]) == 1
    M, K, po = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_size_t()
    mode = ctypes.c_int()
    assert lib.bgemm_bundle_parse_host(head.ctypes.data, total, ctypes.byref(M), ctypes.byref(K), ctypes.byref(mode), ctypes.byref(po), None, None) == 0
    assert (M.value, K.value, mode.value, po.value) == (300, 1000, 1, 256)
    assert lib.bgemm_bundle_parse_host(head.ctypes.data, total - 1, None, None, None, None, None, None) == -2     # buffer too short
    head[4] = 9
    assert lib.bgemm_bundle_parse_host(head.ctypes.data, total, None, None, None, None, None, None) == -6         # other layout version
    assert lib.bgemm_bundle_header_host(head.ctypes.data, 300, 1000, 7) == -4


def test_workspace_queries(lib):
    i64, ci = ctypes.c_int64, ctypes.c_int
    lib.bgemm_gemm_workspace_bytes.restype = ctypes.c_size_t
    lib.bgemm_gemm_workspace_bytes.argtypes = [i64, i64, i64, ci, i64]
    lib.bgemm_linear_workspace_bytes.restype = ctypes.c_size_t
    lib.bgemm_linear_workspace_bytes.argtypes = [i64, i64, i64, ci]
    lib.bgemm_gemm_auto_split_k.argtypes = [i64, i64, i64, i64]
    assert lib.bgemm_gemm_workspace_bytes(4096, 64, 4096, 1, 1) == 0
    assert lib.bgemm_gemm_workspace_bytes(4096, 64, 4096, 8, 1) == 0          # up to 8 partitions reduce on chip
    need = lib.bgemm_gemm_workspace_bytes(4096, 64, 4096, 16, 1)
    assert need >= 32 * 16 * 64 * 128 * 4
    assert lib.bgemm_linear_workspace_bytes(4096, 64, 4096, 1) >= O.plane_bytes(4096, 4096) + 64 * 4096
    s = lib.bgemm_gemm_auto_split_k(4096, 64, 4096, 1)
    assert 1 <= s <= 8
    assert lib.bgemm_gemm_auto_split_k(28672, 4096, 8192, 1) == 1


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_host_prepack_twin_matches_layout_definition(lib, mode):
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.bgemm_pack_weights_host.argtypes = [vp, ci, i64, i64, i64, ci, vp, vp, vp]
    g = O._gen(mode)
    M, K = 130, 520
    w = torch.randint(-2, 3, (M, K), generator=g).to(torch.float16)
    w[0, 0] = -0.0
    ref_plane, ref_pop = O.np_pack_weights(w, mode)
    plane = np.zeros(O.plane_bytes(M, K), dtype=np.uint8)
    pop = np.zeros(M, dtype=np.int32)
    alpha = np.zeros(M, dtype=np.float16)
    assert lib.bgemm_pack_weights_host(w.data_ptr(), 0, M, K, K, mode, plane.ctypes.data, pop.ctypes.data, alpha.ctypes.data) == 0
    assert np.array_equal(plane, ref_plane) and np.array_equal(pop, ref_pop)
    assert np.array_equal(alpha.view(np.uint16), O.c_rowmeanabs_f16(w).view(np.uint16))


def test_host_rowmajor_prepack_matches_reference_words(lib):
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.bgemm_pack_rowmajor_msb_host.argtypes = [vp, ci, i64, i64, i64, vp]
    gold = np.load(ROOT / "tests" / "golden" / "reference_golden.npz")
    w = torch.from_numpy(gold["prepack_w_f16bits"].view(np.float16).copy())
    out = np.zeros(gold["prepack_words"].shape, dtype=np.uint32)
    assert lib.bgemm_pack_rowmajor_msb_host(w.data_ptr(), 0, w.shape[0], w.shape[1], w.shape[1], out.ctypes.data) == 0
    assert np.array_equal(out, gold["prepack_words"])
    for dt, code in [(torch.float32, 2), (torch.bfloat16, 1)]:
        w2 = w.to(dt)
        out2 = np.zeros_like(out)
        assert lib.bgemm_pack_rowmajor_msb_host(w2.data_ptr(), code, w.shape[0], w.shape[1], w.shape[1], out2.ctypes.data) == 0
        assert np.array_equal(out2, out)


def test_extension_module_surface():
    """`lowbit_kernel` keeps the reference's export names and refuses CPU tensors for GPU ops."""
    import lowbit_kernel

    for name in ["bgemm_linear_forward_cuda", "weight_prepacking_cpu", "linear_forward_cuda", "weight_dequant_cpu"]:
        assert hasattr(lowbit_kernel, name)            # lowbit_kernel/csrc/pybind.cpp:9-12
    with pytest.raises(TypeError):
        lowbit_kernel.linear_forward_cuda()
    with pytest.raises(RuntimeError, match="CUDA tensors required"):
        lowbit_kernel.bgemm_linear_forward_cuda(torch.zeros(32, 128).half(), torch.zeros(32, 128).half(), 1, 1)
    w = torch.randn(70, 300, generator=O._gen(1)).half()
    bundle = lowbit_kernel.weight_prepacking_cpu(w)                      # header + plane + rowpop + alpha in one tensor
    plane, alpha, rowpop, M, K, wbit = lowbit_kernel.unpack_bundle(bundle)
    assert (M, K, wbit) == (70, 300, 0) and lowbit_kernel.LAYOUT_VERSION == 1
    ref_plane, ref_pop = O.np_pack_weights(w, 0)
    assert np.array_equal(plane.numpy(), ref_plane) and np.array_equal(rowpop.numpy(), ref_pop)
    assert np.array_equal(alpha.numpy().view(np.uint16), O.c_rowmeanabs_f16(w).view(np.uint16))
    # a bundle of another layout version, a damaged magic or a truncated buffer is refused
    other = bundle.clone(); other[4] = 2
    with pytest.raises(RuntimeError, match="layout version"):
        lowbit_kernel.unpack_bundle(other)
    bad = bundle.clone(); bad[0] = 0
    with pytest.raises(RuntimeError, match="magic"):
        lowbit_kernel.unpack_bundle(bad)
    with pytest.raises(RuntimeError, match="inconsistent"):
        lowbit_kernel.unpack_bundle(bundle[: bundle.numel() - 256].clone())
    words = lowbit_kernel.binary_matrix_prepacking(torch.randn(8, 128, generator=O._gen(2)).half())
    assert words.shape == (8, 4) and words.dtype == torch.int32
