"""ctypes binding of libbgemm_b200.so for callers that hold torch CUDA tensors.

PyTorch is used for device memory and streams only; every computation is a call through the C ABI
declared in ``include/bgemm_b200.h``. There is no CPU or eager fallback: if the shared library is
missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_DIR = Path(__file__).resolve().parent
_LIB_PATH = Path(os.environ.get("BGEMM_B200_LIB", _DIR / "libbgemm_b200.so"))
if not _LIB_PATH.exists():
    raise ImportError(
        f"{_LIB_PATH} not found: build it with `make -C {_DIR}` (nvcc, sm_100a). "
        "This package has no fallback path."
    )
lib = ctypes.CDLL(str(_LIB_PATH))

# ---- constants of include/bgemm_b200.h ----
DT_F16, DT_BF16, DT_F32, DT_I8 = 0, 1, 2, 3
OP_AND, OP_XOR, OP_ATTN, OP_BWTA, OP_W1A8 = 0, 1, 2, 3, 4
WBIT_NEGATIVE, WBIT_NONNEGATIVE, WBIT_NONZERO, WBIT_NEGATIVE_NZ = 0, 1, 2, 3
ACT_SIGN, ACT_TERNARY, ACT_NEG01, ACT_INT8 = 0, 1, 2, 3
OUT_I32, OUT_F16, OUT_F16_SCALED, OUT_F32 = 0, 1, 2, 3
LAYOUT_NM, LAYOUT_MN = 0, 1
ACT_MODE_OF_OP = {OP_AND: ACT_NEG01, OP_XOR: ACT_SIGN, OP_ATTN: ACT_SIGN, OP_BWTA: ACT_TERNARY, OP_W1A8: ACT_INT8}
WBIT_OF_OP = {OP_AND: WBIT_NEGATIVE, OP_XOR: WBIT_NEGATIVE, OP_ATTN: WBIT_NONNEGATIVE, OP_BWTA: WBIT_NEGATIVE, OP_W1A8: WBIT_NEGATIVE}

_i64, _int, _vp, _sz = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t
lib.bgemm_plane_bytes.restype = _sz
lib.bgemm_plane_bytes.argtypes = [_i64, _i64]
lib.bgemm_act_ld.restype = _i64
lib.bgemm_act_ld.argtypes = [_i64]
lib.bgemm_status_string.restype = ctypes.c_char_p
lib.bgemm_status_string.argtypes = [_int]
lib.bgemm_version.restype = _int
lib.bgemm_launch_count.restype = ctypes.c_uint64
lib.bgemm_pack_rowmajor_msb.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _vp]
lib.bgemm_pack_rowmajor_msb_host.argtypes = [_vp, _int, _i64, _i64, _i64, _vp]
lib.bgemm_retile_rowmajor_msb.argtypes = [_vp, _vp, _i64, _i64, _int, _vp]
lib.bgemm_pack_weights.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _int, _vp, _vp, _vp, _i64, _i64]
lib.bgemm_pack_weights_host.argtypes = [_vp, _int, _i64, _i64, _i64, _int, _vp, _vp, _vp]
lib.bgemm_prepare_acts.argtypes = [_vp, _vp, _int, _i64, _i64, _i64, _int, _int, _vp, _vp, _i64, _i64]
lib.bgemm_gemm.argtypes = [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _int, _vp, _int, _int, _vp, _int, _vp, _sz, _i64]
lib.bgemm_gemm_static_weights.argtypes = lib.bgemm_gemm.argtypes
lib.bgemm_gemm_ex.argtypes = lib.bgemm_gemm.argtypes + [_int]
FLAG_STATIC_WEIGHTS, FLAG_BALANCE_WORKSPACE = 1, 2
lib.bgemm_gemm_multi_out.argtypes = [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _int, _vp, _int, _i64, _int, _int, _vp, _int, _vp, _sz, _int]
lib.bgemm_w1a16_gemm.argtypes = [_vp, _vp, _i64, _i64, _vp, _i64, _i64, _vp, _int, _int, _vp, _int]
lib.bgemm_gemm_to_acts.argtypes = [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _int, _vp, _int, _vp, _vp, _int, _vp, _sz, _i64]
lib.bgemm_gemm_to_acts_ex.argtypes = [_vp, _vp, _i64, _i64, _vp, _vp, _i64, _int, _vp, _int, _vp, _vp, _int, _vp, _sz, _i64, _int]
FLAG_SUMS_ZEROED = 4
lib.bgemm_gemm_workspace_bytes.restype = _sz
lib.bgemm_gemm_workspace_bytes.argtypes = [_i64, _i64, _i64, _int, _i64]
lib.bgemm_debug_set_pair_kernel.restype = None
lib.bgemm_debug_set_pair_kernel.argtypes = [_int]
lib.bgemm_gemm_balance_workspace_bytes.restype = _sz
lib.bgemm_gemm_balance_workspace_bytes.argtypes = [_i64, _i64, _i64, _int, _i64]
lib.bgemm_gemm_auto_split_k.argtypes = [_i64, _i64, _i64, _i64]
lib.bgemm_linear_forward.argtypes = [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _int, _int, _vp, _int, _vp, _sz]
lib.bgemm_linear_workspace_bytes.restype = _sz
lib.bgemm_linear_workspace_bytes.argtypes = [_i64, _i64, _i64, _int]
lib.bgemm_device_status.restype = _int
lib.bgemm_device_status.argtypes = [_int]
lib.bgemm_debug_set_wait_test.restype = None
lib.bgemm_debug_set_wait_test.argtypes = [_i64, _int]


class BgemmError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: status {status}: {lib.bgemm_status_string(status).decode()}")


def check(status: int, where: str) -> None:
    if status != 0:
        raise BgemmError(status, where)


_DT = {torch.float16: DT_F16, torch.bfloat16: DT_BF16, torch.float32: DT_F32, torch.int8: DT_I8}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported source dtype {t.dtype}; use float16, bfloat16, float32 or int8") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


def plane_bytes(M: int, K: int) -> int:
    return lib.bgemm_plane_bytes(M, K)


def act_ld(K: int) -> int:
    return lib.bgemm_act_ld(K)


def launch_count() -> int:
    return lib.bgemm_launch_count()


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("expected a CUDA tensor (this library has no CPU path)")


def pack_weights(w: torch.Tensor, wbit_mode: int = WBIT_NEGATIVE, want_rowpop: bool = False, want_alpha: bool = False):
    """[M, K] or [B, M, K] unpacked -> (plane uint8 [B * plane_bytes], rowpop int32 | None, alpha fp16 | None)."""
    _require_cuda(w)
    batched = w.dim() == 3
    w3 = w if batched else w.unsqueeze(0)
    if w3.stride(-1) != 1 or (w3.shape[0] > 1 and w3.stride(0) < 0):
        w3 = w3.contiguous()
    B, M, K = w3.shape
    plane = torch.empty(B * plane_bytes(M, K), dtype=torch.uint8, device=w.device)
    rowpop = torch.empty(B * M, dtype=torch.int32, device=w.device) if want_rowpop else None
    alpha = torch.empty(B * M, dtype=torch.float16, device=w.device) if want_alpha else None
    with torch.cuda.device(w.device):
        check(lib.bgemm_pack_weights(_stream(), w3.data_ptr(), dtype_code(w3), M, K, w3.stride(1), wbit_mode, plane.data_ptr(),
                                     _ptr(rowpop), _ptr(alpha), B, w3.stride(0) if B > 1 else 0), "bgemm_pack_weights")
    if not batched:
        return plane, rowpop, alpha
    return plane, (rowpop.view(B, M) if want_rowpop else None), (alpha.view(B, M) if want_alpha else None)


def prepare_acts(x: torch.Tensor, act_mode: int, transpose: bool = False):
    """[N, K] (or [K, N] with transpose; optional leading batch dim) -> (int8 [B, N, act_ld(K)], colsum int32 [B, N])."""
    _require_cuda(x)
    batched = x.dim() == 3
    x3 = x if batched else x.unsqueeze(0)
    if x3.stride(-1) != 1:
        x3 = x3.contiguous()
    B = x3.shape[0]
    N, K = (x3.shape[2], x3.shape[1]) if transpose else (x3.shape[1], x3.shape[2])
    dst = torch.empty((B, N, act_ld(K)), dtype=torch.int8, device=x.device)
    colsum = torch.empty((B, N), dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.bgemm_prepare_acts(_stream(), x3.data_ptr(), dtype_code(x3), N, K, x3.stride(1), act_mode, 1 if transpose else 0,
                                     dst.data_ptr(), colsum.data_ptr(), B, x3.stride(0) if B > 1 else 0), "bgemm_prepare_acts")
    if not batched:
        return dst[0], colsum[0]
    return dst, colsum


_workspaces: dict = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch per (device, current stream), grown on demand (the library keeps its counter prefix
    zero). One buffer per stream: calls on one stream run in order and may share it, calls on different streams may
    overlap on the GPU and must not (bgemm_linear_forward parks its packed operands there)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (device.type, index, torch.cuda.current_stream(index).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        if key in _workspaces:
            _workspaces[key].record_stream(torch.cuda.current_stream(index))   # the smaller buffer may still be in use
        _workspaces[key] = ws
    return ws


_balance_workspaces: dict = {}


def balance_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """The optional workspace of bgemm_gemm (exact work split for wide activation matrices), per (device, current
    stream). Kept apart from `workspace`: its first 64 KiB are flags that must stay zero between launches, and the other
    buffer also parks packed operands."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (device.type, index, torch.cuda.current_stream(index).cuda_stream)
    ws = _balance_workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        if key in _balance_workspaces:
            _balance_workspaces[key].record_stream(torch.cuda.current_stream(index))
        _balance_workspaces[key] = ws
    return ws


def gemm(plane: torch.Tensor, M: int, K: int, acts: torch.Tensor, colsum: torch.Tensor, op: int, out_kind: int = OUT_I32,
         out_layout: int = LAYOUT_NM, alpha: torch.Tensor | None = None, split_k: int = 0, out: torch.Tensor | None = None,
         ws: torch.Tensor | None = None, static_weights: bool = False, balance: bool = True):
    """GEMM on prepared operands. acts: int8 [N, ld] or [B, N, ld]; returns [N, M] / [M, N] (with leading B if batched).
    static_weights=True: the caller promises that `plane` was complete before the previous kernel on the current stream
    was launched. `ws`: the workspace that split_k > 8 needs, or (other calls) a balance workspace -- zeroed once, used for
    nothing else -- for the exact work split of wide activation matrices; by default one is kept per stream
    (balance=False: whole tiles only)."""
    _require_cuda(plane, acts, colsum, alpha)
    batched = acts.dim() == 3
    B = acts.shape[0] if batched else 1
    N = acts.shape[-2]
    assert acts.shape[-1] == act_ld(K) and acts.is_contiguous() and colsum.is_contiguous()
    shape = (N, M) if out_layout == LAYOUT_NM else (M, N)
    if batched:
        shape = (B,) + shape
    if out is None:
        out = torch.empty(shape, dtype=torch.int32 if out_kind == OUT_I32 else torch.float16, device=acts.device)
    flags = FLAG_STATIC_WEIGHTS if static_weights else 0
    need = lib.bgemm_gemm_workspace_bytes(M, N, K, split_k, B)
    if need and ws is None:
        ws = workspace(acts.device, need)
    if not need:
        bal = lib.bgemm_gemm_balance_workspace_bytes(M, N, K, split_k, B)      # optional: exact work split for wide N
        if bal and ws is None and balance:
            ws = balance_workspace(acts.device, bal)
        if bal and ws is not None and ws.numel() >= bal and balance:
            flags |= FLAG_BALANCE_WORKSPACE
        else:
            ws = None
    with torch.cuda.device(acts.device):
        check(lib.bgemm_gemm_ex(_stream(), plane.data_ptr(), M, K, acts.data_ptr(), colsum.data_ptr(), N, op, out.data_ptr(), out_kind,
                                out_layout, _ptr(alpha), split_k, _ptr(ws), ws.numel() if ws is not None else 0, B, flags), "bgemm_gemm")
    return out


def gemm_multi_out(plane: torch.Tensor, M: int, K: int, acts: torch.Tensor, colsum: torch.Tensor, op: int, out_ptrs, out_ld: int,
                   out_kind: int = OUT_F16, out_layout: int = LAYOUT_NM, alpha: torch.Tensor | None = None, split_k: int = 0,
                   static_weights: bool = False, ws: torch.Tensor | None = None) -> None:
    """GEMM whose result is stored once at every address in `out_ptrs` (ints: device pointers, local or peer-mapped),
    inside matrices of row pitch `out_ld` elements: a row shard writing its slab into every rank's full result."""
    _require_cuda(plane, acts, colsum, alpha)
    assert acts.dim() == 2 and acts.shape[-1] == act_ld(K) and acts.is_contiguous() and colsum.is_contiguous()
    N = acts.shape[0]
    ptrs = (ctypes.c_void_p * len(out_ptrs))(*[int(p) for p in out_ptrs])
    flags = FLAG_STATIC_WEIGHTS if static_weights else 0
    need = lib.bgemm_gemm_workspace_bytes(M, N, K, split_k, 1)
    if need and ws is None:
        ws = workspace(acts.device, need)
    if not need:
        bal = lib.bgemm_gemm_balance_workspace_bytes(M, N, K, split_k, 1)
        if bal and ws is None:
            ws = balance_workspace(acts.device, bal)
        if bal and ws is not None and ws.numel() >= bal:
            flags |= FLAG_BALANCE_WORKSPACE
        else:
            ws = None
    with torch.cuda.device(acts.device):
        check(lib.bgemm_gemm_multi_out(_stream(), plane.data_ptr(), M, K, acts.data_ptr(), colsum.data_ptr(), N, op, ptrs, len(out_ptrs), out_ld,
                                       out_kind, out_layout, _ptr(alpha), split_k, _ptr(ws), ws.numel() if ws is not None else 0,
                                       flags), "bgemm_gemm_multi_out")


def w1a16_gemm(plane: torch.Tensor, M: int, K: int, x: torch.Tensor, out_kind: int = OUT_F32, out_layout: int = LAYOUT_NM,
               alpha: torch.Tensor | None = None, static_weights: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
    """Binary weight x fp16 activation: x fp16 [N, K] (unprepared) -> [N, M] / [M, N], fp32 or fp16, fp32 accumulation."""
    _require_cuda(plane, x, alpha)
    assert x.dim() == 2 and x.dtype == torch.float16 and x.shape[1] == K and x.stride(1) == 1
    N = x.shape[0]
    shape = (N, M) if out_layout == LAYOUT_NM else (M, N)
    if out is None:
        out = torch.empty(shape, dtype=torch.float32 if out_kind == OUT_F32 else torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.bgemm_w1a16_gemm(_stream(), plane.data_ptr(), M, K, x.data_ptr(), x.stride(0), N, out.data_ptr(), out_kind, out_layout,
                                   _ptr(alpha), 1 if static_weights else 0), "bgemm_w1a16_gemm")
    return out


def gemm_to_acts(plane: torch.Tensor, M: int, K: int, acts: torch.Tensor, colsum: torch.Tensor, op: int, next_act_mode: int,
                 alpha: torch.Tensor | None = None, split_k: int = 0, ws: torch.Tensor | None = None, sums: torch.Tensor | None = None):
    """GEMM whose result becomes the next layer's prepared activations: (int8 [.., N, act_ld(M)], colsum int32 [.., N]).
    `sums`: an int32 tensor the caller has zeroed on the current stream; it receives the row sums (BGEMM_FLAG_SUMS_ZEROED)."""
    _require_cuda(plane, acts, colsum, alpha)
    batched = acts.dim() == 3
    B = acts.shape[0] if batched else 1
    N = acts.shape[-2]
    assert acts.shape[-1] == act_ld(K) and acts.is_contiguous() and colsum.is_contiguous()
    lead = (B,) if batched else ()
    nxt = torch.empty(lead + (N, act_ld(M)), dtype=torch.int8, device=acts.device)
    if sums is not None:        # zeroed by the caller on the current stream: the call enqueues nothing but its kernel
        assert sums.dtype == torch.int32 and sums.is_contiguous() and sums.numel() == B * N and sums.device == acts.device
        ncs = sums.view(lead + (N,))
    else:
        ncs = torch.empty(lead + (N,), dtype=torch.int32, device=acts.device)
    need = lib.bgemm_gemm_workspace_bytes(M, N, K, split_k, B)
    if need and ws is None:
        ws = workspace(acts.device, need)
    with torch.cuda.device(acts.device):
        check(lib.bgemm_gemm_to_acts_ex(_stream(), plane.data_ptr(), M, K, acts.data_ptr(), colsum.data_ptr(), N, op, _ptr(alpha), next_act_mode,
                                        nxt.data_ptr(), ncs.data_ptr(), split_k, _ptr(ws) if need else None, ws.numel() if need else 0, B,
                                        FLAG_SUMS_ZEROED if sums is not None else 0),
              "bgemm_gemm_to_acts")
    return nxt, ncs


def linear_forward(weight_f16: torch.Tensor, acts_f16: torch.Tensor, op: int = OP_XOR, out_kind: int = OUT_F16,
                   out_layout: int = LAYOUT_NM, alpha: torch.Tensor | None = None, split_k: int = 0,
                   out: torch.Tensor | None = None, ws: torch.Tensor | None = None):
    """Unpacked fp16 [M, K] x [N, K] -> [N, M]: the drop-in for the reference's bin_pack_linear_kernel."""
    _require_cuda(weight_f16, acts_f16, alpha)
    assert weight_f16.dtype == torch.float16 and acts_f16.dtype == torch.float16
    assert weight_f16.is_contiguous() and acts_f16.is_contiguous()
    M, K = weight_f16.shape
    N = acts_f16.shape[0]
    assert acts_f16.shape[1] == K
    shape = (N, M) if out_layout == LAYOUT_NM else (M, N)
    if out is None:
        out = torch.empty(shape, dtype=torch.int32 if out_kind == OUT_I32 else torch.float16, device=acts_f16.device)
    need = lib.bgemm_linear_workspace_bytes(M, N, K, split_k)
    if ws is None:
        ws = workspace(acts_f16.device, need)
    with torch.cuda.device(acts_f16.device):
        check(lib.bgemm_linear_forward(_stream(), weight_f16.data_ptr(), acts_f16.data_ptr(), out.data_ptr(), M, N, K, op, out_kind,
                                       out_layout, _ptr(alpha), split_k, ws.data_ptr(), ws.numel()), "bgemm_linear_forward")
    return out
