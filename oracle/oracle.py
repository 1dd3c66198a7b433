"""CPU oracle for the binary / ternary GEMM path -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this module; the
shipped library never does. It holds

* ctypes bindings of ``liboracle.so`` (the C restatement in ``bgemm_oracle.c``) and, when it was
  built, of ``_ref/libref_prepack.so`` (the reference's own prepack compiled from its header);
* the reference's CPU definition of each product -- dense fp32 torch matmul on sign / ternary mapped
  tensors (tests/python/bgemm_linear.py:633-645 ``BNNLinear.forward``, :246-275
  ``nn_linear_elastic_signed.forward``, tests/python/test_kernel.py:50-56) -- exact because every
  partial sum is an integer below 2**24;
* a numpy restatement of the tiled bit-plane and prepared-activation formats the GPU library defines
  (``include/bgemm_b200.h``), used to check the prepack kernels bit for bit;
* seeded generators for the five benchmark workloads.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np
import torch

_HERE = Path(__file__).resolve().parent

OP_AND, OP_XOR, OP_ATTN, OP_BWTA = 0, 1, 2, 3
OP_W1A8 = 4          # BWTA's arithmetic on general int8 activations (a routing hint of the library, not a new formula)
OUT_I32, OUT_F16, OUT_F16_SCALED = 0, 1, 2
ACT_SIGN, ACT_TERNARY, ACT_NEG01, ACT_INT8 = 0, 1, 2, 3
ACT_MODE_OF_OP = {OP_AND: ACT_NEG01, OP_XOR: ACT_SIGN, OP_ATTN: ACT_SIGN, OP_BWTA: ACT_TERNARY}
WBIT_OF_OP = {OP_AND: 0, OP_XOR: 0, OP_ATTN: 1, OP_BWTA: 0}


# --------------------------------------------------------------------------------------------------
# C oracle bindings
# --------------------------------------------------------------------------------------------------
def build(force: bool = False) -> None:
    """Compile liboracle.so (and _ref/ when a reference checkout is present)."""
    if force or not (_HERE / "liboracle.so").exists():
        subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True, capture_output=True)
    ref_root = reference_root()
    if ref_root and (force or not (_HERE / "_ref" / "libref_prepack.so").exists()):
        subprocess.run(["make", "-C", str(_HERE), "ref", f"REFERENCE_ROOT={ref_root}"], check=True, capture_output=True)


def reference_root():
    """A checkout of the reference project, if one is reachable: $REFERENCE_ROOT, else a directory named `reference`
    beside this repository. None when there is none (the GPU box): prebuilt files under _ref/ are then used as they are."""
    cand = os.environ.get("REFERENCE_ROOT") or str(_HERE.parent.parent / "reference")
    return cand if os.path.isfile(os.path.join(cand, "lowbit_kernel", "csrc", "utils", "weight_prepacking.h")) else None


_lib = None
_ref = None


def clib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_HERE / "liboracle.so"))
        _lib.oracle_f16_to_f32.restype = ctypes.c_float
        _lib.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.oracle_f32_to_f16.restype = ctypes.c_uint16
        _lib.oracle_f32_to_f16.argtypes = [ctypes.c_float]
    return _lib


def reflib():
    """The reference's own prepack (None when oracle/_ref was not built)."""
    global _ref
    if _ref is None:
        p = _HERE / "_ref" / "libref_prepack.so"
        if not p.exists():
            return None
        _ref = ctypes.CDLL(str(p))
    return _ref


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _f16_bits(t) -> np.ndarray:
    """fp16 bit patterns (uint16, C-contiguous 2-D) of a tensor / array."""
    if isinstance(t, torch.Tensor):
        t = t.detach().cpu().to(torch.float16).contiguous().numpy()
    a = np.ascontiguousarray(np.asarray(t, dtype=np.float16))
    return a.view(np.uint16)


def c_pack_rowmajor_msb(w) -> np.ndarray:
    b = _f16_bits(w)
    rows, K = b.shape
    assert K % 32 == 0
    out = np.zeros((rows, K // 32), dtype=np.uint32)
    clib().oracle_pack_rowmajor_msb(_p(b), ctypes.c_int64(rows), ctypes.c_int64(K), ctypes.c_int64(K), _p(out))
    return out


def ref_pack_rowmajor_msb(w) -> np.ndarray:
    """bin_matrix_prepacking_to_uint32 itself (needs oracle/_ref)."""
    lib = reflib()
    assert lib is not None, "oracle/_ref/libref_prepack.so is not built"
    b = _f16_bits(w)
    rows, K = b.shape
    assert K % 128 == 0
    out = np.zeros((rows, K // 32), dtype=np.uint32)
    lib.ref_bin_matrix_prepacking_to_uint32(_p(out), _p(b), ctypes.c_size_t(rows), ctypes.c_size_t(K))
    return out


def c_bgemm_bits(wbits: np.ndarray, xbits: np.ndarray, K: int, instr: int) -> np.ndarray:
    M, N = wbits.shape[0], xbits.shape[0]
    out = np.zeros((N, M), dtype=np.int32)
    clib().oracle_bgemm_bits(_p(np.ascontiguousarray(wbits)), _p(np.ascontiguousarray(xbits)),
                             ctypes.c_int64(M), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(instr), _p(out))
    return out


def c_bgemm_dense(w, x, op: int) -> np.ndarray:
    wb, xb = _f16_bits(w), _f16_bits(x)
    M, K = wb.shape
    N = xb.shape[0]
    out = np.zeros((N, M), dtype=np.int32)
    clib().oracle_bgemm_dense(_p(wb), ctypes.c_int64(K), _p(xb), ctypes.c_int64(K), ctypes.c_int64(M),
                              ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(op), _p(out))
    return out


def c_store_f16(acc: np.ndarray) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    out = np.zeros(acc.shape, dtype=np.uint16)
    clib().oracle_store_f16(_p(acc), ctypes.c_int64(acc.size), _p(out))
    return out.view(np.float16)


def c_store_f16_scaled(acc: np.ndarray, alpha) -> np.ndarray:
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    N, M = acc.shape
    ab = _f16_bits(np.asarray(alpha).reshape(1, -1)).reshape(-1)
    out = np.zeros((N, M), dtype=np.uint16)
    clib().oracle_store_f16_scaled(_p(acc), _p(ab), ctypes.c_int64(M), ctypes.c_int64(N), _p(out))
    return out.view(np.float16)


def c_splitk_f16(w, x, op: int, split_k: int) -> np.ndarray:
    """Reference split-K semantics: fp32 partial slabs over equal K/128-block ranges, then one rounding."""
    wb, xb = _f16_bits(w), _f16_bits(x)
    M, K = wb.shape
    N = xb.shape[0]
    slabs = np.zeros((split_k, N, M), dtype=np.float32)
    nblk = K // 128
    avg, extra = divmod(nblk, split_k)          # kernel_matmul.cuh:397-404
    start = 0
    for s in range(split_k):
        cnt = avg + (1 if s < extra else 0)
        clib().oracle_bgemm_dense_partial_f32(_p(wb), ctypes.c_int64(K), _p(xb), ctypes.c_int64(K),
                                              ctypes.c_int64(M), ctypes.c_int64(N),
                                              ctypes.c_int64(start * 128), ctypes.c_int64((start + cnt) * 128),
                                              ctypes.c_int(op), _p(slabs[s]))
        start += cnt
    out = np.zeros((N, M), dtype=np.uint16)
    clib().oracle_splitk_reduce_f16(_p(slabs), ctypes.c_int64(N * M), ctypes.c_int(split_k), _p(out))
    return out.view(np.float16)


def c_rowmeanabs_f16(w) -> np.ndarray:
    wb = _f16_bits(w)
    M, K = wb.shape
    out = np.zeros(M, dtype=np.uint16)
    clib().oracle_rowmeanabs_f16(_p(wb), ctypes.c_int64(M), ctypes.c_int64(K), ctypes.c_int64(K), _p(out))
    return out.view(np.float16)


# --------------------------------------------------------------------------------------------------
# The reference's CPU definition: dense torch fp32 matmul on mapped operands
# --------------------------------------------------------------------------------------------------
def signbit(t: torch.Tensor) -> torch.Tensor:
    return torch.signbit(t.to(torch.float16))


def map_weight(w: torch.Tensor, op: int) -> torch.Tensor:
    """fp32 value each weight-slot element contributes under `op`."""
    s = signbit(w)
    if op == OP_AND:
        return s.float()                      # 1 where negative
    if op == OP_ATTN:
        return (~s).float()                   # 1 where the mask is "1" (sign bit clear)
    return 1.0 - 2.0 * s.float()              # -1 / +1 by sign bit


def map_act(x: torch.Tensor, op: int) -> torch.Tensor:
    s = signbit(x)
    if op == OP_AND:
        return s.float()
    if op == OP_BWTA:
        return torch.sign(x.to(torch.float16).float())     # torch.sign: 0 for +-0
    return 1.0 - 2.0 * s.float()


def ref_acc(w: torch.Tensor, x: torch.Tensor, op: int) -> torch.Tensor:
    """int32 [N, M] = mapped(x) @ mapped(w).T in fp32 on the CPU (exact for K < 2**24)."""
    assert w.shape[-1] == x.shape[-1]
    acc = map_act(x.cpu(), op) @ map_weight(w.cpu(), op).transpose(-1, -2)
    return acc.to(torch.int32)


def ref_w1a16(w: torch.Tensor, x: torch.Tensor, alpha: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 [N, M] = fp16(x) @ sgn(w).T (* alpha[m]) in fp32 on the CPU: binary weight x fp16 activation, the variant the
    reference lists as to-do (README.md:29), defined like its dense layers (tests/python/bgemm_linear.py:270-272) with
    sgn read from the sign bit."""
    acc = x.cpu().to(torch.float16).float() @ map_weight(w.cpu(), OP_XOR).transpose(-1, -2)
    return acc if alpha is None else acc * alpha.cpu().to(torch.float16).float()


def ref_out(acc: torch.Tensor, out_kind: int, alpha: torch.Tensor | None = None) -> torch.Tensor:
    """Store conversion of an [..., N, M] int32 accumulator."""
    if out_kind == OUT_I32:
        return acc
    if out_kind == OUT_F16:
        return acc.to(torch.float32).to(torch.float16)
    return (acc.to(torch.float32) * alpha.cpu().to(torch.float16).float()).to(torch.float16)


# --------------------------------------------------------------------------------------------------
# numpy restatement of the library's own formats (include/bgemm_b200.h)
# --------------------------------------------------------------------------------------------------
def plane_bytes(M: int, K: int) -> int:
    return -(-M // 128) * -(-K // 256) * 4096


def act_ld(K: int) -> int:
    return -(-K // 256) * 256


def np_tiled_plane(bits: np.ndarray) -> np.ndarray:
    """bits: bool/0-1 array [M, K] -> uint8 array of plane_bytes(M, K) in the tiled layout.

    Tile (mt, kb) = rows [128 mt, +128) x columns [256 kb, +256), stored kb-fastest, 4096 bytes each.
    A row owns 8 little-endian uint32 words; element k = 256 kb + 32 j + 4 c + b is bit (8 b + j) of
    word c; word c of row r sits at byte (c // 4) * 2048 + r * 16 + (c % 4) * 4 of the tile.
    """
    M, K = bits.shape
    MT, KB = -(-M // 128), -(-K // 256)
    full = np.zeros((MT * 128, KB * 256), dtype=np.uint32)
    full[:M, :K] = bits.astype(np.uint32)
    # index as [mt, r, kb, j, c, b]
    v = full.reshape(MT, 128, KB, 8, 8, 4)
    words = np.zeros((MT, KB, 128, 8), dtype=np.uint32)
    for j in range(8):
        for b in range(4):
            # v[mt, r, kb, j, c, b] -> words[mt, kb, r, c] bit 8b+j
            words |= np.transpose(v[:, :, :, j, :, b], (0, 2, 1, 3)) << np.uint32(8 * b + j)
    # [mt, kb, r, c] -> [mt, kb, c // 4, r, c % 4]
    words = np.ascontiguousarray(np.transpose(words.reshape(MT, KB, 128, 2, 4), (0, 1, 3, 2, 4)))
    return words.reshape(-1).view(np.uint8)


def np_pack_weights(w, wbit_mode: int):
    """(plane uint8, rowpop int32[M]) from unpacked weights."""
    wt = w.detach().cpu() if isinstance(w, torch.Tensor) else torch.as_tensor(np.asarray(w))
    s = torch.signbit(wt).numpy()
    nz = (wt != 0).numpy()
    bits = {0: s, 1: ~s, 2: nz, 3: s & nz}[wbit_mode]
    return np_tiled_plane(bits), bits.sum(axis=1).astype(np.int32)


def np_prepare_acts(x, act_mode: int):
    """(int8 [N, act_ld(K)], colsum int32 [N]) from unpacked activations."""
    xt = x.detach().cpu() if isinstance(x, torch.Tensor) else torch.as_tensor(np.asarray(x))
    s = torch.signbit(xt)
    if act_mode == ACT_SIGN:
        v = (1 - 2 * s.to(torch.int8))
    elif act_mode == ACT_TERNARY:
        v = torch.sign(xt.float()).to(torch.int8)
    elif act_mode == ACT_INT8:
        v = xt.to(torch.int8)
    else:
        v = s.to(torch.int8)
    N, K = v.shape
    out = np.zeros((N, act_ld(K)), dtype=np.int8)
    out[:, :K] = v.numpy()
    return out, out.astype(np.int32).sum(axis=1).astype(np.int32)


# --------------------------------------------------------------------------------------------------
# Seeded synthetic workloads (shapes and value distributions of the five benchmark configurations)
# --------------------------------------------------------------------------------------------------
def _gen(seed: int) -> torch.Generator:
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def rand_pm1(shape, g) -> torch.Tensor:
    return (2 * torch.randint(0, 2, shape, generator=g) - 1).to(torch.float16)


def rand_ternary(shape, g, p_neg=0.35, p_pos=0.35) -> torch.Tensor:
    u = torch.rand(shape, generator=g)
    x = torch.zeros(shape)
    x[u < p_neg] = -1.0
    x[(u >= p_neg) & (u < p_neg + p_pos)] = 1.0
    return x.to(torch.float16)


def config1(M=4096, K=4096, N=64, seed=1001):
    g = _gen(seed)
    return dict(w=rand_pm1((M, K), g), x=rand_pm1((N, K), g), op=OP_XOR)


def config2(M=4096, K=4096, N=128, seed=1002):
    g = _gen(seed)
    w = rand_pm1((M, K), g)
    x = rand_ternary((N, K), g)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    return dict(w=w, x=x, alpha=alpha, op=OP_BWTA)


def config3(heads=384, S=512, d=64, seed=1003):
    g = _gen(seed)
    a = torch.bernoulli(torch.full((heads, S, S), 0.5), generator=g).to(torch.float16)   # {0,1}
    v = rand_pm1((heads, S, d), g)
    return dict(attn=a, v=v, op=OP_ATTN)


def config4(batch=256, dims=(1024, 4096, 4096, 10), seed=1004):
    g = _gen(seed)
    ws = [(0.02 * torch.randn(dims[i + 1], dims[i], generator=g)).to(torch.float16) for i in range(3)]
    x = torch.randn(batch, dims[0], generator=g).to(torch.float16)
    return dict(ws=ws, x=x)


def config5(M=28672, K=8192, N=128, seed=1005):
    g = _gen(seed)
    w = rand_pm1((M, K), g)
    x = rand_ternary((N, K), g)
    alpha = (0.01 + 0.09 * torch.rand(M, generator=g)).to(torch.float16)
    return dict(w=w, x=x, alpha=alpha, op=OP_BWTA)


def ref_attn_heads(attn01: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """int32 [heads, Sq, d] = attn01 @ sign(v): torch.bmm on CPU (bgemm_linear.py:107-108 `mm.forward`)."""
    vv = 1.0 - 2.0 * torch.signbit(v).float()
    return torch.bmm(attn01.float(), vv).to(torch.int32)


def ref_mlp(ws, x):
    """Binary MLP forward of benchmark configuration 4 on the CPU.

    h0 = sign+(x); h_l = sign+(alpha_l * (B_l h_{l-1})) for hidden layers; logits fp16 = alpha_L * (B_L h).
    sign+(0) = +1 (BinActive, bgemm_linear.py:604-608); alpha_l[m] = mean(|W_l[m,:]|) in fp16.
    Returns (logits fp16 [batch, out], list of int32 accumulators per layer).
    """
    h = x
    accs = []
    for i, w in enumerate(ws):
        alpha = torch.from_numpy(c_rowmeanabs_f16(w).copy())
        acc = ref_acc(w, h, OP_XOR)
        accs.append(acc)
        y = ref_out(acc, OUT_F16_SCALED, alpha)
        if i == len(ws) - 1:
            return y, accs
        h = y
    raise AssertionError
