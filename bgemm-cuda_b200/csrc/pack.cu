// Operand preparation kernels: weight-slot matrices -> tiled 1-bit planes, activation-slot matrices ->
// zero-padded int8 rows + column sums, plus the reference-compatible row-major MSB-first prepack.
//
// Replaces the reference's CPU prepack bin_matrix_prepacking_to_uint32
// (lowbit_kernel/csrc/utils/weight_prepacking.h:181-230), its never-implemented GPU twin
// binary_weight_prepacking_cuda (lowbit_kernel/csrc/fp6_linear.cu:519-542) and the on-the-fly sign
// extraction inside the GEMM (SIGN_32_HALF_TO_UINT32, include/ptx_mma.cuh:341-399).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstring>

#include "internal.h"
#include "ptx.cuh"

namespace bgemm {

// ---- element decoding ----------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
    static __host__ __device__ __forceinline__ int neg(const __half& v) { return (reinterpret_cast<const uint16_t&>(v) >> 15) & 1; }
    static __host__ __device__ __forceinline__ int zero(const __half& v) { return (reinterpret_cast<const uint16_t&>(v) & 0x7fffu) == 0; }
    static __device__ __forceinline__ float mag(const __half& v) { return fabsf(__half2float(v)); }
    static __host__ __device__ __forceinline__ int8_t as_int8(const __half&) { return 0; }
};
template <> struct Elem<__nv_bfloat16> {
    static __host__ __device__ __forceinline__ int neg(const __nv_bfloat16& v) { return (reinterpret_cast<const uint16_t&>(v) >> 15) & 1; }
    static __host__ __device__ __forceinline__ int zero(const __nv_bfloat16& v) { return (reinterpret_cast<const uint16_t&>(v) & 0x7fffu) == 0; }
    static __device__ __forceinline__ float mag(const __nv_bfloat16& v) { return fabsf(__bfloat162float(v)); }
    static __host__ __device__ __forceinline__ int8_t as_int8(const __nv_bfloat16&) { return 0; }
};
template <> struct Elem<float> {
    static __host__ __device__ __forceinline__ int neg(const float& v) { return (reinterpret_cast<const uint32_t&>(v) >> 31) & 1; }
    static __host__ __device__ __forceinline__ int zero(const float& v) { return (reinterpret_cast<const uint32_t&>(v) & 0x7fffffffu) == 0; }
    static __device__ __forceinline__ float mag(const float& v) { return fabsf(v); }
    static __host__ __device__ __forceinline__ int8_t as_int8(const float&) { return 0; }
};
template <> struct Elem<int8_t> {
    static __host__ __device__ __forceinline__ int neg(const int8_t& v) { return v < 0; }
    static __host__ __device__ __forceinline__ int zero(const int8_t& v) { return v == 0; }
    static __device__ __forceinline__ float mag(const int8_t& v) { return fabsf((float)v); }
    static __host__ __device__ __forceinline__ int8_t as_int8(const int8_t& v) { return v; }
};

// Byte offset of word c (0..7) of row r (0..127) inside a 4096-byte tile: two 2 KB halves, each holding
// four words of every row, so that a warp's 16-byte reads of consecutive rows are contiguous.
__host__ __device__ __forceinline__ int tile_word_offset(int r, int c) { return (c >> 2) * 2048 + r * 16 + (c & 3) * 4; }

// Bit a weight-slot element contributes under BGEMM_WBIT_* mode.
template <typename T>
__host__ __device__ __forceinline__ int weight_bit(const T& v, int mode) {
    const int neg = Elem<T>::neg(v);
    if (mode == BGEMM_WBIT_NEGATIVE) return neg;
    if (mode == BGEMM_WBIT_NONNEGATIVE) return neg ^ 1;
    const int nz = Elem<T>::zero(v) ^ 1;
    return mode == BGEMM_WBIT_NONZERO ? nz : (neg & nz);
}

// Weight-slot bits of two 16-bit floats (fp16 or bf16) held in one 32-bit word: bit 0 = low element, bit 16 = high.
__device__ __forceinline__ uint32_t weight_bits_x2(uint32_t w, int mode) {
    const uint32_t s = (w >> 15) & 0x00010001u;
    if (mode == BGEMM_WBIT_NEGATIVE) return s;
    if (mode == BGEMM_WBIT_NONNEGATIVE) return s ^ 0x00010001u;
    const uint32_t nz = (((w & 0x7fff7fffu) + 0x7fff7fffu) >> 15) & 0x00010001u;
    return mode == BGEMM_WBIT_NONZERO ? nz : (nz & s);
}

// ---- weights -> tiled plane (+ rowpop, alpha) ---------------------------------------------------------------
// Bit 8 b + j of word c of a row's K block is element k = 32 j + 4 c + b of that block, so the words 2 cp and 2 cp + 1
// are made of the eight 8-element pieces k = 32 j + 8 cp ... + 7 (j = 0..7; 16 bytes of a 2-byte type each) and of
// nothing else. A warp therefore packs one K block of EIGHT consecutive rows per step: lane = 4 * (row in the group)
// + cp loads its eight pieces (eight independent 16-byte streaming loads; the four lanes of a row cover 64 contiguous
// bytes per load), builds its two words without any exchange between lanes, and stores them as 8 bytes (the eight
// rows of the group are 128 contiguous bytes in each half of the tile). For the two sign modes the sign bits of four
// elements come out of one byte permute (the high bytes of four 16-bit floats) and one shift-and-mask.
// `ksplit` (1, 2, 4 or 8) warps of a CTA share a row group by K blocks, so that a matrix with few rows still puts
// loads from every SM in flight; their row sums meet in shared memory.
template <typename T>
struct RawBlock {
    T v[8][8];      // [piece j][element e]
};

template <typename T>
__device__ __forceinline__ void load_block(RawBlock<T>& raw, const T* __restrict__ rp, long long k0, long long K, bool live, bool vec_ok) {
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const long long k = k0 + 32 * j;
        if (live && vec_ok && k + 8 <= K) {         // one piece = 8 elements: 8, 16 or 32 bytes
            if (sizeof(T) == 1) {
                *reinterpret_cast<uint2*>(raw.v[j]) = __ldcs(reinterpret_cast<const uint2*>(rp + k));
            } else if (sizeof(T) == 2) {
                *reinterpret_cast<uint4*>(raw.v[j]) = __ldcs(reinterpret_cast<const uint4*>(rp + k));
            } else {
                reinterpret_cast<uint4*>(raw.v[j])[0] = __ldcs(reinterpret_cast<const uint4*>(rp + k));
                reinterpret_cast<uint4*>(raw.v[j])[1] = __ldcs(reinterpret_cast<const uint4*>(rp + k) + 1);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++) raw.v[j][e] = (live && k + e < K) ? rp[k + e] : T();
        }
    }
}

// The weight-slot bits of four int8 elements held in one word, at bit 0 of their bytes (no -0 among integers: "negative
// and non-zero" is "negative").
__device__ __forceinline__ uint32_t weight_bits_i8x4(uint32_t x, int mode) {
    const uint32_t neg = (x >> 7) & 0x01010101u;
    if (mode == BGEMM_WBIT_NEGATIVE) return neg;
    if (mode == BGEMM_WBIT_NONNEGATIVE) return neg ^ 0x01010101u;
    return mode == BGEMM_WBIT_NONZERO ? (__vcmpne4(x, 0u) & 0x01010101u) : neg;
}

template <typename T>
__device__ __forceinline__ void bits_of_block(const RawBlock<T>& raw, long long k0, long long K, bool live, bool vec_ok, int mode, bool want_mag,
                                              uint32_t& w0, uint32_t& w1, float& mag) {
    w0 = 0;
    w1 = 0;
    if (!live) return;
    const bool whole = vec_ok && k0 + 32 * 7 + 8 <= K;               // all eight pieces complete
    if (sizeof(T) == 2 && whole) {
        if (mode == BGEMM_WBIT_NEGATIVE || mode == BGEMM_WBIT_NONNEGATIVE) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint4 q = *reinterpret_cast<const uint4*>(raw.v[j]);
                const uint32_t hi0 = __byte_perm(q.x, q.y, 0x7531), hi1 = __byte_perm(q.z, q.w, 0x7531);   // high bytes of e0..e3, e4..e7
                w0 |= (hi0 >> (7 - j)) & (0x01010101u << j);
                w1 |= (hi1 >> (7 - j)) & (0x01010101u << j);
            }
            if (mode == BGEMM_WBIT_NONNEGATIVE) {
                w0 = ~w0;
                w1 = ~w1;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint4 q = *reinterpret_cast<const uint4*>(raw.v[j]);
                const uint32_t q0 = weight_bits_x2(q.x, mode), q1 = weight_bits_x2(q.y, mode);
                const uint32_t q2 = weight_bits_x2(q.z, mode), q3 = weight_bits_x2(q.w, mode);
                w0 |= ((((q0 | (q0 >> 8)) & 0x101u) | (((q1 | (q1 >> 8)) & 0x101u) << 16))) << j;
                w1 |= ((((q2 | (q2 >> 8)) & 0x101u) | (((q3 | (q3 >> 8)) & 0x101u) << 16))) << j;
            }
        }
        if (want_mag) {
#pragma unroll
            for (int j = 0; j < 8; j++)
#pragma unroll
                for (int e = 0; e < 8; e++) mag += Elem<T>::mag(raw.v[j][e]);
        }
    } else if (sizeof(T) == 1 && whole) {
        uint32_t abs_sum = 0;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint2 q = *reinterpret_cast<const uint2*>(raw.v[j]);
            w0 |= weight_bits_i8x4(q.x, mode) << j;
            w1 |= weight_bits_i8x4(q.y, mode) << j;
            if (want_mag) {     // |v| <= 128 per byte, summed as integers: exact, like the element-wise fp32 sum below
                abs_sum = __dp4a(__vabsdiffs4(q.x, 0u), 0x01010101u, abs_sum);
                abs_sum = __dp4a(__vabsdiffs4(q.y, 0u), 0x01010101u, abs_sum);
            }
        }
        mag += (float)abs_sum;
    } else {
#pragma unroll
        for (int j = 0; j < 8; j++) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                if (k0 + 32 * j + e < K) {
                    const uint32_t bit = (uint32_t)weight_bit<T>(raw.v[j][e], mode);
                    if (e < 4) w0 |= bit << (8 * e + j); else w1 |= bit << (8 * (e - 4) + j);
                    if (want_mag) mag += Elem<T>::mag(raw.v[j][e]);
                }
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256) pack_weights_kernel(const T* __restrict__ src, long long M, long long K, long long ld, int mode,
                                                           uint8_t* __restrict__ plane, int32_t* __restrict__ rowpop,
                                                           __half* __restrict__ alpha, long long src_batch_stride,
                                                           long long plane_batch_bytes, int ksplit) {
    grid_launch_dependents();
    grid_dependency_wait();
    __shared__ int s_pop[8][8];         // [warp][row of the group]: partial row sums of the warps that share a group
    __shared__ float s_mag[8][8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kpart = warp % ksplit, rg = lane >> 2, cp = lane & 3;
    const long long group = (long long)blockIdx.x * (8 / ksplit) + warp / ksplit;
    const long long row = group * 8 + rg;
    const long long batch = blockIdx.y;
    const long long mtiles = (M + 127) / 128, kblocks = (K + 255) / 256;
    const bool in_plane = row < mtiles * 128;
    const bool live = row < M;
    src += batch * src_batch_stride;
    plane += batch * plane_batch_bytes;
    const T* rp = src + row * ld;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(rp) & (sizeof(T) == 1 ? 7 : 15)) == 0;     // a piece is loaded as one or two vectors
    const bool want_mag = alpha != nullptr;
    uint8_t* dst = plane + (row / 128) * kblocks * 4096 + (cp >> 1) * 2048 + (int)(row % 128) * 16 + (cp & 1) * 8;
    int pop = 0;
    float mag = 0.f;
    constexpr int U = sizeof(T) <= 2 ? 2 : 1;       // K blocks in flight per warp (16 loads of 8 or 16 bytes per lane; fp32: 16 of 16)
    for (long long kb0 = kpart; kb0 < kblocks; kb0 += (long long)ksplit * U) {
        RawBlock<T> raw[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const long long kb = kb0 + (long long)u * ksplit;
            if (kb < kblocks) load_block(raw[u], rp, kb * 256 + 8 * cp, K, live, vec_ok);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const long long kb = kb0 + (long long)u * ksplit;
            if (kb >= kblocks) break;
            uint32_t w0, w1;
            bits_of_block(raw[u], kb * 256 + 8 * cp, K, live, vec_ok, mode, want_mag, w0, w1, mag);
            pop += __popc(w0) + __popc(w1);
            if (in_plane) *reinterpret_cast<uint2*>(dst + kb * 4096) = make_uint2(w0, w1);
        }
    }
    if (rowpop || alpha) {
        pop += __shfl_xor_sync(0xffffffffu, pop, 1);
        pop += __shfl_xor_sync(0xffffffffu, pop, 2);
        mag += __shfl_xor_sync(0xffffffffu, mag, 1);
        mag += __shfl_xor_sync(0xffffffffu, mag, 2);
        if (ksplit > 1) {
            if (cp == 0) {
                s_pop[warp][rg] = pop;
                s_mag[warp][rg] = mag;
            }
            __syncthreads();
            if (kpart == 0 && cp == 0) {
                for (int i = 1; i < ksplit; i++) {
                    pop += s_pop[warp + i][rg];
                    mag += s_mag[warp + i][rg];
                }
            }
        }
        if (kpart == 0 && cp == 0 && live) {
            if (rowpop) rowpop[batch * M + row] = pop;
            if (alpha) alpha[batch * M + row] = __float2half_rn(mag / (float)K);
        }
    }
}

// ---- activations -> int8 rows + colsum ----------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ int8_t act_value(const T& v, int mode) {
    const int neg = Elem<T>::neg(v);
    if (mode == BGEMM_ACT_SIGN) return (int8_t)(1 - 2 * neg);
    if (mode == BGEMM_ACT_TERNARY) return Elem<T>::zero(v) ? (int8_t)0 : (int8_t)(1 - 2 * neg);
    if (mode == BGEMM_ACT_INT8) return Elem<T>::as_int8(v);        // int8 sources only (checked at the entry point)
    return (int8_t)neg;
}

// Eight 16-bit floats (fp16 or bf16: same sign / zero tests) -> eight int8 activation values, two elements per 32-bit
// operation. Per 16-bit lane: t = "not +-0", s = sign bit; the value byte is 0x00, 0x01 or 0xFF (= 0x01 | 0xFE).
// Returns the signed sum of the eight values as well (dp4a).
__device__ __forceinline__ uint2 act_values_x8(const uint4& w, int mode, int& sum) {
    const uint32_t in[4] = {w.x, w.y, w.z, w.w};
    uint32_t b[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t s = (in[i] >> 15) & 0x00010001u;
        if (mode == BGEMM_ACT_NEG01) {
            b[i] = s;
        } else {
            const uint32_t mag = in[i] & 0x7fff7fffu;
            const uint32_t t = mode == BGEMM_ACT_SIGN ? 0x00010001u : (((mag + 0x7fff7fffu) >> 15) & 0x00010001u);
            const uint32_t m = t & s;
            b[i] = t | ((m << 8) - (m << 1));
        }
    }
    uint2 o;
    o.x = __byte_perm(b[0], b[1], 0x6420);      // low bytes of the four 16-bit lanes, in element order
    o.y = __byte_perm(b[2], b[3], 0x6420);
    sum = __dp4a((int)o.x, 0x01010101, sum);
    sum = __dp4a((int)o.y, 0x01010101, sum);
    return o;
}

// Eight int8 source values -> eight int8 activation values, four elements per 32-bit operation (per-byte compares).
__device__ __forceinline__ uint2 act_values_i8x8(const uint2& w, int mode, int& sum) {
    const uint32_t in[2] = {w.x, w.y};
    uint32_t o[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const uint32_t neg = __vcmplts4(in[i], 0u);                 // 0xff where the byte is negative
        if (mode == BGEMM_ACT_INT8) o[i] = in[i];
        else if (mode == BGEMM_ACT_NEG01) o[i] = neg & 0x01010101u;
        else if (mode == BGEMM_ACT_SIGN) o[i] = neg | 0x01010101u;  // 0xff (-1) or 0x01 (+1)
        else o[i] = neg | (__vcmpne4(in[i], 0u) & 0x01010101u);     // torch.sign: 0xff, 0x00, 0x01
        sum = __dp4a((int)o[i], 0x01010101, sum);
    }
    return make_uint2(o[0], o[1]);
}

// Activation rows (rows of all batches numbered through) -> int8 rows + column sums. The launcher picks the split:
// many rows: a warp converts `rows_per_warp` consecutive rows, sized so that the launch is one resident wave (with
// one short row per warp a launch of 1.3 waves ran its last third on a nearly idle GPU); few rows: `warps_per_row`
// (2, 4 or 8) warps of a CTA share a row by 256-column blocks and add their partial sums through shared memory, so
// that a handful of long rows still puts loads from every SM in flight. A lane handles 8 consecutive elements per
// step (one 16-byte streaming load for 2-byte types, one 8-byte store) and keeps eight such loads in flight.
template <typename T>
__global__ void __launch_bounds__(256, 4) prepare_acts_kernel(const T* __restrict__ src, long long N, long long K, long long ld, int mode,
                                                           int8_t* __restrict__ dst, int32_t* __restrict__ colsum,
                                                           long long src_batch_stride, long long total_rows, int rows_per_warp,
                                                           int warps_per_row) {
    __shared__ int part[8];
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const long long kld = (K + 255) / 256 * 256;
    const long long kblocks = kld / 256;
    constexpr int U = 8;
    // rows [r0, r1) and 256-column blocks [b0, b1) of this warp
    long long r0, r1, b0 = 0, b1 = kblocks;
    if (warps_per_row > 1) {
        const int rows_per_cta = 8 / warps_per_row, slice = wib % warps_per_row;
        r0 = (long long)blockIdx.x * rows_per_cta + wib / warps_per_row;
        r1 = r0 + 1;
        const long long per = (kblocks + warps_per_row - 1) / warps_per_row;
        b0 = slice * per;
        b1 = b0 + per < kblocks ? b0 + per : kblocks;
    } else {
        r0 = ((long long)blockIdx.x * 8 + wib) * rows_per_warp;
        r1 = r0 + rows_per_warp;
    }
    for (long long gr = r0; gr < r1; gr++) {
        int sum = 0;
        if (gr < total_rows) {
            const long long batch = gr / N, row = gr - batch * N;
            const T* rp = src + batch * src_batch_stride + row * ld;
            int8_t* dp = dst + gr * kld;
            const bool vec_ok = (sizeof(T) == 2) && ((reinterpret_cast<uintptr_t>(rp) & 15) == 0);
            const bool vec8_ok = (sizeof(T) == 1) && ((reinterpret_cast<uintptr_t>(rp) & 7) == 0);
            for (long long kbase = b0 * 256 + lane * 8; kbase < b1 * 256; kbase += 256 * U) {
                if (vec_ok && kbase + 256 * (U - 1) + 8 <= K && kbase + 256 * (U - 1) < b1 * 256) {
                    // all U blocks inside the row and the slice: loads first, then two elements per operation
                    uint4 v[U];
#pragma unroll
                    for (int u = 0; u < U; u++) v[u] = __ldcs(reinterpret_cast<const uint4*>(rp + kbase + 256 * u));
#pragma unroll
                    for (int u = 0; u < U; u++) *reinterpret_cast<uint2*>(dp + kbase + 256 * u) = act_values_x8(v[u], mode, sum);
                    continue;
                }
                if (vec8_ok && kbase + 256 * (U - 1) + 8 <= K && kbase + 256 * (U - 1) < b1 * 256) {
                    // int8 sources: the same with 8-byte loads and four elements per operation
                    uint2 v[U];
#pragma unroll
                    for (int u = 0; u < U; u++) v[u] = __ldcs(reinterpret_cast<const uint2*>(rp + kbase + 256 * u));
#pragma unroll
                    for (int u = 0; u < U; u++) *reinterpret_cast<uint2*>(dp + kbase + 256 * u) = act_values_i8x8(v[u], mode, sum);
                    continue;
                }
#pragma unroll 1
                for (int u = 0; u < U; u++) {                     // ragged tail, other element types, unaligned rows
                    const long long k0 = kbase + 256 * u;
                    if (k0 >= b1 * 256) break;
                    int8_t o[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        o[e] = (k0 + e < K) ? act_value<T>(rp[k0 + e], mode) : (int8_t)0;
                        sum += o[e];
                    }
                    *reinterpret_cast<uint2*>(dp + k0) = *reinterpret_cast<const uint2*>(o);
                }
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        if (warps_per_row > 1) {          // one row per warp group, one pass: every warp of the CTA reaches the barriers
            if (lane == 0) part[wib] = sum;
            __syncthreads();
            if (lane == 0 && wib % warps_per_row == 0 && gr < total_rows) {
                int tot = 0;
                for (int i = 0; i < warps_per_row; i++) tot += part[wib + i];
                colsum[gr] = tot;
            }
        } else if (lane == 0 && gr < total_rows) {
            colsum[gr] = sum;
        }
    }
}

// Transposing variant: source is [K, N]. A CTA owns 64 output rows (n) and walks K in tiles of 128. Thread (kq, nc)
// reads four source rows k = 4 kq .. 4 kq + 3 at columns 8 nc .. 8 nc + 7 (one 16-byte load per row for 2-byte types; the
// eight threads of a row cover 128 contiguous bytes), converts them, transposes the 4 x 8 bytes in registers with byte
// permutes and writes eight 32-bit words (four consecutive k of one n each) into a [64][32 + 1]-word tile; the tile
// leaves as 16-byte stores, 128 contiguous bytes per output row. Column sums are kept per thread (dp4a over each word)
// and meet in shared memory. With `kparts` > 1 the K tiles are divided over gridDim.z and the sums are added to a
// zeroed `colsum` atomically (integers: the result does not depend on the order).
template <typename T>
__global__ void __launch_bounds__(256) prepare_acts_t_kernel(const T* __restrict__ src, long long N, long long K, long long ld, int mode,
                                                             int8_t* __restrict__ dst, int32_t* __restrict__ colsum,
                                                             long long src_batch_stride, int kparts) {
    __shared__ uint32_t tile[64][33];
    __shared__ int s_col[64];
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = threadIdx.x, nc = t & 7, kq = t >> 3;
    const long long n0 = (long long)blockIdx.x * 64;
    const long long batch = blockIdx.y;
    const long long kld = (K + 255) / 256 * 256, ktiles = kld / 128;
    const long long kt_begin = ktiles * blockIdx.z / kparts, kt_end = ktiles * (blockIdx.z + 1) / kparts;
    const T* sp = src + batch * src_batch_stride;
    int8_t* dp = dst + batch * N * kld;
    const bool vec_ok = sizeof(T) == 2 && (reinterpret_cast<uintptr_t>(sp) & 15) == 0 && (ld * (long long)sizeof(T)) % 16 == 0;
    const long long nbase = n0 + 8 * nc;
    if (t < 64) s_col[t] = 0;
    int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long kt = kt_begin; kt < kt_end; kt++) {
        const long long k0 = kt * 128, kbase = k0 + 4 * kq;
        uint2 b[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const long long k = kbase + i;
            if (sizeof(T) == 2 && vec_ok && k < K && nbase + 8 <= N) {
                int unused = 0;
                b[i] = act_values_x8(__ldcs(reinterpret_cast<const uint4*>(sp + k * ld + nbase)), mode, unused);
            } else {
                uint32_t w[2] = {0u, 0u};
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    if (k < K && nbase + e < N) w[e >> 2] |= (uint32_t)(uint8_t)act_value<T>(sp[k * ld + nbase + e], mode) << (8 * (e & 3));
                }
                b[i] = make_uint2(w[0], w[1]);
            }
        }
        uint32_t out[8];
        {
            const uint32_t lo01 = __byte_perm(b[0].x, b[1].x, 0x5140), hi01 = __byte_perm(b[0].x, b[1].x, 0x7362);
            const uint32_t lo23 = __byte_perm(b[2].x, b[3].x, 0x5140), hi23 = __byte_perm(b[2].x, b[3].x, 0x7362);
            out[0] = __byte_perm(lo01, lo23, 0x5410);
            out[1] = __byte_perm(lo01, lo23, 0x7632);
            out[2] = __byte_perm(hi01, hi23, 0x5410);
            out[3] = __byte_perm(hi01, hi23, 0x7632);
        }
        {
            const uint32_t lo01 = __byte_perm(b[0].y, b[1].y, 0x5140), hi01 = __byte_perm(b[0].y, b[1].y, 0x7362);
            const uint32_t lo23 = __byte_perm(b[2].y, b[3].y, 0x5140), hi23 = __byte_perm(b[2].y, b[3].y, 0x7362);
            out[4] = __byte_perm(lo01, lo23, 0x5410);
            out[5] = __byte_perm(lo01, lo23, 0x7632);
            out[6] = __byte_perm(hi01, hi23, 0x5410);
            out[7] = __byte_perm(hi01, hi23, 0x7632);
        }
#pragma unroll
        for (int e = 0; e < 8; e++) {
            acc[e] = __dp4a((int)out[e], 0x01010101, acc[e]);
            tile[8 * nc + e][kq] = out[e];
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int idx = t + 256 * h, nl = idx >> 3, c = idx & 7;
            if (n0 + nl < N)
                *reinterpret_cast<uint4*>(dp + (n0 + nl) * kld + k0 + 16 * c) =
                    make_uint4(tile[nl][4 * c], tile[nl][4 * c + 1], tile[nl][4 * c + 2], tile[nl][4 * c + 3]);
        }
        __syncthreads();
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; e++) atomicAdd(&s_col[8 * nc + e], acc[e]);
    __syncthreads();
    if (t < 64 && n0 + t < N) {
        if (kparts > 1) atomicAdd(&colsum[batch * N + n0 + t], s_col[t]);
        else colsum[batch * N + n0 + t] = s_col[t];
    }
}

// ---- reference-compatible row-major prepack: element k -> bit 31 - k % 32 of word k / 32 --------------------
template <typename T>
__global__ void __launch_bounds__(256) pack_rowmajor_msb_kernel(const T* __restrict__ src, long long rows, long long K, long long ld,
                                                                uint32_t* __restrict__ dst) {
    const int lane = threadIdx.x & 31;
    const long long words = K / 32;
    const long long warp_id = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long w = warp_id; w < rows * words; w += nwarps) {
        const long long r = w / words, c = w % words;
        const int neg = Elem<T>::neg(src[r * ld + c * 32 + lane]);
        const uint32_t ballot = __ballot_sync(0xffffffffu, neg);
        if (lane == 0) dst[w] = __brev(ballot);
    }
}

// Row-major MSB-first words -> tiled plane. One thread per (row, 256-column block).
__global__ void __launch_bounds__(256) retile_kernel(const uint32_t* __restrict__ src, long long M, long long K, int invert,
                                                     uint8_t* __restrict__ plane) {
    const long long mtiles = (M + 127) / 128, kblocks = (K + 255) / 256, words = K / 32;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= mtiles * 128 * kblocks) return;
    const long long row = idx / kblocks, kb = idx % kblocks;
    uint32_t out[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (row < M) {
        for (int j = 0; j < 8; j++) {
            const long long wi = kb * 8 + j;
            if (wi >= words) break;
            uint32_t s = src[row * words + wi];
            if (invert) s = ~s;
            for (int t = 0; t < 32; t++) {   // element k = 32 j + t sits at bit 31 - t; t = 4 c + b
                const uint32_t bit = (s >> (31 - t)) & 1u;
                out[t >> 2] |= bit << (8 * (t & 3) + j);
            }
        }
    }
    uint8_t* tile = plane + ((row / 128) * kblocks + kb) * 4096;
    const int r = (int)(row % 128);
    *reinterpret_cast<uint4*>(tile + tile_word_offset(r, 0)) = make_uint4(out[0], out[1], out[2], out[3]);
    *reinterpret_cast<uint4*>(tile + tile_word_offset(r, 4)) = make_uint4(out[4], out[5], out[6], out[7]);
}

// ---- launchers --------------------------------------------------------------------------------------------
#define BGEMM_DISPATCH_DTYPE(dtype, ...)                                            \
    switch (dtype) {                                                                \
        case BGEMM_DT_F16: { using T = __half; __VA_ARGS__; break; }                \
        case BGEMM_DT_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; }        \
        case BGEMM_DT_F32: { using T = float; __VA_ARGS__; break; }                 \
        case BGEMM_DT_I8: { using T = int8_t; __VA_ARGS__; break; }                 \
        default: return BGEMM_ERR_ENUM;                                             \
    }

int launch_pack_weights(cudaStream_t stream, const void* src, int dtype, long long M, long long K, long long ld, int wbit_mode,
                        void* plane, int32_t* rowpop, void* alpha, long long batch, long long src_batch_stride) {
    // Groups of eight rows, one warp each; with fewer groups than fill the GPU, up to eight warps share a group by K blocks.
    const long long groups = (M + 127) / 128 * 16, kblocks = (K + 255) / 256;
    int ksplit = 1;
    while (ksplit < 8 && groups * batch * ksplit < 16LL * sm_count() && 2 * ksplit <= kblocks) ksplit *= 2;
    dim3 grid((unsigned)(groups / (8 / ksplit)), (unsigned)batch);
    const long long pbytes = (long long)bgemm_plane_bytes(M, K);
    cudaError_t e = cudaSuccess;
    BGEMM_DISPATCH_DTYPE(dtype, (e = launch_pdl(pack_weights_kernel<T>, grid, dim3(256), stream, static_cast<const T*>(src), M, K, ld, wbit_mode,
                                                static_cast<uint8_t*>(plane), rowpop, static_cast<__half*>(alpha), src_batch_stride, pbytes,
                                                ksplit)));
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_prepare_acts(cudaStream_t stream, const void* src, int dtype, long long N, long long K, long long ld, int act_mode,
                        int transpose, int8_t* dst, int32_t* colsum, long long batch, long long src_batch_stride) {
    cudaError_t e = cudaSuccess;
    if (transpose) {
        // One CTA per 64 output rows and problem; with fewer CTAs than SMs the K tiles of a source of some size (2^20
        // elements or more: the memset of the sums costs about as much as a small kernel) are divided over gridDim.z as well.
        const long long ctas = (N + 63) / 64 * batch, ktiles = (K + 255) / 256 * 2;
        int kparts = 1;
        while (N * K * batch >= (1LL << 20) && kparts < 32 && ctas * kparts < sm_count() && 2 * kparts <= ktiles) kparts *= 2;
        if (kparts > 1) {
            e = cudaMemsetAsync(colsum, 0, sizeof(int32_t) * (size_t)(N * batch), stream);
            if (e != cudaSuccess) return (int)e;
        }
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)batch, (unsigned)kparts);
        BGEMM_DISPATCH_DTYPE(dtype, (e = launch_pdl(prepare_acts_t_kernel<T>, grid, dim3(256), stream, static_cast<const T*>(src), N, K, ld, act_mode,
                                                    dst, colsum, src_batch_stride, kparts)));
    } else {
        // At most one resident wave of 8-warp CTAs (4 per SM): longer launches give every warp several rows, launches
        // far below a wave split every row over 2, 4 or 8 warps.
        const long long total_rows = N * batch, wave_warps = (long long)sm_count() * 32;
        int rows_per_warp = 1, warps_per_row = 1;
        if (total_rows > wave_warps) {
            rows_per_warp = (int)((total_rows + wave_warps - 1) / wave_warps);
        } else {
            const long long kblocks = (K + 255) / 256;
            while (warps_per_row < 8 && total_rows * warps_per_row * 2 <= wave_warps && kblocks >= warps_per_row * 2 * 2) warps_per_row *= 2;
        }
        const long long ctas = warps_per_row > 1 ? (total_rows * warps_per_row + 7) / 8 : ((total_rows + rows_per_warp - 1) / rows_per_warp + 7) / 8;
        dim3 grid((unsigned)ctas);
        BGEMM_DISPATCH_DTYPE(dtype, (e = launch_pdl(prepare_acts_kernel<T>, grid, dim3(256), stream, static_cast<const T*>(src), N, K, ld, act_mode, dst,
                                                    colsum, src_batch_stride, total_rows, rows_per_warp, warps_per_row)));
    }
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

int launch_pack_rowmajor_msb(cudaStream_t stream, const void* src, int dtype, long long rows, long long K, long long ld, uint32_t* dst) {
    const long long total = rows * (K / 32);
    long long blocks = (total + 7) / 8;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    BGEMM_DISPATCH_DTYPE(dtype, (pack_rowmajor_msb_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(static_cast<const T*>(src), rows, K, ld, dst)));
    count_launch();
    return (int)cudaGetLastError();
}

int launch_retile(cudaStream_t stream, const uint32_t* src_words, long long M, long long K, int invert, void* plane) {
    const long long total = (M + 127) / 128 * 128 * ((K + 255) / 256);
    retile_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(src_words, M, K, invert, static_cast<uint8_t*>(plane));
    count_launch();
    return (int)cudaGetLastError();
}

// ---- CPU twins (host pointers) ------------------------------------------------------------------------------
template <typename T> static int host_neg(const T* p) { return Elem<T>::neg(*p); }
static float host_mag(const void* p, int dtype) {
    switch (dtype) {
        case BGEMM_DT_F16: return fabsf(__half2float(*static_cast<const __half*>(p)));
        case BGEMM_DT_BF16: return fabsf(__bfloat162float(*static_cast<const __nv_bfloat16*>(p)));
        case BGEMM_DT_F32: return fabsf(*static_cast<const float*>(p));
        default: return fabsf((float)*static_cast<const int8_t*>(p));
    }
}
static int host_neg_any(const void* p, int dtype) {
    switch (dtype) {
        case BGEMM_DT_F16: return host_neg(static_cast<const __half*>(p));
        case BGEMM_DT_BF16: return host_neg(static_cast<const __nv_bfloat16*>(p));
        case BGEMM_DT_F32: return host_neg(static_cast<const float*>(p));
        default: return host_neg(static_cast<const int8_t*>(p));
    }
}
static int host_bit_any(const void* p, int dtype, int mode) {
    switch (dtype) {
        case BGEMM_DT_F16: return weight_bit(*static_cast<const __half*>(p), mode);
        case BGEMM_DT_BF16: return weight_bit(*static_cast<const __nv_bfloat16*>(p), mode);
        case BGEMM_DT_F32: return weight_bit(*static_cast<const float*>(p), mode);
        default: return weight_bit(*static_cast<const int8_t*>(p), mode);
    }
}
static size_t dtype_size(int dtype) { return dtype == BGEMM_DT_F32 ? 4 : (dtype == BGEMM_DT_I8 ? 1 : 2); }

}  // namespace bgemm

using namespace bgemm;

extern "C" int bgemm_pack_weights_host(const void* src, int dtype, int64_t M, int64_t K, int64_t ld, int wbit_mode, void* plane,
                                       int32_t* rowpop, void* alpha) {
    if (!src || !plane) return BGEMM_ERR_NULL;
    if (M < 1 || K < 1 || ld < K) return BGEMM_ERR_SHAPE;
    if (dtype < 0 || dtype > 3 || wbit_mode < 0 || wbit_mode > 3) return BGEMM_ERR_ENUM;
    const int64_t kblocks = (K + 255) / 256;
    std::memset(plane, 0, bgemm_plane_bytes(M, K));
    const size_t es = dtype_size(dtype);
    const char* s = static_cast<const char*>(src);
    for (int64_t m = 0; m < M; m++) {
        int pop = 0;
        double mag = 0.0;
        uint8_t* tile_row = static_cast<uint8_t*>(plane) + (m / 128) * kblocks * 4096;
        const int r = (int)(m % 128);
        for (int64_t k = 0; k < K; k++) {
            const void* e = s + (size_t)(m * ld + k) * es;
            const int bit = host_bit_any(e, dtype, wbit_mode);
            if (alpha) mag += host_mag(e, dtype);
            if (!bit) continue;
            pop++;
            const int64_t kb = k / 256;
            const int kk = (int)(k % 256), j = kk / 32, c = (kk % 32) / 4, b = kk % 4;
            uint32_t* w = reinterpret_cast<uint32_t*>(tile_row + kb * 4096 + tile_word_offset(r, c));
            *w |= 1u << (8 * b + j);
        }
        if (rowpop) rowpop[m] = pop;
        if (alpha) static_cast<__half*>(alpha)[m] = __float2half_rn((float)(mag / (double)K));
    }
    return BGEMM_OK;
}

extern "C" int bgemm_pack_rowmajor_msb_host(const void* src, int dtype, int64_t rows, int64_t K, int64_t ld, uint32_t* dst) {
    if (!src || !dst) return BGEMM_ERR_NULL;
    if (rows < 1 || K < 32 || K % 32 != 0 || ld < K) return BGEMM_ERR_SHAPE;
    if (dtype < 0 || dtype > 3) return BGEMM_ERR_ENUM;
    const size_t es = dtype_size(dtype);
    const char* s = static_cast<const char*>(src);
    for (int64_t r = 0; r < rows; r++)
        for (int64_t w = 0; w < K / 32; w++) {
            uint32_t v = 0;
            for (int t = 0; t < 32; t++) v |= (uint32_t)host_neg_any(s + (size_t)(r * ld + w * 32 + t) * es, dtype) << (31 - t);
            dst[r * (K / 32) + w] = v;
        }
    return BGEMM_OK;
}
