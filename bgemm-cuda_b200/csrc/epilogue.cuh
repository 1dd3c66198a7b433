// Epilogue helpers shared by the GEMM kernels: an accumulator tile staged in shared (or global) memory as
// int32 [columns][128] is summed over K partitions, mapped to the op's result (D or colsum - 2 D), scaled per row
// where asked, and stored with 16-byte coalesced stores in either output layout -- or turned straight into the next
// layer's int8 activations and their row sums.
#pragma once
#include <cuda_fp16.h>

#include "internal.h"

namespace bgemm {

// ---- epilogue: converting and storing 8 results --------------------------------------------------------------
struct TileOut {
    const GemmParams* p;
    const float* s_alpha;    // [128] per-row scale of this tile (1 when unused)
    const int* s_colsum;     // [NT] column sums of this tile (0 when unused)
    int batch, m_base, n_base;
    bool streaming = false;  // results are written with streaming stores (first out of L2): for kernels that keep other data there
};
__device__ __forceinline__ void store16B(void* dst, const uint4& v, bool streaming) {
    if (streaming) __stcs(reinterpret_cast<uint4*>(dst), v);
    else *reinterpret_cast<uint4*>(dst) = v;
}

// 8 consecutive rows m0..m0+7 (tile-local) of column n (tile-local): the [N, M] layout.
__device__ __forceinline__ void store8_rows(const TileOut& t, int n, int m0, const int (&acc)[8]) {
    const GemmParams& p = *t.p;
    const int gn = t.n_base + n, gm = t.m_base + m0;
    if (gn >= p.N || gm >= p.M) return;
    const int cs = t.s_colsum[n];
    int val[8];
#pragma unroll
    for (int q = 0; q < 8; q++) val[q] = p.epi ? cs - 2 * acc[q] : acc[q];
    const size_t idx = (size_t)t.batch * p.M * p.N + (size_t)gn * p.ldo + gm;
    const bool full = gm + 8 <= p.M;
    if (p.out_kind == kOutActs) return;       // handled by store8_rows_as_acts
    if (p.out_kind == BGEMM_OUT_I32) {
        auto put = [&](void* base) {
            int* o = reinterpret_cast<int*>(base) + idx;
            if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
                store16B(o, make_uint4((uint32_t)val[0], (uint32_t)val[1], (uint32_t)val[2], (uint32_t)val[3]), t.streaming);
                store16B(o + 4, make_uint4((uint32_t)val[4], (uint32_t)val[5], (uint32_t)val[6], (uint32_t)val[7]), t.streaming);
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) if (gm + q < p.M) o[q] = val[q];
            }
        };
        put(p.out);
        // further destinations (peer-mapped copies of the result: plain stores over NVLink); none in the common case
#pragma unroll 1
        for (int d = 0; d < p.n_out_more; d++) put(p.out_more[d]);
    } else {
        __align__(16) __half h[8];
#pragma unroll
        for (int q = 0; q < 8; q++)
            h[q] = __float2half_rn(p.out_kind == BGEMM_OUT_F16 ? (float)val[q] : (float)val[q] * t.s_alpha[m0 + q]);
        auto put = [&](void* base) {
            __half* o = reinterpret_cast<__half*>(base) + idx;
            if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
                store16B(o, *reinterpret_cast<const uint4*>(h), t.streaming);
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) if (gm + q < p.M) o[q] = h[q];
            }
        };
        put(p.out);
#pragma unroll 1
        for (int d = 0; d < p.n_out_more; d++) put(p.out_more[d]);
    }
}

// The same 8 results written as the next layer's activations: act(fp16 result) as int8 at row n of an [N, out_ld]
// matrix (columns = this GEMM's rows m). The fp16 result is rounded exactly as the fp16 output kinds round it, so
// the bytes equal prepare_acts applied to that output. Returns the sum of the 8 values (0 for a unit outside the
// matrix); rows beyond M inside the chunk are written as zero padding.
__device__ __forceinline__ int store8_rows_as_acts(const TileOut& t, int n, int m0, const int (&acc)[8], bool valid) {
    const GemmParams& p = *t.p;
    const int gn = t.n_base + n, gm = t.m_base + m0;
    if (!valid) return 0;
    const int cs = t.s_colsum[n];
    int sum = 0;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const int val = p.epi ? cs - 2 * acc[q] : acc[q];
        const __half hv = __float2half_rn(p.alpha ? (float)val * t.s_alpha[m0 + q] : (float)val);
        const uint32_t bits = __half_as_ushort(hv);
        const int neg = (int)(bits >> 15), zero = (bits & 0x7fffu) == 0;
        int v = p.act_mode == BGEMM_ACT_SIGN ? 1 - 2 * neg : (p.act_mode == BGEMM_ACT_TERNARY ? (zero ? 0 : 1 - 2 * neg) : neg);
        if (gm + q >= p.M) v = 0;
        sum += v;
        w[q >> 2] |= (uint32_t)(v & 0xff) << (8 * (q & 3));
    }
    int8_t* o = reinterpret_cast<int8_t*>(p.out) + ((size_t)t.batch * p.N + gn) * p.out_ld + gm;
    *reinterpret_cast<uint2*>(o) = make_uint2(w[0], w[1]);      // gm is a multiple of 8, the pitch of 256
    return sum;
}

// 8 consecutive columns n0..n0+7 (tile-local) of row m (tile-local): the [M, N] layout.
__device__ __forceinline__ void store8_cols(const TileOut& t, int m, int n0, const int (&acc)[8]) {
    const GemmParams& p = *t.p;
    const int gm = t.m_base + m, gn = t.n_base + n0;
    if (gm >= p.M || gn >= p.N) return;
    int val[8];
#pragma unroll
    for (int q = 0; q < 8; q++) val[q] = p.epi ? t.s_colsum[n0 + q] - 2 * acc[q] : acc[q];
    const size_t idx = (size_t)t.batch * p.M * p.N + (size_t)gm * p.ldo + gn;
    const bool full = gn + 8 <= p.N;
    if (p.out_kind == BGEMM_OUT_I32) {
        auto put = [&](void* base) {
            int* o = reinterpret_cast<int*>(base) + idx;
            if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
                store16B(o, make_uint4((uint32_t)val[0], (uint32_t)val[1], (uint32_t)val[2], (uint32_t)val[3]), t.streaming);
                store16B(o + 4, make_uint4((uint32_t)val[4], (uint32_t)val[5], (uint32_t)val[6], (uint32_t)val[7]), t.streaming);
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) if (gn + q < p.N) o[q] = val[q];
            }
        };
        put(p.out);
#pragma unroll 1
        for (int d = 0; d < p.n_out_more; d++) put(p.out_more[d]);
    } else {
        const float a = t.s_alpha[m];
        __align__(16) __half h[8];
#pragma unroll
        for (int q = 0; q < 8; q++) h[q] = __float2half_rn(p.out_kind == BGEMM_OUT_F16 ? (float)val[q] : (float)val[q] * a);
        auto put = [&](void* base) {
            __half* o = reinterpret_cast<__half*>(base) + idx;
            if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
                store16B(o, *reinterpret_cast<const uint4*>(h), t.streaming);
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) if (gn + q < p.N) o[q] = h[q];
            }
        };
        put(p.out);
#pragma unroll 1
        for (int d = 0; d < p.n_out_more; d++) put(p.out_more[d]);
    }
}

// [M, N] results of an unpartitioned tile in the tile-per-CTA kernel: the accumulator tile is staged ROW-major,
// [128 rows][row_pitch_of(NT)] int32 (an accumulator row leaves tensor memory as consecutive columns, so the staging
// stores are 16-byte vectors), and consecutive threads take consecutive 8-column chunks of a row: both the shared-memory
// reads and the global stores of a warp are contiguous runs. (Storing straight from registers, as the persistent kernel
// does with its four dedicated epilogue warps, measured slower here: 42 against 36 us on the batched attention product.)
__host__ __device__ constexpr int row_pitch_of(int nt) { return nt + 4; }      // (pitch / 4) odd: 16-byte row accesses spread over all banks
template <int NT>
__device__ __forceinline__ void write_tile_rowmajor(const TileOut& t, const int* staged, int et, int nthreads) {
    constexpr int CH = NT / 8, PITCH = row_pitch_of(NT);
#pragma unroll 1
    for (int u = et; u < 128 * CH; u += nthreads) {
        const int m = u / CH, c0 = (u - m * CH) * 8;
        const int4* g = reinterpret_cast<const int4*>(staged + m * PITCH + c0);
        const int4 a = g[0], b = g[1];
        const int acc[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        store8_cols(t, m, c0, acc);
    }
}

// Sum `parts` partial tiles (each `stride` ints apart, starting at `base`) over 8 consecutive rows at element
// offset `off` of a [columns][128] int32 tile. GLOBAL: the tiles are slabs in global memory (L2 reads).
template <bool GLOBAL>
__device__ __forceinline__ void gather8_rows(const int* base, int parts, int stride, int off, int (&acc)[8]) {
#pragma unroll
    for (int q = 0; q < 8; q++) acc[q] = 0;
#pragma unroll 4
    for (int s = 0; s < parts; s++) {
        const int4* g = reinterpret_cast<const int4*>(base + (size_t)s * stride + off);
        const int4 a = GLOBAL ? __ldcg(g) : g[0];
        const int4 b = GLOBAL ? __ldcg(g + 1) : g[1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
}

// The same over 8 consecutive columns c0..c0+7 of row m.
template <bool GLOBAL>
__device__ __forceinline__ void gather8_cols(const int* base, int parts, int stride, int c0, int m, int (&acc)[8]) {
#pragma unroll
    for (int q = 0; q < 8; q++) acc[q] = 0;
#pragma unroll 2
    for (int s = 0; s < parts; s++) {
        const int* g = base + (size_t)s * stride + c0 * 128 + m;
#pragma unroll
        for (int q = 0; q < 8; q++) acc[q] += GLOBAL ? __ldcg(g + q * 128) : g[q * 128];
    }
}

// Convert and store `ncols` columns with `nthreads` epilogue threads (`et` = this thread's index among them).
// Column c of the partial tiles at `base` is tile column n_first + c.
template <bool GLOBAL>
__device__ __forceinline__ void write_tile(const TileOut& t, const int* base, int parts, int stride, int n_first, int ncols, int et, int nthreads) {
    const GemmParams& p = *t.p;
    if (p.out_layout == BGEMM_LAYOUT_NM) {
        const int units = ncols * 16;                           // (column, 8-row chunk)
        if (p.out_kind == kOutActs) {
            // Every lane runs every iteration (the row sums are reduced with warp shuffles over the 16 lanes that
            // share a column); one atomic per column and tile.
#pragma unroll 1
            for (int u0 = 0; u0 < units; u0 += nthreads) {
                const int u = u0 + et;
                const int c = u >> 4, m0 = (u & 15) * 8;
                const bool valid = u < units && t.n_base + n_first + c < p.N && t.m_base + m0 < p.M;
                int acc[8];
                if (valid) gather8_rows<GLOBAL>(base, parts, stride, c * 128 + m0, acc);
                int sum = store8_rows_as_acts(t, n_first + c, m0, acc, valid);
#pragma unroll
                for (int off = 8; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
                if ((et & 15) == 0 && u < units && t.n_base + n_first + c < p.N)
                    atomicAdd(p.colsum_next + (size_t)t.batch * p.N + t.n_base + n_first + c, sum);
            }
            return;
        }
#pragma unroll 1
        for (int u = et; u < units; u += nthreads) {
            const int c = u >> 4, m0 = (u & 15) * 8;
            if (t.n_base + n_first + c >= p.N || t.m_base + m0 >= p.M) continue;
            int acc[8];
            gather8_rows<GLOBAL>(base, parts, stride, c * 128 + m0, acc);
            store8_rows(t, n_first + c, m0, acc);
        }
    } else {
        const int units = (ncols >> 3) * 128;                   // (8-column chunk, row)
#pragma unroll 1
        for (int u = et; u < units; u += nthreads) {
            const int m = u & 127, c0 = (u >> 7) * 8;
            if (t.n_base + n_first + c0 >= p.N || t.m_base + m >= p.M) continue;
            int acc[8];
            gather8_cols<GLOBAL>(base, parts, stride, c0, m, acc);
            store8_cols(t, m, n_first + c0, acc);
        }
    }
}

}  // namespace bgemm
