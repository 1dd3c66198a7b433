// Persistent binary-weight GEMM on CTA pairs (tcgen05.mma.cta_group::2) for wide activation matrices: the two CTAs of
// a cluster -- the two SMs of a TPC -- compute one 256(M) x 256(N) tile together. Each CTA streams and unpacks ITS OWN
// 128 weight rows into its own tensor memory and loads only HALF of the activation tile (128 of the 256 activation
// rows) into its own shared memory; one thread of the even CTA issues a single 256 x 256 x 32 UMMA for both SMs, which
// reads both halves. Against the 128-row kernels each SM pulls half the activation bytes from L2 per unit of tensor
// work (36 KB per 1024 clocks of UMMA instead of 36 KB per 512), the issuing thread spends one instruction per 128
// clocks of tensor work instead of one per 64, and the tensor-memory stores of the unpacked weights -- which complete
// only between the UMMAs of a K block, ~330 clocks per K block -- are paid once per 1024 clocks of UMMA, not per 512.
//
// Work split: the K blocks of all tiles form one sequence of units, and every cluster takes an equal, contiguous
// range of it. With a workspace the ranges are cut exactly (a tile that straddles a boundary is accumulated in parts:
// every cluster that stops inside a tile writes its partial accumulator to the workspace, the cluster that ends the
// tile adds the parts and stores the result), so all SMs finish together whatever the number of tiles; without one
// the ranges are rounded to whole tiles.
//
// Same math and operand formats as gemm_kernel (gemm_umma.cu) and gemm_persist_kernel; replaces the same reference
// code (PACK_BGEMM_Kernel, lowbit_kernel/csrc/include/kernel_matmul.cuh:370-547).
//
// Tensor memory (all 512 columns, allocated by both CTAs together): one accumulator of 256 columns (each CTA holds
// its 128 rows of the tile) and a ring of four u8 weight-operand stages of 64 columns.
//   warps 0-15   unpack, four sets of four warps; set s takes the K blocks g of the CTA's stream with g % 4 == s
//   warps 16-23  epilogue: warp w reads lane quadrant w % 4 of column half (w - 16) / 4 into an int16 staging tile, hands
//                the accumulator back, then converts and stores under the next item's mainloop
//   warp 24      tensor-memory allocation; in the even CTA one lane issues all UMMAs
//   warp 25      one lane streams this CTA's packed weight tiles (cp.async.bulk)
//   warp 26      one lane loads this CTA's half of the activation tiles (TMA, 128B swizzle); the bytes of both halves
//                are counted on the even CTA's barrier
// Signals across the pair: the odd CTA's unpack and epilogue warps arrive on the even CTA's barriers with plain
// remote arrivals (no data crosses; every CTA loads what it needs itself); the issuer's commits arrive on the barrier
// of the same name in both CTAs. Every wait is bounded as in the other kernels, and both CTAs meet in a cluster
// barrier before either frees tensor memory or exits, so no signal is ever sent to a CTA that has left.
#include <cuda.h>

#include <atomic>
#include <cuda_fp16.h>

#include <cstdlib>

#include "epilogue.cuh"
#include "internal.h"
#include "prof.cuh"
#include "ptx.cuh"

namespace bgemm {

// Unpack sets of four warps; set s takes the K blocks g with g % kQSets == s, i.e. always the same operand stage. A set
// needs ~2100 clocks per K block (its tensor-memory stores complete only between UMMAs), a K block of UMMAs 1024: two
// sets leave the tensor pipe waiting (28672 x 8192 x 4096: 656 us), four do not (580 us).
constexpr int kQSets = 4;
constexpr int kQEpiThreads = 256;
constexpr int kQWarpEpi = 4 * kQSets, kQWarpMma = kQWarpEpi + 8, kQWarpW = kQWarpMma + 1, kQWarpB = kQWarpMma + 2;
constexpr int kQThreads = 32 * (kQWarpB + 1);
// 864 threads start with 72 registers each; the unpack warps (16 of 27) release down to 48, which lets the 8 epilogue
// warps hold 120: 16 * 32 * 24 registers change hands.
constexpr int kQUnpackRegs = 48, kQEpiRegs = 120;
constexpr long long kQCopyDrainClocks = 4000000;   // ~2 ms: far beyond any TMA copy of a 32 KB tile

struct QCfg {
    static constexpr int NT = 256;                          // columns of a pair tile
    static constexpr int A_STAGE_COLS = 64;
    static constexpr int STAGES = 4;                        // operand stages: (512 - NT) / 64 columns of tensor memory
    static constexpr int A_COL0 = NT;
    static constexpr int B_HALF_ROWS = NT / 2;              // activation rows this CTA loads
    static constexpr int B_STAGE_BYTES = B_HALF_ROWS * 256;
    static constexpr int W_STAGES = kQSets == 4 ? 4 : 6;
    static constexpr int ROW_PITCH = 68;                    // words per row of a half in the row-major ([M, N] results) staging: 64 + 4
    static constexpr int HALF_WORDS = 128 * ROW_PITCH;      // staging words of one column half (>= 64 x 128 of the column-major form)
    static constexpr int STAGE_TILE_BYTES = 2 * HALF_WORDS * 4;   // this CTA's 128 x 256 accumulator as int16 pairs
    static constexpr int PART_INTS = 128 * NT;              // a CTA's partial accumulator in the workspace
    // w_full/w_empty, full/empty, d_full, d_empty, drained
    static constexpr int NBARS = 2 * W_STAGES + 2 * STAGES + 3;
    static constexpr int MISC_BYTES = 512 /*barriers*/ + 512 /*alpha*/ + 1024 /*colsum*/ + 512 /*flags*/;
    static constexpr int SMEM_BYTES = STAGES * B_STAGE_BYTES + W_STAGES * 4096 + STAGE_TILE_BYTES + MISC_BYTES + 1024 /*align*/;
    static_assert(W_STAGES % kQSets == 0 && STAGES % kQSets == 0, "stage -> unpack set must stay fixed");
    static_assert(NT + STAGES * A_STAGE_COLS <= 512, "tensor memory budget");
    static_assert(NBARS * 8 <= 512, "barrier area");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(SMEM_BYTES > 114 * 1024, "one CTA per SM");
};

// The issuer's signal to both CTAs of the pair: one commit whose arrival is delivered to the barrier at the same
// offset in each of them.
__device__ __forceinline__ void commit_both(uint32_t bar) { umma_commit_pair_mask(bar, (uint16_t)3); }

// First unit (K block of the global sequence) of cluster c. Exact split: c * units / ncl; whole-tile split: the same on
// tiles. Both are monotonic with range(0) = 0 and range(ncl) = everything.
__device__ __forceinline__ long long pair_range_begin(long long c, long long ncl, long long total_tiles, int nkb, int exact) {
    return exact ? (c * total_tiles * nkb) / ncl : ((c * total_tiles) / ncl) * nkb;
}

// fp16 results of 8 adjacent columns (n0 .. n0 + 7) of row m of the [M, N] layout; same values as store8_cols.
__device__ __forceinline__ void store_row8_f16(const TileOut& t, int m, int n0, const int (&acc)[8]) {
    const GemmParams& p = *t.p;
    const int gm = t.m_base + m, gn = t.n_base + n0;
    if (gm >= p.M || gn >= p.N) return;
    const bool full = gn + 8 <= p.N;
    const int4 c0 = *reinterpret_cast<const int4*>(t.s_colsum + n0), c1 = *reinterpret_cast<const int4*>(t.s_colsum + n0 + 4);
    const int cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    int big = 0;
#pragma unroll
    for (int q = 0; q < 8; q++) big |= abs(cs[q]);
    const bool small = big < (1 << 21);
    const float a = t.s_alpha[m];
    float f[8];
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const int val = p.epi ? cs[q] - 2 * acc[q] : acc[q];
        f[q] = small ? __int_as_float(0x4B400000 + val) - 12582912.f : (float)val;
        if (p.out_kind == BGEMM_OUT_F16_SCALED) f[q] *= a;
    }
    __align__(16) __half2 h2[4];
#pragma unroll
    for (int q = 0; q < 4; q++) h2[q] = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
    const size_t idx = (size_t)t.batch * p.M * p.N + (size_t)gm * p.ldo + gn;
    auto put = [&](void* base) {
        __half* o = reinterpret_cast<__half*>(base) + idx;
        if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
            store16B(o, *reinterpret_cast<const uint4*>(h2), t.streaming);
        } else {
            const __half* hs = reinterpret_cast<const __half*>(h2);
#pragma unroll
            for (int q = 0; q < 8; q++) if (gn + q < p.N) o[q] = hs[q];
        }
    };
    put(p.out);
#pragma unroll 1
    for (int d = 0; d < p.n_out_more; d++) put(p.out_more[d]);
}

// fp16 results of two adjacent columns (n, n + 1) x 8 rows (m0 .. m0 + 7) of the [N, M] layout from 8 staged int16
// pairs: the same values as store8_rows produces (exact int -> float, one rounding in the multiply, round-to-nearest-
// even to fp16), with conversions that stay off the slow conversion pipe -- int -> float by adding the integer to the
// bit pattern of 1.5 * 2^23 (exact below 2^22; larger column sums take the ordinary conversion) and two floats -> half2
// in one instruction.
__device__ __forceinline__ void store2cols_f16(const TileOut& t, int n, int m0, const uint32_t (&wv)[8]) {
    const GemmParams& p = *t.p;
    const int gm = t.m_base + m0;
    if (gm >= p.M) return;
    const bool full = gm + 8 <= p.M;
    float al[8];
    if (p.out_kind == BGEMM_OUT_F16_SCALED) {
        const float4 a0 = *reinterpret_cast<const float4*>(t.s_alpha + m0), a1 = *reinterpret_cast<const float4*>(t.s_alpha + m0 + 4);
        al[0] = a0.x; al[1] = a0.y; al[2] = a0.z; al[3] = a0.w; al[4] = a1.x; al[5] = a1.y; al[6] = a1.z; al[7] = a1.w;
    } else {
#pragma unroll
        for (int q = 0; q < 8; q++) al[q] = 1.f;
    }
#pragma unroll
    for (int c = 0; c < 2; c++) {
        const int gn = t.n_base + n + c;
        if (gn >= p.N) break;
        const int cs = t.s_colsum[n + c];
        float f[8];
        const bool small = cs > -(1 << 21) && cs < (1 << 21);
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const int v = c ? ((int)wv[q] >> 16) : (int)(short)(wv[q] & 0xffffu);
            const int val = p.epi ? cs - 2 * v : v;
            f[q] = small ? __int_as_float(0x4B400000 + val) - 12582912.f : (float)val;
            if (p.out_kind == BGEMM_OUT_F16_SCALED) f[q] *= al[q];
        }
        __align__(16) __half2 h2[4];
#pragma unroll
        for (int q = 0; q < 4; q++) h2[q] = __floats2half2_rn(f[2 * q], f[2 * q + 1]);
        const size_t idx = (size_t)t.batch * p.M * p.N + (size_t)gn * p.ldo + gm;
        auto put = [&](void* base) {
            __half* o = reinterpret_cast<__half*>(base) + idx;
            if (full && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
                store16B(o, *reinterpret_cast<const uint4*>(h2), t.streaming);
            } else {
                const __half* hs = reinterpret_cast<const __half*>(h2);
#pragma unroll
                for (int q = 0; q < 8; q++) if (gm + q < p.M) o[q] = hs[q];
            }
        };
        put(p.out);
#pragma unroll 1
        for (int d = 0; d < p.n_out_more; d++) put(p.out_more[d]);
    }
}

// The items of a cluster's range [u0, u1), in the order it works through them: a tile's K blocks that belong to one
// cluster form one item. Parts of a tile that stop before its last K block are handed over through the workspace and
// come FIRST (at most one per cluster: the head of the range's last tile, or a range that lies inside one tile); the
// part that ends a tile begun by other clusters comes after the first whole tile and adds their parts, which were
// written as those clusters' first items -- a tile's time earlier at the least; the other whole tiles follow. So
// nobody waits for work that is scheduled late, the partial sums are read back while they are still in L2, and every
// cluster ends on a whole tile.
struct PairItems {
    long long ta, tb;     // first and last tile of the range
    int a, b;             // first K block of the range in tile ta, end K block in tile tb
    int nkb, has_head, has_tail, n;
    __device__ __forceinline__ PairItems(long long u0, long long u1, int nkb_) : nkb(nkb_) {
        ta = u0 / nkb; a = (int)(u0 - ta * nkb);
        tb = (u1 - 1) / nkb; b = (int)(u1 - tb * nkb);
        if (u1 <= u0) { has_head = has_tail = 0; n = 0; }
        else if (ta == tb) { has_head = 1; has_tail = 0; n = 1; }                  // one item; "head" slot whatever its kind
        else {
            has_head = b < nkb ? 1 : 0;
            has_tail = a > 0 ? 1 : 0;
            n = has_head + has_tail + (int)(tb - ta + 1 - has_head - has_tail);
        }
    }
    __device__ __forceinline__ void get(int idx, long long& t, int& kb0, int& kb1) const {
        if (ta == tb) { t = ta; kb0 = a; kb1 = b; return; }
        if (idx < has_head) { t = tb; kb0 = 0; kb1 = b; return; }
        idx -= has_head;
        const int n_full = n - has_head - has_tail;
        // one whole tile (if there is one) before the part that needs other clusters' sums: by then they are written
        const int tail_at = n_full > 0 ? 1 : 0;
        if (has_tail && idx == tail_at) { t = ta; kb0 = a; kb1 = nkb; return; }
        if (has_tail && idx > tail_at) idx--;
        t = ta + has_tail + idx; kb0 = 0; kb1 = nkb;
    }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kQThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_acts, const GemmParams p, const long long total_tiles, const int exact) {
    using C = QCfg;
    constexpr int NT = C::NT;
    BGEMM_TUNING_ONLY(const long long t_cta0 = clock64();)
    grid_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    // identical offsets in both CTAs of the pair (the dynamic shared-memory base is the same in every CTA of a launch)
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sB = smem;
    uint8_t* sW = sB + C::STAGES * C::B_STAGE_BYTES;
    int* sP = reinterpret_cast<int*>(sW + C::W_STAGES * 4096);
    uint8_t* misc = reinterpret_cast<uint8_t*>(sP) + C::STAGE_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc);
    float* s_alpha = reinterpret_cast<float*>(misc + 512);
    int* s_colsum = reinterpret_cast<int*>(misc + 1024);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(misc + 2048);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const uint32_t w_full = smem_u32(bars);
    const uint32_t w_empty = w_full + 8 * C::W_STAGES;
    const uint32_t full = w_empty + 8 * C::W_STAGES;     // [S] even CTA only: operand stage filled in BOTH CTAs
    const uint32_t empty = full + 8 * C::STAGES;         // [S] both CTAs: operand stage consumed (one commit)
    const uint32_t d_full = empty + 8 * C::STAGES;       // both CTAs: accumulator complete (one commit)
    const uint32_t d_empty = d_full + 8;                 // even CTA only: accumulator read out by the epilogue warps of both CTAs
    const uint32_t drained = d_empty + 8;                // both CTAs: every UMMA of the pair has been executed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();             // 0: the CTA that issues the UMMAs and owns the "filled" barriers
    const bool leader = rank == 0;
    const int nkb = p.kblocks;
    const long long cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
    // units of this cluster: [u0, u1) of the sequence (tile 0: K blocks 0 .. nkb - 1, tile 1: ..., ...);
    // tile index = (batch * (mtiles / 2) + mt / 2) * ntiles + nt
    const long long u0 = pair_range_begin(cid, ncl, total_tiles, nkb, exact);
    const long long u1 = pair_range_begin(cid + 1, ncl, total_tiles, nkb, exact);
    const PairItems items(u0, u1, nkb);
    const int mpairs = p.mtiles >> 1;
    // the even CTA's barriers as seen from either CTA
    const uint32_t full_leader = mapa_shared(full, 0);
    const uint32_t d_empty_leader = mapa_shared(d_empty, 0);

    if (warp == 0) {
        for (int i = lane; i < C::NBARS; i += 32) {
            const int f0 = 2 * C::W_STAGES, d0 = f0 + 2 * C::STAGES;
            int count = 1;
            if (i >= C::W_STAGES && i < 2 * C::W_STAGES) count = 4;           // w_empty: unpack warps of a set
            else if (i >= f0 && i < f0 + C::STAGES) count = 9;                // full: activation producer + unpack warps of a set in both CTAs
            else if (i == d0 + 1) count = 16;                                 // d_empty: epilogue warps of both CTAs
            mbar_init(w_full + 8 * i, count);
        }
        if (lane == 0) { *abort_flag = 0; set_wait_budget(abort_flag, p.wait_budget); }
        mbar_fence_init();
    } else if (warp == kQWarpB) {
        if (lane == 0) tma_prefetch_desc(&tmap_acts);
    } else if (warp == kQWarpMma) {
        tmem_alloc_pair(smem_u32(tmem_holder), 512);
    }
    tc_fence_before();
    __syncwarp();
    // Both CTAs' barriers exist before anybody signals across the pair.
    cluster_arrive_release();
    cluster_wait_acquire();
    tc_fence_after();
    grid_dependency_wait();      // nothing above touches global memory (programmatic dependent launch)
    const uint32_t tmem = *tmem_holder;
    const uint32_t tmem_d = tmem;
    const uint32_t tmem_a = tmem + C::A_COL0;

    if (warp == kQWarpW) {
        // ---------------- weight producer: this CTA's 128 rows ----------------
        if (lane == 0) {
            long long g = 0;
            bool ok = true;
            for (int item = 0; item < items.n && ok; item++) {
                long long t; int kb0, kb1;
                items.get(item, t, kb0, kb1);
                const long long bm = t / p.ntiles;                      // batch * mpairs + pair row
                const int mt = 2 * (int)(bm % mpairs) + (int)rank, batch = (int)(bm / mpairs);
                const uint8_t* src = p.plane + (size_t)batch * p.plane_batch_bytes + (size_t)mt * nkb * 4096;
                for (int i = kb0; i < kb1; i++, g++) {
                    const int s = (int)(g % C::W_STAGES);
                    if (g >= C::W_STAGES) ok = mbar_wait_relaxed(w_empty + 8 * s, (uint32_t)((g / C::W_STAGES) - 1) & 1, abort_flag, p.status, 41);
                    if (!ok) break;
                    if (g == p.test_skip_kblock) continue;          // test hook: this K block never arrives, its consumers' waits run out
                    mbar_arrive_expect_tx(w_full + 8 * s, 4096);
                    bulk_g2s(smem_u32(sW + s * 4096), src + (size_t)i * 4096, 4096, w_full + 8 * s);
                }
            }
            if (*abort_flag) {  // drain own copies before the CTA may exit
                for (long long i = g - 1; i >= 0 && i >= g - C::W_STAGES; i--) {
                    const long long t0 = clock64();
                    while (!mbar_test(w_full + 8 * (int)(i % C::W_STAGES), (uint32_t)(i / C::W_STAGES) & 1) && clock64() - t0 < wait_budget_of(abort_flag)) {}
                }
            }
        }
    } else if (warp == kQWarpB) {
        // ---------------- activation producer: this CTA's half of the tile's activation rows ----------------
        if (lane == 0) {
            long long g = 0;
            bool ok = true;
            for (int item = 0; item < items.n && ok; item++) {
                long long t; int kb0, kb1;
                items.get(item, t, kb0, kb1);
                const int nt = (int)(t % p.ntiles);
                const int batch = (int)(t / p.ntiles / mpairs);
                const int row0 = nt * NT + (int)rank * C::B_HALF_ROWS;
                for (int i = kb0; i < kb1; i++, g++) {
                    const int s = (int)(g % C::STAGES);
                    if (g >= C::STAGES) ok = mbar_wait_relaxed(empty + 8 * s, (uint32_t)((g / C::STAGES) - 1) & 1, abort_flag, p.status, 42);
                    if (!ok) break;
                    BGEMM_TRACE(4, g);
                    // one arrival for the pair, announcing the bytes of both halves
                    if (leader) mbar_arrive_expect_tx(full + 8 * s, 2 * C::B_STAGE_BYTES);
                    const uint32_t dst = smem_u32(sB + s * C::B_STAGE_BYTES);
                    tma_load_3d_pair(dst, &tmap_acts, i * 256, row0, batch, full_leader + 8 * s);
                    tma_load_3d_pair(dst + C::B_HALF_ROWS * 128, &tmap_acts, i * 256 + 128, row0, batch, full_leader + 8 * s);
                }
            }
            if (*abort_flag) {
                // The copies in flight must land before the CTA may exit. Their barrier also needs the unpack warps,
                // which have stopped: wait for the longest plausible copy time instead of the barrier.
                const long long t0 = clock64();
                while (g > 0 && clock64() - t0 < kQCopyDrainClocks) {}
            }
        }
    } else if (warp == kQWarpMma) {
        // ---------------- UMMA issuer (even CTA) ----------------
        // A 256 x 256 x 32 UMMA keeps both tensor pipes busy for 128 clocks and costs its issuer ~85, so one thread is
        // enough; it also makes the hand-over of the single accumulator trivial: the first K block of an item
        // (accumulate = 0) is issued once the epilogue warps of both CTAs have read the previous item out.
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_u8s8_m(NT, 256);
            bool ok = true;
            long long g = 0;
            for (int item = 0; item < items.n && ok; item++) {
                long long t; int kb0, kb1;
                items.get(item, t, kb0, kb1);
                if (item >= 1) ok = mbar_wait(d_empty, (uint32_t)(item - 1) & 1, abort_flag, p.status, 45);
                if (!ok) break;
                BGEMM_TRACE(7, item);
                tc_fence_after();
                for (int i = kb0; i < kb1; i++, g++) {
                    const int s = (int)(g % C::STAGES);
                    ok = mbar_wait(full + 8 * s, (uint32_t)(g / C::STAGES) & 1, abort_flag, p.status, 43);
                    if (!ok) break;
                    BGEMM_TRACE(0, g);
                    tc_fence_after();
                    const uint32_t bbase = smem_u32(sB + s * C::B_STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        // the same descriptor is applied in both CTAs: rows 0-127 of B here, rows 128-255 in the partner
                        const uint64_t bdesc = umma_desc_sw128(bbase + (j >> 2) * (C::B_HALF_ROWS * 128) + (j & 3) * 32);
                        umma_i8_ts_pair(tmem_d, tmem_a + s * C::A_STAGE_COLS + j * 8, bdesc, idesc, (i > kb0 || j) ? 1u : 0u);
                    }
                    commit_both(empty + 8 * s);
                    BGEMM_TRACE(1, g);
                }
                if (!ok) break;
                commit_both(d_full);
            }
            commit_both(drained);
        }
    } else if (warp < 4 * kQSets) {
        // ---------------- unpack: set s = warps 4 s .. 4 s + 3 takes the K blocks g of the stream with g % kQSets == s ----
        regs_release<kQUnpackRegs>();                         // the epilogue warps get what these sixteen warps do not need
        const int set = warp >> 2;
        const int r = (warp & 3) * 32 + lane;                 // weight row of this CTA's half tile == tensor-memory lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const long long total_kb = u1 - u0;
        bool ok = true;
        for (long long g = set; g < total_kb && ok; g += kQSets) {
            const int ws = (int)(g % C::W_STAGES);
            ok = mbar_wait(w_full + 8 * ws, (uint32_t)(g / C::W_STAGES) & 1, abort_flag, p.status, 47);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint4 lo = *reinterpret_cast<const uint4*>(sW + ws * 4096 + r * 16);
            const uint4 hi = *reinterpret_cast<const uint4*>(sW + ws * 4096 + 2048 + r * 16);
            fence_proxy_async_smem();     // generic-proxy reads before the producer's next bulk copy into this stage
            __syncwarp();
            if (lane == 0) mbar_arrive(w_empty + 8 * ws);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const int as = (int)(g % C::STAGES);
            if (g >= C::STAGES) ok = mbar_wait_relaxed(empty + 8 * as, (uint32_t)((g / C::STAGES) - 1) & 1, abort_flag, p.status, 48);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if ((tid & 127) == 0) BGEMM_TRACE(2, g);
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                uint32_t v[8];
#pragma unroll
                for (int c = 0; c < 8; c++) v[c] = (w[c] >> j) & 0x01010101u;
                tmem_st8(tmem_a + lane_base + as * C::A_STAGE_COLS + j * 8, v);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(full_leader + 8 * as);
            if ((tid & 127) == 0) BGEMM_TRACE(3, g);
        }
    } else if (warp >= kQWarpEpi && warp < kQWarpEpi + 8) {
        // ---------------- epilogue: this CTA's 128 rows of the tile, columns [128 h, 128 h + 128) per half h ----------------
        // The single accumulator must be handed back quickly: the warps first move it into a shared-memory staging tile
        // as int16 pairs (64 KB; |D| <= K for ternary and binary activations), release it, and only then convert and
        // store -- under the next item's mainloop. A half whose values do not fit 16 bits (general int8 activations)
        // keeps the accumulator and converts straight from tensor memory through a small int32 tile aliased on its
        // part of the staging area.
        // Items that cover only part of a tile's K range (see PairItems): an item that stops before the tile's last K
        // block writes its accumulator to this CTA's slot of the workspace and raises the slot's flag; the item that
        // ends a tile begun by other clusters waits for their flags (they took those items FIRST), adds their slots
        // while it reads its own accumulator, and clears the flags for the next launch.
        regs_request<kQEpiRegs>();
        const int h = (warp - kQWarpEpi) >> 2;
        const int et = (warp & 3) * 32 + lane;                // accumulator row == tensor-memory lane
        const int eall = h * 128 + et;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        // staging of this half: [64 column pairs][128 rows] for [N, M] results (a column's rows are contiguous in the
        // result), [128 rows][68] for [M, N] results (a row's columns are)
        uint32_t* sS = reinterpret_cast<uint32_t*>(sP) + h * C::HALF_WORDS;
        const bool rowmajor = p.out_layout == BGEMM_LAYOUT_MN;
        TileOut tout;
        tout.p = &p; tout.s_alpha = s_alpha; tout.s_colsum = s_colsum;
        // with the exact split the partial sums must survive in L2 from the kernel's first item to its last: results stream out
        tout.streaming = exact != 0;
        const uint64_t keep = l2_policy_evict_last();
        for (int item = 0; item < items.n; item++) {
            long long t; int kb0, kb1;
            items.get(item, t, kb0, kb1);
            const int nt = (int)(t % p.ntiles);
            const long long bm = t / p.ntiles;
            const int mt = 2 * (int)(bm % mpairs) + (int)rank, batch = (int)(bm / mpairs);
            const bool writes_part = kb1 < nkb;
            // clusters cid - 1 .. cid - nparts computed the earlier K blocks of this tile (each as its first item)
            int nparts = 0;
            if (kb1 == nkb && kb0 > 0)
                while (cid - 1 - nparts >= 0 && pair_range_begin(cid - nparts, ncl, total_tiles, nkb, exact) > t * nkb) nparts++;
            tout.batch = batch; tout.m_base = mt * 128; tout.n_base = nt * NT;
            if (!writes_part) {
                if (h == 0) {
                    const int m = mt * 128 + et;
                    s_alpha[et] = (p.out_kind == BGEMM_OUT_F16_SCALED && m < p.M) ? __half2float(p.alpha[(size_t)batch * p.M + m]) : 1.f;
                }
                const int n = nt * NT + eall;
                s_colsum[eall] = (p.epi && n < p.N) ? __ldg(p.colsum + (size_t)batch * p.N + n) : 0;
            }
            bool ok = mbar_wait_relaxed(d_full, (uint32_t)item & 1, abort_flag, p.status, 49);
            if (ok && nparts > 0 && eall == 0) {
                // bounded wait for the continuing clusters' partial sums (flags live in the zero-initialised counter area)
                const long long t0 = clock64(), budget = wait_budget_of(abort_flag);
                for (int q = 0; q < nparts && ok; q++) {
                    volatile unsigned int* f = p.ws_counters + 2 * (cid - 1 - q) + rank;
                    while (*f == 0u) {
                        if (*abort_flag || clock64() - t0 > budget) {
                            *abort_flag = 1;
                            if (p.status) atomicCAS(p.status, 0, 50);
                            ok = false;
                            break;
                        }
                        __nanosleep(100);
                    }
                }
                __threadfence();
            }
            ok = __all_sync(0xffffffffu, ok);
            // One answer for all eight warps (either everybody handles this item or everybody leaves); the barrier also
            // makes this tile's scales and column sums, and the other clusters' partial sums, visible to all of them.
            if (named_bar_or(2, kQEpiThreads, !ok)) break;
            if (warp == kQWarpEpi && lane == 0) BGEMM_TRACE(6, item * 4);
            tc_fence_after();
            // this thread's 32 accumulator values of columns h * 128 + c0 .. + 31, plus the other clusters' parts
            auto issue32 = [&](int c0, uint32_t (&v0)[16], uint32_t (&v1)[16]) {
                tmem_ld16(tmem_d + lane_base + h * 128 + c0, v0);
                tmem_ld16(tmem_d + lane_base + h * 128 + c0 + 16, v1);
            };
            auto add_parts32 = [&](int c0, uint32_t (&v0)[16], uint32_t (&v1)[16]) {
                for (int q = 0; q < nparts; q++) {
                    const int* part = p.ws_partial + (size_t)(2 * (cid - 1 - q) + rank) * C::PART_INTS + (h * 128 + c0) * 128 + et;
#pragma unroll
                    for (int i = 0; i < 16; i++) v0[i] += (uint32_t)ld_global_hint(part + i * 128, keep);
#pragma unroll
                    for (int i = 0; i < 16; i++) v1[i] += (uint32_t)ld_global_hint(part + (16 + i) * 128, keep);
                }
            };
            auto load32 = [&](int c0, uint32_t (&v0)[16], uint32_t (&v1)[16]) {
                issue32(c0, v0, v1);
                tmem_wait_ld();
                add_parts32(c0, v0, v1);
            };
            auto release_accumulator = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(d_empty_leader);
                if (warp == kQWarpEpi && lane == 0) BGEMM_TRACE(6, item * 4 + 1);
            };
            if (writes_part) {
                int* part = p.ws_partial + (size_t)(2 * cid + rank) * C::PART_INTS + (h * 128) * 128 + et;
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t v0[16], v1[16];
                    load32(c0, v0, v1);
                    if (c0 + 32 >= 128) release_accumulator();
#pragma unroll
                    for (int i = 0; i < 16; i++) st_global_hint(part + (c0 + i) * 128, (int)v0[i], keep);
#pragma unroll
                    for (int i = 0; i < 16; i++) st_global_hint(part + (c0 + 16 + i) * 128, (int)v1[i], keep);
                }
                __threadfence();
                named_bar_sync(7, kQEpiThreads);
                if (eall == 0) {
                    __threadfence();
                    *(volatile unsigned int*)(p.ws_counters + 2 * cid + rank) = 1u;
                }
                continue;
            }
            int lo16 = 0, hi16 = 0;                               // value range of this thread's part of the accumulator
            auto stage32 = [&](int c0, uint32_t (&v0)[16], uint32_t (&v1)[16]) {
                add_parts32(c0, v0, v1);
#pragma unroll
                for (int q = 0; q < 16; q++) { lo16 = min(lo16, min((int)v0[q], (int)v1[q])); hi16 = max(hi16, max((int)v0[q], (int)v1[q])); }
                uint32_t w0[8], w1[8];
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    w0[q] = __byte_perm(v0[2 * q], v0[2 * q + 1], 0x5410);      // low halves of two values in one word
                    w1[q] = __byte_perm(v1[2 * q], v1[2 * q + 1], 0x5410);
                }
                if (rowmajor) {
                    uint4* dst = reinterpret_cast<uint4*>(sS + et * C::ROW_PITCH + (c0 >> 1));
                    dst[0] = make_uint4(w0[0], w0[1], w0[2], w0[3]); dst[1] = make_uint4(w0[4], w0[5], w0[6], w0[7]);
                    dst[2] = make_uint4(w1[0], w1[1], w1[2], w1[3]); dst[3] = make_uint4(w1[4], w1[5], w1[6], w1[7]);
                } else {
#pragma unroll
                    for (int q = 0; q < 8; q++) { sS[((c0 >> 1) + q) * 128 + et] = w0[q]; sS[((c0 >> 1) + 8 + q) * 128 + et] = w1[q]; }
                }
            };
            {
                // 128 columns in four loads of 32, two in flight: the second pair is requested while the first is packed
                uint32_t a0[16], a1[16], b0[16], b1[16];
                issue32(0, a0, a1);
                issue32(32, b0, b1);
                tmem_wait_ld();
                stage32(0, a0, a1);
                issue32(64, a0, a1);
                stage32(32, b0, b1);
                issue32(96, b0, b1);
                tmem_wait_ld();
                stage32(64, a0, a1);
                stage32(96, b0, b1);
            }
            // One answer per half: did every value fit 16 bits? (The barrier also publishes the staging tile.)
            const bool wide = named_bar_or(3 + h, 128, lo16 < -32768 || hi16 > 32767);
            if (!wide) {
                release_accumulator();
                if (p.out_layout == BGEMM_LAYOUT_NM) {
                    // unit = (column pair, 8 rows): 16 lanes cover the 128 rows of a column, i.e. 256 contiguous bytes (fp16)
#pragma unroll 1
                    for (int un = et; un < 64 * 16; un += 128) {
                        const int cp = un >> 4, m0 = (un & 15) * 8;
                        const uint4 a = *reinterpret_cast<const uint4*>(sS + cp * 128 + m0);
                        const uint4 b = *reinterpret_cast<const uint4*>(sS + cp * 128 + m0 + 4);
                        const uint32_t wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                        if (p.out_kind != BGEMM_OUT_I32) {
                            store2cols_f16(tout, h * 128 + 2 * cp, m0, wv);
                        } else {
                            int even[8], odd[8];
#pragma unroll
                            for (int q = 0; q < 8; q++) { even[q] = (int)(short)(wv[q] & 0xffffu); odd[q] = (int)wv[q] >> 16; }
                            store8_rows(tout, h * 128 + 2 * cp, m0, even);
                            store8_rows(tout, h * 128 + 2 * cp + 1, m0, odd);
                        }
                    }
                } else {
                    // unit = (row, 8 columns): 16 lanes cover the 128 columns of a row, i.e. 256 contiguous bytes (fp16)
#pragma unroll 1
                    for (int un = et; un < 128 * 16; un += 128) {
                        const int m = un >> 4, cg = un & 15;
                        const uint4 a = *reinterpret_cast<const uint4*>(sS + m * C::ROW_PITCH + cg * 4);
                        const int acc[8] = {(int)(short)(a.x & 0xffffu), (int)a.x >> 16, (int)(short)(a.y & 0xffffu), (int)a.y >> 16,
                                            (int)(short)(a.z & 0xffffu), (int)a.z >> 16, (int)(short)(a.w & 0xffffu), (int)a.w >> 16};
                        if (p.out_kind != BGEMM_OUT_I32) store_row8_f16(tout, m, h * 128 + cg * 8, acc);
                        else store8_cols(tout, m, h * 128 + cg * 8, acc);
                    }
                }
            } else {
                // values beyond 16 bits: straight from tensor memory, 32 columns at a time through an int32 tile
                int* sPh = reinterpret_cast<int*>(sS);
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    const int n0 = h * 128 + c0;
                    uint32_t v0[16], v1[16];
                    named_bar_sync(5 + h, 128);                   // the tile is free (first round: the int16 pass is over)
                    load32(c0, v0, v1);
                    if (c0 + 32 >= 128) release_accumulator();
#pragma unroll
                    for (int q = 0; q < 16; q++) sPh[q * 128 + et] = (int)v0[q];
#pragma unroll
                    for (int q = 0; q < 16; q++) sPh[(16 + q) * 128 + et] = (int)v1[q];
                    named_bar_sync(5 + h, 128);
                    write_tile<false>(tout, sPh, 1, 0, n0, 32, et, 128);
                }
            }
            if (warp == kQWarpEpi && lane == 0) BGEMM_TRACE(6, item * 4 + 2);
            named_bar_sync(7, kQEpiThreads);                      // staging tile, scales and column sums are free for the next item
            if (nparts > 0 && eall == 0)                          // every thread has read the parts: clear their flags for the next launch
                for (int q = 0; q < nparts; q++) *(volatile unsigned int*)(p.ws_counters + 2 * (cid - 1 - q) + rank) = 0u;
        }
    }
    tc_fence_before();
    __syncwarp();
    // Both CTAs are done with each other's barriers and tensor memory before either frees it or exits.
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == kQWarpMma) {
        if (lane == 0) {   // every UMMA has been executed before the columns are freed (immediate unless a wait ran out)
            const long long t0 = clock64();
            while (!mbar_test(drained, 0) && clock64() - t0 < wait_budget_of(abort_flag)) {}
        }
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem, 512);
    }
}

static int env_int_q(const char* name) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : -1;
}
// BGEMM_PAIR in the environment, or bgemm_debug_set_pair_kernel at run time (which wins): 0 = never, 1 = whenever the
// shape allows, anything else = the rule below.
static std::atomic<int> g_pair_mode{-2};        // -2: not set by the hook
static int pair_forced() {
    static const int env = env_int_q("BGEMM_PAIR");
    const int m = g_pair_mode.load(std::memory_order_relaxed);
    return m == -2 ? env : m;
}
void set_pair_mode(int mode) { g_pair_mode.store(mode < -1 || mode > 1 ? -2 : mode, std::memory_order_relaxed); }

// Shapes the pair kernel CAN take: at least one full 256-column tile, an even number of 128-row tiles, two K blocks.
static bool pair_possible(long long mtiles, long long N, long long kblocks) { return !(mtiles & 1) && N >= QCfg::NT && kblocks >= 2; }

// ... and those it is given. Measured against the tile-per-CTA kernel (128-column tiles, two CTAs per SM) inside single
// runs: a 256 x 256 tile costs ~8k clocks beyond its K blocks (1024 clocks each), so short K loses (K = 512 / 1024 /
// 2048: 241 against 192, 248 against 218, 28.7 against 25.0 us; from K = 2560 on it wins: 145 against 165 us at
// 28672 x 2560 x 2048); up to two tiles across N it is level or behind (28672 x 8192 x 512: 98.4 against 96.1; 12288 x
// 4096 x 512: 36.3 against 30.3), from three on ahead (28672 x 8192 x 768: 120 against 134; x 1024: 158 against 172;
// 11008 x 4096 x 2048: 74 against 91); a last tile that is mostly padding costs more than the pairing gains (N = 640:
// 118 against 112, N = 320: 95 against 73); and with fewer than ~1.5 tiles per SM pair the cut into equal ranges no
// longer covers the per-tile cost (8192 x 8192 x 768, 96 tiles: 54 against 48).
static bool pair_worthwhile(long long mtiles, long long N, long long kblocks, long long batch) {
    const long long n256 = (N + 255) / 256 * 256, n128 = (N + 127) / 128 * 128;
    const long long tiles = (mtiles / 2) * (n256 / 256) * batch;
    return kblocks >= 10 && N > 512 && n256 * 100 <= n128 * 107 && tiles * 4 >= (long long)sm_count() * 3;
}

bool pair_supported(const GemmParams& p, long long batch) {
    const int forced = pair_forced();
    if (forced == 0) return false;
    if (p.split_k != 1 || p.out_kind == kOutActs || !pair_possible(p.mtiles, p.N, p.kblocks)) return false;
    if (forced == 1) return true;
    if (p.test_skip_kblock >= 0) return false;
    return pair_worthwhile(p.mtiles, p.N, p.kblocks, batch);
}

// Workspace with which the pair kernel cuts its work into exactly equal ranges: the 64 KiB counter area (flags; zeroed
// once, left zero by every launch) and one partial accumulator per CTA. 0 when the shape would not use it.
size_t pair_balance_workspace_bytes(long long M, long long N, long long K, long long batch) {
    const int forced = pair_forced();
    if (forced == 0) return 0;
    const long long mtiles = (M + 127) / 128, kblocks = (K + 255) / 256;
    if (!pair_possible(mtiles, N, kblocks)) return 0;
    if (forced != 1 && !pair_worthwhile(mtiles, N, kblocks, batch)) return 0;
    return (size_t)65536 + (size_t)sm_count() * QCfg::PART_INTS * 4;
}

int launch_gemm_pair(cudaStream_t stream, const void* tensor_map, const GemmParams& p, long long batch) {
    using C = QCfg;
    const CUtensorMap& tmap = *static_cast<const CUtensorMap*>(tensor_map);
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    const long long total_tiles = (long long)(p.mtiles / 2) * p.ntiles * batch;
    const long long units = total_tiles * p.kblocks;
    // clusters that can be resident at once (normally one per SM pair): the exact split needs all of its clusters
    // running, because a cluster waits for the partial sums of its predecessors
    static int resident[64] = {};
    if (dev < 64 && !resident[dev]) {
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3((unsigned)(sm_count() / 2 * 2), 1, 1);
        q.blockDim = dim3(kQThreads, 1, 1);
        q.dynamicSmemBytes = C::SMEM_BYTES;
        int n = 0;
        resident[dev] = (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel, &q) == cudaSuccess && n > 0) ? n : -1;
        cudaGetLastError();
    }
    long long pairs = sm_count() / 2;
    if (dev < 64 && resident[dev] > 0 && resident[dev] < pairs) pairs = resident[dev];
    const bool can_wait = dev < 64 && resident[dev] > 0;       // unknown residency: whole tiles only
    // exact ranges need the workspace and every cluster resident at once (a cluster waits for its successors' parts):
    // one cluster per SM pair, at least four K blocks each
    // -- and it pays when every cluster has at least a tile's worth of work and the tiles do not divide evenly anyway
    int exact = (can_wait && p.ws_partial && p.ws_counters && units >= 4 * pairs && total_tiles >= pairs && total_tiles % pairs != 0) ? 1 : 0;
    if (pair_forced() == 1 && can_wait && p.ws_partial && p.ws_counters && units >= 4 * pairs) exact = 1;      // tuning / tests: whenever possible
    static const int no_exact = env_int_q("BGEMM_PAIR_EXACT");     // tuning override: 0 = whole tiles only
    if (no_exact == 0) exact = 0;
    const long long clusters = exact ? pairs : (total_tiles < pairs ? total_tiles : pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    cfg.blockDim = dim3(kQThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (programmatic_launch_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel, tmap, p, total_tiles, exact);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace bgemm
