// Persistent binary-weight GEMM on CTA pairs (tcgen05.mma.cta_group::2) for wide activation matrices: the two CTAs of
// a cluster -- the two SMs of a TPC -- compute one 256(M) x 256(N) tile together. Each CTA streams and unpacks ITS OWN
// 128 weight rows into its own tensor memory and loads only HALF of the activation tile (128 of the 256 activation
// rows) into its own shared memory; one thread of the even CTA issues a single 256 x 256 x 32 UMMA for both SMs, which
// reads both halves. Against the 128-row kernels that halves the activation bytes an SM pulls from L2 per unit of
// tensor work (36 KB per 1024 clocks of UMMA instead of 36 KB per 512) and halves the instructions, waits and commits
// per unit of tensor work for the issuing threads -- the two walls those kernels run into.
//
// Same math and operand formats as gemm_kernel (gemm_umma.cu) and gemm_persist_kernel; replaces the same reference
// code (PACK_BGEMM_Kernel, lowbit_kernel/csrc/include/kernel_matmul.cuh:370-547).
//
// Tensor memory (all 512 columns, allocated by both CTAs together): one accumulator of 256 columns (each CTA holds
// its 128 rows of the tile) and a ring of four u8 weight-operand stages of 64 columns.
//   warps 0-7    unpack, two sets taking alternate K blocks of the CTA's whole K-block stream (as gemm_persist_kernel)
//   warps 8-15   epilogue: warp w reads lane quadrant w % 4 of column half (w - 8) / 4 into an int16 staging tile, hands
//                the accumulator back, then converts and stores under the next tile's mainloop
//   warp 16      tensor-memory allocation; in the even CTA one lane issues the UMMAs of the even K blocks
//   warp 19      in the even CTA one lane issues the UMMAs of the odd K blocks
//   warp 17      one lane streams this CTA's packed weight tiles (cp.async.bulk)
//   warp 18      one lane loads this CTA's half of the activation tiles (TMA, 128B swizzle); the bytes of both halves
//                are counted on the even CTA's barrier
// Signals across the pair: the odd CTA's unpack and epilogue warps arrive on the even CTA's barriers with plain
// remote arrivals (no data crosses; every CTA loads what it needs itself); the issuers' commits arrive on the barrier
// of the same name in both CTAs. Every wait is bounded as in the other kernels, and both CTAs meet in a cluster
// barrier before either frees tensor memory or exits, so no signal is ever sent to a CTA that has left.
#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "epilogue.cuh"
#include "internal.h"
#include "prof.cuh"
#include "ptx.cuh"

namespace bgemm {

constexpr int kQThreads = 640;
constexpr int kQEpiThreads = 256;
constexpr int kQWarpEpi = 8, kQWarpMma0 = 16, kQWarpW = 17, kQWarpB = 18, kQWarpMma1 = 19;
constexpr long long kQCopyDrainClocks = 4000000;   // ~2 ms: far beyond any TMA copy of a 32 KB tile

struct QCfg {
    static constexpr int NT = 256;                          // columns of a pair tile
    static constexpr int A_STAGE_COLS = 64;
    static constexpr int STAGES = 4;                        // operand stages: (512 - NT) / 64 columns of tensor memory
    static constexpr int A_COL0 = NT;
    static constexpr int B_HALF_ROWS = NT / 2;              // activation rows this CTA loads
    static constexpr int B_STAGE_BYTES = B_HALF_ROWS * 256;
    static constexpr int W_STAGES = 6;
    static constexpr int STAGE_TILE_BYTES = 128 * NT * 2;   // this CTA's 128 x 256 accumulator as int16
    // w_full/w_empty, full/empty, d_full, d_empty, first_done, drained
    static constexpr int NBARS = 2 * W_STAGES + 2 * STAGES + 4;
    static constexpr int MISC_BYTES = 512 /*barriers*/ + 512 /*alpha*/ + 1024 /*colsum*/ + 512 /*flags*/;
    static constexpr int SMEM_BYTES = STAGES * B_STAGE_BYTES + W_STAGES * 4096 + STAGE_TILE_BYTES + MISC_BYTES + 1024 /*align*/;
    static_assert(W_STAGES % 2 == 0 && STAGES % 2 == 0, "stage -> unpack set / issuer must stay fixed");
    static_assert(NT + STAGES * A_STAGE_COLS <= 512, "tensor memory budget");
    static_assert(NBARS * 8 <= 512, "barrier area");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(SMEM_BYTES > 114 * 1024, "one CTA per SM");
};

// The issuers' signal to both CTAs of the pair: one commit whose arrival is delivered to the barrier at the same
// offset in each of them.
__device__ __forceinline__ void commit_both(uint32_t bar) { umma_commit_pair_mask(bar, (uint16_t)3); }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kQThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_acts, const GemmParams p, const long long total_tiles) {
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
    const uint32_t d_full = empty + 8 * C::STAGES;       // both CTAs: accumulator complete (one commit per issuer)
    const uint32_t d_empty = d_full + 8;                 // even CTA only: accumulator read out by the epilogue warps of both CTAs
    const uint32_t first_done = d_empty + 8;             // even CTA only: the K block that zeroes the accumulator has been executed
    const uint32_t drained = first_done + 8;             // both CTAs: every UMMA of the pair has been executed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();             // 0: the CTA that issues the UMMAs and owns the "filled" barriers
    const bool leader = rank == 0;
    const int nkb = p.kblocks;
    const long long cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
    // pair tiles of this cluster: cid, cid + ncl, ... (pair tile index = (batch * (mtiles / 2) + mt / 2) * ntiles + nt)
    const long long my_tiles = cid < total_tiles ? (total_tiles - cid + ncl - 1) / ncl : 0;
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
            else if (i == d0) count = 2;                                      // d_full: both issuers
            else if (i == d0 + 1) count = 16;                                 // d_empty: epilogue warps of both CTAs
            else if (i == d0 + 3) count = 2;                                  // drained: both issuers
            mbar_init(w_full + 8 * i, count);
        }
        if (lane == 0) { *abort_flag = 0; set_wait_budget(abort_flag, p.wait_budget); }
        mbar_fence_init();
    } else if (warp == kQWarpB) {
        if (lane == 0) tma_prefetch_desc(&tmap_acts);
    } else if (warp == kQWarpMma0) {
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
            for (long long t = cid; t < total_tiles && ok; t += ncl) {
                const long long bm = t / p.ntiles;                      // batch * mpairs + pair row
                const int mt = 2 * (int)(bm % mpairs) + (int)rank, batch = (int)(bm / mpairs);
                const uint8_t* src = p.plane + (size_t)batch * p.plane_batch_bytes + (size_t)mt * nkb * 4096;
                for (int i = 0; i < nkb; i++, g++) {
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
            for (long long t = cid; t < total_tiles && ok; t += ncl) {
                const int nt = (int)(t % p.ntiles);
                const int batch = (int)(t / p.ntiles / mpairs);
                const int row0 = nt * NT + (int)rank * C::B_HALF_ROWS;
                for (int i = 0; i < nkb; i++, g++) {
                    const int s = (int)(g % C::STAGES);
                    if (g >= C::STAGES) ok = mbar_wait_relaxed(empty + 8 * s, (uint32_t)((g / C::STAGES) - 1) & 1, abort_flag, p.status, 42);
                    if (!ok) break;
                    // one arrival for the pair, announcing the bytes of both halves
                    BGEMM_TRACE(4, g);
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
    } else if (warp == kQWarpMma0 || warp == kQWarpMma1) {
        // ---------------- UMMA issuers (even CTA): issuer `me` takes the K blocks with g % 2 == me ----------------
        const int me = warp == kQWarpMma0 ? 0 : 1;
        if (lane == 0 && leader) {
            constexpr uint32_t idesc = umma_idesc_u8s8_m(NT, 256);
            bool ok = true;
            long long g = 0;
            for (long long lt = 0; lt < my_tiles && ok; lt++) {
                // The first K block of a tile overwrites the accumulator (accumulate = 0). Its issuer (the "opener",
                // whoever owns that K block) waits until the epilogue warps of both CTAs have read the previous tile
                // out; the other issuer waits until that K block has been executed before it adds anything. Integer
                // accumulation commutes, so no other order is needed. Parity waits never name a phase their barrier
                // has not reached -- the argument is the one in gemm_persist_kernel with a single accumulator buffer:
                // d_empty phase lt - 2 was awaited by the opener of tile lt - 1, and the other issuer waited for that
                // tile to be opened; first_done phase lt - 1 was either awaited by this thread or committed by it
                // before it reused one of its operand stages (odd K-block counts are only launched with at least
                // STAGES K blocks per tile).
                const bool opener = (int)(g & 1) == me;
                if (opener) {
                    if (lt >= 1) ok = mbar_wait(d_empty, (uint32_t)(lt - 1) & 1, abort_flag, p.status, 45);
                } else {
                    ok = mbar_wait(first_done, (uint32_t)lt & 1, abort_flag, p.status, 46);
                }
                if (!ok) break;
                if (opener) BGEMM_TRACE(7, lt);
                tc_fence_after();
                for (int i = 0; i < nkb; i++, g++) {
                    if ((int)(g & 1) != me) continue;
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
                        umma_i8_ts_pair(tmem_d, tmem_a + s * C::A_STAGE_COLS + j * 8, bdesc, idesc, (i | j) ? 1u : 0u);
                    }
                    if (i == 0) umma_commit_pair(first_done);
                    commit_both(empty + 8 * s);
                    BGEMM_TRACE(1, g);
                }
                if (!ok) break;
                commit_both(d_full);
            }
            commit_both(drained);
        }
    } else if (warp < 8) {
        // ---------------- unpack: set 0 = warps 0-3 takes even K blocks of the stream, set 1 = warps 4-7 odd ones ----
        const int set = warp >> 2;
        const int r = (warp & 3) * 32 + lane;                 // weight row of this CTA's half tile == tensor-memory lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const long long total_kb = my_tiles * nkb;
        bool ok = true;
        // The tensor-memory stores of a K block take ~1000 clocks to complete while the UMMAs keep the memory busy, so
        // their completion (tcgen05.wait::st, then the "filled" arrival) is deferred until the weights of the set's
        // NEXT K block have been fetched from shared memory: `pend` is the stage whose stores are still in flight.
        int pend = -1;
        for (long long g = set; g < total_kb && ok; g += 2) {
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
            if (pend >= 0) {              // the previous K block of this set is complete in tensor memory
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(full_leader + 8 * pend);
                if ((tid & 127) == 0) BGEMM_TRACE(3, g - 2);
            }
            const int as = (int)(g % C::STAGES);
            if (g >= C::STAGES) ok = mbar_wait_relaxed(empty + 8 * as, (uint32_t)((g / C::STAGES) - 1) & 1, abort_flag, p.status, 48);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) { pend = -1; break; }
            if ((tid & 127) == 0) BGEMM_TRACE(2, g);
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < 8; j++) {
                uint32_t v[8];
#pragma unroll
                for (int c = 0; c < 8; c++) v[c] = (w[c] >> j) & 0x01010101u;
                tmem_st8(tmem_a + lane_base + as * C::A_STAGE_COLS + j * 8, v);
            }
            if ((tid & 127) == 0) BGEMM_TRACE(5, g);
            pend = as;
        }
        tmem_wait_st();                   // (also on the way out after a wait ran out: no store is left in flight)
        if (pend >= 0) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(full_leader + 8 * pend);
        }
    } else if (warp >= kQWarpEpi && warp < kQWarpEpi + 8) {
        // ---------------- epilogue: this CTA's 128 rows of the tile, columns [128 h, 128 h + 128) per half h ----------------
        // The single accumulator must be handed back quickly: the warps first move it into a shared-memory staging tile
        // as int16 pairs (64 KB; |D| <= K for ternary and binary activations), release it, and only then convert and
        // store -- under the next tile's mainloop. A half whose values do not fit 16 bits (general int8 activations)
        // keeps the accumulator and converts straight from tensor memory through a small int32 tile aliased on its
        // part of the staging area.
        const int h = (warp - kQWarpEpi) >> 2;
        const int et = (warp & 3) * 32 + lane;                // accumulator row == tensor-memory lane
        const int eall = h * 128 + et;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        uint32_t* sS = reinterpret_cast<uint32_t*>(sP) + h * (64 * 128);      // [64 column pairs][128 rows] of this half
        TileOut tout;
        tout.p = &p; tout.s_alpha = s_alpha; tout.s_colsum = s_colsum;
        long long lt = 0;
        for (long long t = cid; t < total_tiles; t += ncl, lt++) {
            const int nt = (int)(t % p.ntiles);
            const long long bm = t / p.ntiles;
            const int mt = 2 * (int)(bm % mpairs) + (int)rank, batch = (int)(bm / mpairs);
            tout.batch = batch; tout.m_base = mt * 128; tout.n_base = nt * NT;
            if (h == 0) {
                const int m = mt * 128 + et;
                s_alpha[et] = (p.out_kind == BGEMM_OUT_F16_SCALED && m < p.M) ? __half2float(p.alpha[(size_t)batch * p.M + m]) : 1.f;
            }
            {
                const int n = nt * NT + eall;
                s_colsum[eall] = (p.epi && n < p.N) ? __ldg(p.colsum + (size_t)batch * p.N + n) : 0;
            }
            bool ok = mbar_wait_relaxed(d_full, (uint32_t)lt & 1, abort_flag, p.status, 49);
            ok = __all_sync(0xffffffffu, ok);
            // One answer for all eight warps (either everybody stores this tile or everybody leaves); the barrier also
            // makes this tile's scales and column sums visible to all of them.
            if (named_bar_or(2, kQEpiThreads, !ok)) break;
            if (warp == kQWarpEpi && lane == 0) BGEMM_TRACE(6, lt * 4);
            tc_fence_after();
            int lo16 = 0, hi16 = 0;                               // value range of this thread's part of the accumulator
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 32) {
                uint32_t v0[16], v1[16];
                tmem_ld16(tmem_d + lane_base + h * 128 + c0, v0);
                tmem_ld16(tmem_d + lane_base + h * 128 + c0 + 16, v1);
                tmem_wait_ld();
#pragma unroll
                for (int q = 0; q < 16; q += 2) {
                    lo16 = min(lo16, min((int)v0[q], (int)v0[q + 1])); hi16 = max(hi16, max((int)v0[q], (int)v0[q + 1]));
                    sS[((c0 + q) >> 1) * 128 + et] = ((uint32_t)v0[q] & 0xffffu) | ((uint32_t)v0[q + 1] << 16);
                }
#pragma unroll
                for (int q = 0; q < 16; q += 2) {
                    lo16 = min(lo16, min((int)v1[q], (int)v1[q + 1])); hi16 = max(hi16, max((int)v1[q], (int)v1[q + 1]));
                    sS[((c0 + 16 + q) >> 1) * 128 + et] = ((uint32_t)v1[q] & 0xffffu) | ((uint32_t)v1[q + 1] << 16);
                }
            }
            // One answer per half: did every value fit 16 bits? (The barrier also publishes the staging tile.)
            const bool wide = named_bar_or(3 + h, 128, lo16 < -32768 || hi16 > 32767);
            if (!wide) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(d_empty_leader);
                if (warp == kQWarpEpi && lane == 0) BGEMM_TRACE(6, lt * 4 + 1);
                if (p.out_layout == BGEMM_LAYOUT_NM) {
                    // unit = (column pair, 8 rows): 16 lanes cover the 128 rows of a column, i.e. 256 contiguous bytes (fp16)
#pragma unroll 1
                    for (int u = et; u < 64 * 16; u += 128) {
                        const int cp = u >> 4, m0 = (u & 15) * 8;
                        const uint4 a = *reinterpret_cast<const uint4*>(sS + cp * 128 + m0);
                        const uint4 b = *reinterpret_cast<const uint4*>(sS + cp * 128 + m0 + 4);
                        const uint32_t wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                        int even[8], odd[8];
#pragma unroll
                        for (int q = 0; q < 8; q++) { even[q] = (int)(short)(wv[q] & 0xffffu); odd[q] = (int)wv[q] >> 16; }
                        store8_rows(tout, h * 128 + 2 * cp, m0, even);
                        store8_rows(tout, h * 128 + 2 * cp + 1, m0, odd);
                    }
                } else {
                    // unit = (row, 8 columns): a lane owns a row
#pragma unroll 1
                    for (int u = et; u < 16 * 128; u += 128) {
                        const int m = u & 127, cp0 = (u >> 7) * 4;
                        int acc[8];
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            const uint32_t wv = sS[(cp0 + q) * 128 + m];
                            acc[2 * q] = (int)(short)(wv & 0xffffu); acc[2 * q + 1] = (int)wv >> 16;
                        }
                        store8_cols(tout, m, h * 128 + 2 * cp0, acc);
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
                    tmem_ld16(tmem_d + lane_base + n0, v0);
                    tmem_ld16(tmem_d + lane_base + n0 + 16, v1);
                    tmem_wait_ld();
                    if (c0 + 32 >= 128) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(d_empty_leader);
                    }
#pragma unroll
                    for (int q = 0; q < 16; q++) sPh[q * 128 + et] = (int)v0[q];
#pragma unroll
                    for (int q = 0; q < 16; q++) sPh[(16 + q) * 128 + et] = (int)v1[q];
                    named_bar_sync(5 + h, 128);
                    write_tile<false>(tout, sPh, 1, 0, n0, 32, et, 128);
                }
            }
            if (warp == kQWarpEpi && lane == 0) BGEMM_TRACE(6, lt * 4 + 2);
            named_bar_sync(7, kQEpiThreads);                      // staging tile, scales and column sums are free for the next tile
        }
    }
    tc_fence_before();
    __syncwarp();
    // Both CTAs are done with each other's barriers and tensor memory before either frees it or exits.
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == kQWarpMma0) {
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

// Shapes the pair kernel takes: wide activation matrices (at least one full 256-column tile), an even number of
// 128-row tiles, no K partitioning, K-block counts the issuers' hand-over protocol covers.
bool pair_supported(const GemmParams& p, long long batch) {
    static const int forced = env_int_q("BGEMM_PAIR");       // 0: never, 1: whenever the shape allows
    if (forced == 0) return false;
    if (p.split_k != 1 || (p.mtiles & 1) || p.N < QCfg::NT || p.out_kind == kOutActs) return false;
    if (p.kblocks < 2 || !(p.kblocks % 2 == 0 || p.kblocks >= QCfg::STAGES)) return false;
    if (p.test_skip_kblock >= 0 && forced != 1) return false;
    const long long tiles = (long long)(p.mtiles / 2) * ((p.N + QCfg::NT - 1) / QCfg::NT) * batch;
    if (forced == 1) return tiles >= 1;
    // worth it when the pairs have at least one round of tiles
    return tiles >= sm_count() / 2;
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
    const long long clusters = total_tiles < sm_count() / 2 ? total_tiles : sm_count() / 2;
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_pair_kernel, tmap, p, total_tiles);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace bgemm
