// Persistent variant of the binary-weight GEMM for launches with many output tiles (pools of layers or heads,
// wide activation matrices): one CTA per SM walks over tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... and
// keeps the operand pipeline running across tile boundaries, while the finished accumulator of the previous
// tile is converted and stored by separate warps. The per-tile set-up, pipeline fill and epilogue that the
// one-tile-per-CTA kernel pays for every 128 x NT tile are paid once per CTA here.
//
// Same math and operand formats as gemm_kernel (gemm_umma.cu); replaces the same reference code
// (PACK_BGEMM_Kernel, lowbit_kernel/csrc/include/kernel_matmul.cuh:370-547).
//
// Tensor memory (all 512 columns): two accumulators of NT columns (tile t is accumulated into buffer t & 1 while the
// epilogue drains the other one) and a ring of u8 weight operand stages of 64 columns.
//   warps 0-15   unpack, sets of four warps taking the K blocks of the CTA's whole K-block stream in turn (four sets with
//                128-column tiles, two with 64-column tiles)
//   warps 16-19  epilogue: accumulator -> shared memory staging tile -> scaled / converted 16-byte stores (with
//                64-column tiles warps 8-11 are a second epilogue group: each group drains one of the two accumulators)
//   warp 20      tensor-memory allocation; one lane issues the UMMAs of the even K blocks of the stream
//   warp 23      one lane issues the UMMAs of the odd K blocks
//   warp 21      one lane streams the packed weight tiles (cp.async.bulk)
//   warp 22      one lane loads the activation tiles (TMA, 128B swizzle)
// All rings are indexed by the running K-block number g of the CTA, so nothing drains between tiles.
#include <cuda.h>
#include <cuda_fp16.h>

#include "epilogue.cuh"
#include "internal.h"
#include "prof.cuh"
#include "ptx.cuh"

namespace bgemm {

// Warp roles: up to 16 unpack warps (sets of four; with two sets warps 8-11 are a second epilogue group and 12-15 exit
// at once), 4 epilogue warps, two UMMA issuers, two copy producers.
constexpr int kPThreads = 768;
constexpr int kPEpiThreads = 128;                 // per epilogue group
constexpr int kPWarpEpi = 16, kPWarpMma0 = 20, kPWarpW = 21, kPWarpB = 22, kPWarpMma1 = 23;
// 768 threads start with 80 registers each; the unpack warps release down to 48 and the four epilogue warps take 160
// (with two epilogue groups: 128 each, and the four warps without a role release down to 24)
constexpr int kPUnpackRegs = 48, kPIdleRegs = 24;
constexpr long long kCopyDrainClocks = 4000000;   // ~2 ms: far beyond any TMA copy of a 32 KB tile

template <int NT>
struct PCfg {
    // One ring of S operand stages: stage s holds the activation tile of a K block in shared memory (NT x 256 B) and
    // the unpacked weight operand of the same K block in tensor memory (64 columns). Filling it takes one arrival
    // of the activation producer (with the TMA byte count) and one of each unpack warp of the set; one
    // tcgen05.commit of the issuer frees both halves. The issuing threads are a scarce resource -- a UMMA costs its
    // issuer ~85 clocks, a commit ~80, a barrier wait ~100 even when it does not block -- so each K block costs its
    // issuer one wait, eight UMMAs and one commit and nothing else.
    static constexpr int A_STAGE_COLS = 64;
    static constexpr int S_FIT = ((512 - 2 * NT) / A_STAGE_COLS) / 2 * 2;
    static constexpr int STAGES = S_FIT > 6 ? 6 : S_FIT;
    static constexpr int A_COL0 = 2 * NT;
    static constexpr int B_STAGE_BYTES = NT * 256;
    // Unpack sets of four warps; set s takes the K blocks g of the stream with g % NSETS == s (always the same operand
    // stage). A set's tensor-memory stores complete only between UMMAs, so a set needs ~2100 clocks per K block whatever
    // the tile width: with 128-column tiles (512 clocks of UMMA per K block) two sets cap the kernel at ~1050 clocks per
    // K block; four sets lift that cap.
    static constexpr int NSETS = NT == 128 ? 4 : 2;
    // Epilogue groups of four warps (a warp reaches the tensor-memory lanes 32 (warp % 4) ... + 31 only). With two
    // unpack sets warps 8-11 form a second group: group g drains accumulator buffer g, i.e. the tiles lt of the CTA with
    // lt % 2 == g, with its own staging tile, scales and barriers. One group alone (four warps, one per scheduler, one
    // dependent instruction every ~5 clocks) needs ~3200 clocks for a 128 x 64 tile -- more than the two K blocks of an
    // attention tile take -- and was what the batched attention product waited for.
    static constexpr int EPI_GROUPS = NSETS == 2 ? 2 : 1;
    static constexpr int EPI_REGS = EPI_GROUPS == 2 ? 128 : 160;
    static constexpr int W_STAGES = NSETS == 4 ? 4 : 6;
    static constexpr int STAGE_TILE_BYTES = NT * 128 * 4;
    // w_full/w_empty, full/empty, d_full[2], d_empty[2], first_done[2], drained
    static constexpr int NBARS = 2 * W_STAGES + 2 * STAGES + 7;
    static constexpr int MISC_BYTES = 512 /*barriers*/ + 512 /*alpha*/ + 1024 /*colsum, per group*/ + 512 /*flags*/ + 512 /*alpha, second group*/;
    static constexpr int SMEM_BYTES = STAGES * B_STAGE_BYTES + W_STAGES * 4096 + EPI_GROUPS * STAGE_TILE_BYTES + MISC_BYTES + 1024 /*align*/;
    // K block g of the CTA's stream uses stage g % STAGES, is unpacked by set g % 2 and issued by issuer g % 2:
    // with even stage counts a stage and its barriers always meet the same set and the same issuer, so every
    // parity wait has seen the previous phase of its barrier.
    static_assert(W_STAGES % NSETS == 0 && STAGES % NSETS == 0 && STAGES % 2 == 0 && STAGES >= 2, "stage -> unpack set / issuer must stay fixed");
    static_assert(NBARS * 8 <= 512, "barrier area");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    // More than half of an SM's shared memory: at most one CTA per SM, so the 512-column allocation never waits
    // for a co-resident CTA of this kernel.
    static_assert(SMEM_BYTES > 114 * 1024, "one CTA per SM");
};

template <int NT>
__global__ void __launch_bounds__(kPThreads, 1) gemm_persist_kernel(const __grid_constant__ CUtensorMap tmap_acts, const GemmParams p, const long long total_tiles) {
    using C = PCfg<NT>;
    BGEMM_TUNING_ONLY(const long long t_cta0 = clock64();)
    grid_launch_dependents();
    if (threadIdx.x == 0) BGEMM_STAMP(10);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sB = smem;
    uint8_t* sW = sB + C::STAGES * C::B_STAGE_BYTES;
    int* sP = reinterpret_cast<int*>(sW + C::W_STAGES * 4096);
    uint8_t* misc = reinterpret_cast<uint8_t*>(sP) + C::EPI_GROUPS * C::STAGE_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc);
    float* s_alpha = reinterpret_cast<float*>(misc + 512);
    int* s_colsum = reinterpret_cast<int*>(misc + 1024);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(misc + 2048);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const uint32_t w_full = smem_u32(bars);
    const uint32_t w_empty = w_full + 8 * C::W_STAGES;
    const uint32_t full = w_empty + 8 * C::W_STAGES;     // [S] operand stage filled (activation bytes + four unpack warps)
    const uint32_t empty = full + 8 * C::STAGES;         // [S] operand stage consumed (one commit)
    const uint32_t d_full = empty + 8 * C::STAGES;       // [2] accumulator buffer complete (one commit per issuer)
    const uint32_t d_empty = d_full + 16;                // [2] accumulator buffer read out (one arrive per epilogue warp)
    const uint32_t first_done = d_empty + 16;            // [2] per buffer: the K block that zeroes it has been executed
    const uint32_t drained = first_done + 16;            // every UMMA of the CTA has been executed (one commit per issuer)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = p.kblocks;
    // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ... (tile index = (batch * mtiles + mt) * ntiles + nt)
    const long long my_tiles = (total_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;

    if (warp == 0) {
        for (int i = lane; i < C::NBARS; i += 32) {
            const int f0 = 2 * C::W_STAGES, d0 = f0 + 2 * C::STAGES;
            int count = 1;
            if (i >= C::W_STAGES && i < 2 * C::W_STAGES) count = 4;           // w_empty: unpack warps of a set
            else if (i >= f0 && i < f0 + C::STAGES) count = 5;                // full: activation producer + unpack warps of a set
            else if (i == d0 || i == d0 + 1) count = 2;                       // d_full: both issuers
            else if (i == d0 + 2 || i == d0 + 3) count = 4;                   // d_empty: epilogue warps
            else if (i == d0 + 6) count = 2;                                  // drained: both issuers
            mbar_init(w_full + 8 * i, count);
        }
        if (lane == 0) { *abort_flag = 0; set_wait_budget(abort_flag, p.wait_budget); }
        mbar_fence_init();
    } else if (warp == kPWarpB) {
        if (lane == 0) tma_prefetch_desc(&tmap_acts);
    } else if (warp == kPWarpMma0) {
        tmem_alloc(smem_u32(tmem_holder), 512);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    grid_dependency_wait();      // nothing above touches global memory (programmatic dependent launch)
    const uint32_t tmem = *tmem_holder;
    const uint32_t tmem_d = tmem;
    const uint32_t tmem_a = tmem + C::A_COL0;
    if (tid == 0) BGEMM_STAMP(1);

    if (warp == kPWarpW) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            long long g = 0;
            BGEMM_TUNING_ONLY(long long tw = 0;)
            bool ok = true;
            for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const long long bm = t / p.ntiles;                      // batch * mtiles + mt
                const int mt = (int)(bm % p.mtiles), batch = (int)(bm / p.mtiles);
                const uint8_t* src = p.plane + (size_t)batch * p.plane_batch_bytes + (size_t)mt * nkb * 4096;
                for (int i = 0; i < nkb; i++, g++) {
                    const int s = (int)(g % C::W_STAGES);
                    if (g >= C::W_STAGES) BGEMM_TIMED(tw, ok = mbar_wait_relaxed(w_empty + 8 * s, (uint32_t)((g / C::W_STAGES) - 1) & 1, abort_flag, p.status, 21));
                    if (!ok) break;
                    if (g == p.test_skip_kblock) continue;          // test hook: this K block never arrives, its consumers' waits run out
                    mbar_arrive_expect_tx(w_full + 8 * s, 4096);
                    bulk_g2s(smem_u32(sW + s * 4096), src + (size_t)i * 4096, 4096, w_full + 8 * s);
                }
            }
            BGEMM_PUT(20, tw);
            if (*abort_flag) {  // drain own copies before the CTA may exit
                for (long long i = g - 1; i >= 0 && i >= g - C::W_STAGES; i--) {
                    const long long t0 = clock64();
                    while (!mbar_test(w_full + 8 * (int)(i % C::W_STAGES), (uint32_t)(i / C::W_STAGES) & 1) && clock64() - t0 < wait_budget_of(abort_flag)) {}
                }
            }
        }
    } else if (warp == kPWarpB) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            long long g = 0;
            BGEMM_TUNING_ONLY(long long tw = 0;)
            bool ok = true;
            for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int nt = (int)(t % p.ntiles);
                const int batch = (int)(t / p.ntiles / p.mtiles);
                for (int i = 0; i < nkb; i++, g++) {
                    const int s = (int)(g % C::STAGES);
                    if (g >= C::STAGES) BGEMM_TIMED(tw, ok = mbar_wait_relaxed(empty + 8 * s, (uint32_t)((g / C::STAGES) - 1) & 1, abort_flag, p.status, 22));
                    if (!ok) break;
                    BGEMM_TRACE(4, g);
                    mbar_arrive_expect_tx(full + 8 * s, C::B_STAGE_BYTES);
                    const uint32_t dst = smem_u32(sB + s * C::B_STAGE_BYTES);
                    tma_load_3d(dst, &tmap_acts, i * 256, nt * NT, batch, full + 8 * s);
                    tma_load_3d(dst + NT * 128, &tmap_acts, i * 256 + 128, nt * NT, batch, full + 8 * s);
                }
            }
            BGEMM_PUT(21, tw);
            if (*abort_flag) {
                // The copies in flight must land before the CTA may exit. Their barriers also need the unpack warps,
                // which have stopped: wait for the longest plausible copy time instead of the barrier.
                const long long t0 = clock64();
                while (g > 0 && clock64() - t0 < kCopyDrainClocks) {}
            }
        }
    } else if (warp == kPWarpMma0 || warp == kPWarpMma1) {
        // ---------------- UMMA issuers: issuer `me` takes the K blocks with g % 2 == me ----------------
        const int me = warp == kPWarpMma0 ? 0 : 1;
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_u8s8(NT);
            bool ok = true;
            long long g = 0;
            BGEMM_TUNING_ONLY(long long twf = 0, twd = 0;)
            BGEMM_TUNING_ONLY(const long long tloop0 = clock64();)
            for (long long lt = 0; lt < my_tiles && ok; lt++) {
                const int buf = (int)(lt & 1);
                const uint32_t k = (uint32_t)(lt >> 1);             // use number of this accumulator buffer
                const uint32_t d = tmem_d + buf * NT;
                // The first K block of a tile overwrites the accumulator (accumulate = 0). Its issuer (the "opener",
                // whoever owns that K block) waits until the epilogue has read the buffer out (tile lt - 2); the other
                // issuer waits until that K block has been executed before it adds anything. Integer accumulation
                // commutes, so no other order is needed.
                // Parity waits must not name a phase the barrier has not reached. d_empty[buf]: phase k - 2 was
                // awaited by the opener of tile lt - 2 and the other issuer waited for that tile to be opened.
                // first_done[buf]: the waiter either waited for phase k - 1 itself (tile lt - 2; always so when tiles
                // have an even number of K blocks) or committed it and has since reused one of its operand stages
                // (odd K-block counts are only launched with at least STAGES K blocks per tile), whose release was
                // committed after first_done. Neither barrier can be two phases
                // ahead: that needs the epilogue of tile lt, which needs this issuer's d_full commit below.
                const bool opener = (int)(g & 1) == me;
                if (opener) {
                    if (k >= 1) BGEMM_TIMED(twd, ok = mbar_wait(d_empty + 8 * buf, (k - 1) & 1, abort_flag, p.status, 25));
                } else {
                    BGEMM_TIMED(twd, ok = mbar_wait(first_done + 8 * buf, k & 1, abort_flag, p.status, 26));
                }
                if (!ok) break;
                tc_fence_after();
                for (int i = 0; i < nkb; i++, g++) {
                    if ((int)(g & 1) != me) continue;
                    const int s = (int)(g % C::STAGES);
                    BGEMM_TIMED(twf, ok = mbar_wait(full + 8 * s, (uint32_t)(g / C::STAGES) & 1, abort_flag, p.status, 23));
                    if (!ok) break;
                    BGEMM_TRACE(0, g);
                    tc_fence_after();
                    const uint32_t bbase = smem_u32(sB + s * C::B_STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint64_t bdesc = umma_desc_sw128(bbase + (j >> 2) * (NT * 128) + (j & 3) * 32);
                        umma_i8_ts(d, tmem_a + s * C::A_STAGE_COLS + j * 8, bdesc, idesc, (i | j) ? 1u : 0u);
                    }
                    if (i == 0) umma_commit(first_done + 8 * buf);
                    umma_commit(empty + 8 * s);
                    BGEMM_TRACE(1, g);
                }
                if (!ok) break;
                umma_commit(d_full + 8 * buf);
            }
            umma_commit(drained);
            if (me == 0) { BGEMM_PUT(16, twf); BGEMM_PUT(24, clock64() - tloop0); BGEMM_PUT(27, twd); }
        }
    } else if (warp < 4 * C::NSETS) {
        // ---------------- unpack: set s = warps 4 s .. 4 s + 3 takes the K blocks g of the stream with g % NSETS == s ----
        regs_release<kPUnpackRegs>();
        const int set = warp >> 2;
        const int r = (warp & 3) * 32 + lane;                 // weight row of the tile == tensor-memory lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        const long long total_kb = my_tiles * nkb;
        bool ok = true;
        BGEMM_TUNING_ONLY(long long tww = 0, twe = 0;)
        BGEMM_TUNING_ONLY(const long long tloop0 = clock64();)
        for (long long g = set; g < total_kb && ok; g += C::NSETS) {
            const int ws = (int)(g % C::W_STAGES);
            BGEMM_TIMED(tww, ok = mbar_wait(w_full + 8 * ws, (uint32_t)(g / C::W_STAGES) & 1, abort_flag, p.status, 27));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if ((tid & 127) == 0) BGEMM_TRACE(5, g);
            const uint4 lo = *reinterpret_cast<const uint4*>(sW + ws * 4096 + r * 16);
            const uint4 hi = *reinterpret_cast<const uint4*>(sW + ws * 4096 + 2048 + r * 16);
            fence_proxy_async_smem();     // generic-proxy reads before the producer's next bulk copy into this stage
            __syncwarp();
            if (lane == 0) mbar_arrive(w_empty + 8 * ws);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            const int as = (int)(g % C::STAGES);
            if (g >= C::STAGES) BGEMM_TIMED(twe, ok = mbar_wait_relaxed(empty + 8 * as, (uint32_t)((g / C::STAGES) - 1) & 1, abort_flag, p.status, 28));
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
            if (lane == 0) mbar_arrive(full + 8 * as);
            if ((tid & 127) == 0) BGEMM_TRACE(3, g);
        }
        if (tid == 0) { BGEMM_PUT(18, tww); BGEMM_PUT(19, twe); BGEMM_PUT(25, clock64() - tloop0); }
        if (tid == 128) { BGEMM_PUT(22, tww); BGEMM_PUT(23, twe); }
    } else if ((warp >= kPWarpEpi && warp < kPWarpEpi + 4) || (C::EPI_GROUPS == 2 && warp >= 8 && warp < 12)) {
        // ---------------- epilogue: overlaps the mainloop of the next tile ----------------
        regs_request<C::EPI_REGS>();
        const int ge = warp >= kPWarpEpi ? 0 : 1;             // epilogue group
        const int et = (warp & 3) * 32 + lane;                // 0..127 == accumulator row == tensor-memory lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        if (ge) {                                             // the second group's staging tile, scales and column sums
            sP += C::STAGE_TILE_BYTES / 4;
            s_alpha = reinterpret_cast<float*>(misc + 2560);
            s_colsum += 128;
        }
        const int bar_a = 2 + 2 * ge, bar_b = 3 + 2 * ge;     // named barriers of the group
        TileOut tout;
        tout.p = &p; tout.s_alpha = s_alpha; tout.s_colsum = s_colsum;
        // [M, N] results are stored straight from registers (the same for [N, M] results -- 2-byte stores a row pitch
        // apart -- measured 2.4 x slower than the staged path: 381 against 158 us on the 95-layer pool)
        const bool direct = p.out_layout == BGEMM_LAYOUT_MN && p.out_kind != kOutActs;
        BGEMM_TUNING_ONLY(long long twd = 0, tbusy = 0;)
        long long lt = ge;
        for (long long t = blockIdx.x + (long long)ge * gridDim.x; t < total_tiles; t += (long long)C::EPI_GROUPS * gridDim.x, lt += C::EPI_GROUPS) {
            const int nt = (int)(t % p.ntiles);
            const long long bm = t / p.ntiles;
            const int mt = (int)(bm % p.mtiles), batch = (int)(bm / p.mtiles);
            const int buf = (int)(lt & 1);
            tout.batch = batch; tout.m_base = mt * 128; tout.n_base = nt * NT;
            {
                const int m = mt * 128 + et;
                s_alpha[et] = ((p.out_kind == BGEMM_OUT_F16_SCALED || (p.out_kind == kOutActs && p.alpha)) && m < p.M) ? __half2float(p.alpha[(size_t)batch * p.M + m]) : 1.f;
            }
            for (int i = et; i < NT; i += kPEpiThreads) {
                const int n = nt * NT + i;
                s_colsum[i] = (p.epi && n < p.N) ? __ldg(p.colsum + (size_t)batch * p.N + n) : 0;
            }
            bool ok;
            BGEMM_TIMED(twd, ok = mbar_wait_relaxed(d_full + 8 * buf, (uint32_t)(lt >> 1) & 1, abort_flag, p.status, 29));
            ok = __all_sync(0xffffffffu, ok);
#ifdef BGEMM_TUNING
            const long long tb0 = p.prof ? clock64() : 0;
#endif
            if (direct) {
                // [M, N] results: an accumulator row leaves tensor memory as consecutive columns, which are consecutive
                // addresses of the result row -- they are converted and stored straight from registers (no staging, no
                // second pass); the barrier makes this tile's scales and column sums visible to all four warps.
                if (named_bar_or(bar_a, kPEpiThreads, !ok)) break;
                tc_fence_after();
#pragma unroll 1
                for (int n0 = 0; n0 < NT; n0 += 32) {
                    uint32_t v0[16], v1[16];
                    tmem_ld16(tmem_d + buf * NT + lane_base + n0, v0);
                    tmem_ld16(tmem_d + buf * NT + lane_base + n0 + 16, v1);
                    tmem_wait_ld();
                    if (n0 + 32 >= NT) {                         // the last columns are in registers: the accumulator may be overwritten
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(d_empty + 8 * buf);
                    }
#pragma unroll
                    for (int c = 0; c < 2; c++) {
                        const int a0[8] = {(int)v0[8 * c], (int)v0[8 * c + 1], (int)v0[8 * c + 2], (int)v0[8 * c + 3],
                                           (int)v0[8 * c + 4], (int)v0[8 * c + 5], (int)v0[8 * c + 6], (int)v0[8 * c + 7]};
                        store8_cols(tout, et, n0 + 8 * c, a0);
                        const int a1[8] = {(int)v1[8 * c], (int)v1[8 * c + 1], (int)v1[8 * c + 2], (int)v1[8 * c + 3],
                                           (int)v1[8 * c + 4], (int)v1[8 * c + 5], (int)v1[8 * c + 6], (int)v1[8 * c + 7]};
                        store8_cols(tout, et, n0 + 16 + 8 * c, a1);
                    }
                }
            } else {
            if (ok) {
                tc_fence_after();
#pragma unroll 1
                for (int n0 = 0; n0 < NT; n0 += 32) {
                    uint32_t v0[16], v1[16];
                    tmem_ld16(tmem_d + buf * NT + lane_base + n0, v0);
                    tmem_ld16(tmem_d + buf * NT + lane_base + n0 + 16, v1);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < 16; q++) sP[(n0 + q) * 128 + et] = (int)v0[q];
#pragma unroll
                    for (int q = 0; q < 16; q++) sP[(n0 + 16 + q) * 128 + et] = (int)v1[q];
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(d_empty + 8 * buf);   // the accumulator may be overwritten from here on
            }
            // One answer for all four warps: either everybody stores this tile or everybody leaves.
            if (named_bar_or(bar_a, kPEpiThreads, !ok)) break;
            write_tile<false>(tout, sP, 1, 0, 0, NT, et, kPEpiThreads);
            }
            named_bar_sync(bar_b, kPEpiThreads);                      // staging tile and scales are free for the next tile
#ifdef BGEMM_TUNING
            if (p.prof) tbusy += clock64() - tb0;
#endif
        }
        if (et == 0 && ge == 0) { BGEMM_PUT(28, twd); BGEMM_PUT(29, tbusy); }
    } else if (warp < 16) {
        regs_release<kPIdleRegs>();     // no role in this variant: the registers go to the epilogue warps
    }
    if (tid == 0) BGEMM_STAMP(8);
    tc_fence_before();
    __syncthreads();
    if (warp == kPWarpMma0) {
        if (lane == 0) {   // every UMMA has been executed before the columns are freed (immediate unless a wait ran out)
            const long long t0 = clock64();
            while (!mbar_test(drained, 0) && clock64() - t0 < wait_budget_of(abort_flag)) {}
        }
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
    if (tid == 0) { BGEMM_STAMP(9); BGEMM_STAMP(11); }
}

template <int NT>
static int launch_persist_variant(cudaStream_t stream, const CUtensorMap& tmap, const GemmParams& p, long long total_tiles, int ctas) {
    using C = PCfg<NT>;
    if (!persistent_kblocks_ok(NT, p.kblocks)) return BGEMM_ERR_UNSUPPORTED;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_persist_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, 1, 1);
    cfg.blockDim = dim3(kPThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (programmatic_launch_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_persist_kernel<NT>, tmap, p, total_tiles);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

bool persistent_supported(int NT) { return NT == 64 || NT == 128; }

// With an even number of K blocks per tile issuer 0 opens every tile and issuer 1 waits for every phase of
// first_done itself. With an odd number the opener alternates, and the argument in the issuer loop needs tiles of at
// least STAGES K blocks.
bool persistent_kblocks_ok(int NT, int kblocks) {
    const int stages = NT == 64 ? PCfg<64>::STAGES : PCfg<128>::STAGES;
    return kblocks >= 2 && (kblocks % 2 == 0 || kblocks >= stages);
}

int launch_gemm_persistent(cudaStream_t stream, const void* tensor_map, const GemmParams& p, int NT, long long total_tiles, int ctas) {
    const CUtensorMap& tmap = *static_cast<const CUtensorMap*>(tensor_map);
    switch (NT) {
        case 64: return launch_persist_variant<64>(stream, tmap, p, total_tiles, ctas);
        case 128: return launch_persist_variant<128>(stream, tmap, p, total_tiles, ctas);
        default: return BGEMM_ERR_UNSUPPORTED;
    }
}

}  // namespace bgemm
