// Binary-weight GEMM mainloop for sm_100a: packed 1-bit weights are unpacked on chip to u8 and fed to
// tcgen05.mma kind::i8 as the A operand straight from tensor memory; int8 activations arrive by TMA.
//
// Replaces PACK_BGEMM_Kernel (lowbit_kernel/csrc/include/kernel_matmul.cuh:370-547) and the separate
// SplitK_Reduction launch (kernel_reduction.cuh:29-48) of the reference. The legacy b1 mma.sync path
// the reference uses runs at ~0.4 POP/s on B200 (measured), an order of magnitude below kind::i8.
//
// One CTA computes a 128(M) x NT(N) tile over a K range [kb0, kb1) of 256-column blocks.
//   warps 0-7  unpack, two sets of four warps taking alternate K blocks: thread r of a set owns weight row r
//              of the tile; per K block it reads its 32 packed bytes from shared memory, expands them to
//              8 x (128 x 32) u8 operand slices with one or two logic ops per 4 elements, and writes them to
//              tensor memory (tcgen05.st). Afterwards all eight warps run the epilogue.
//   warp 8     allocates tensor memory; one lane issues the 8 UMMAs (128 x NT x 32) of every even K block.
//   warp 11    one lane issues the UMMAs of the odd K blocks. Issuing a UMMA blocks the thread until the tensor pipe
//              accepts it and an mbarrier poll costs it ~200 clocks, so one issuer leaves the pipe idle between K
//              blocks; two issuers, each polling while the other feeds the pipe, keep it busy (measured 1.4x).
//   warp 9     one lane streams the packed weight tiles (4 KB each, contiguous) with cp.async.bulk.
//   warp 10    one lane loads the activation tiles [NT x 256 B] with two 128B-swizzled TMA boxes.
//
// POW2 variant (NT <= 32, weight-streaming shapes): slice j keeps the weight bit at byte value 2^j
// (a single AND per 4 elements) and accumulates into its own accumulator D_j; the epilogue adds
// D_j >> j. The plain variant shifts the bit down to {0,1} and uses one accumulator.
//
// With D = sum_k bit_w(k) * x(k):  XOR / BWTA results are colsum_x[n] - 2 D, AND / ATTN results are D.
//
// Epilogue: the accumulator tile leaves tensor memory into shared memory as int32 [NT][128]; K partitions
// are then summed -- by the CTAs of a thread-block cluster through distributed shared memory (up to 8
// partitions), or through a global workspace by the last CTA to arrive (more than 8) -- and the result is
// converted (fused per-row scale) and stored with 16-byte coalesced stores.
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "epilogue.cuh"
#include "internal.h"
#include "prof.cuh"
#include "ptx.cuh"

namespace bgemm {

constexpr int kUnpackThreads = 256;
constexpr int kGemmThreads = 384;
constexpr int kWarpMma = 8, kWarpW = 9, kWarpB = 10, kWarpMma2 = 11;

__host__ __device__ constexpr int pow2_ceil(int v) {
    int p = 32;
    while (p < v) p <<= 1;
    return p;
}

// DEEP: the CTA takes all 512 tensor-memory columns (one CTA per SM, six K blocks of operand in flight) -- best
// when the launch has at most one CTA per SM. Otherwise 256 columns, two CTAs per SM covering each other's bubbles.
template <int NT, bool POW2, bool DEEP>
struct Cfg {
    static constexpr int D_COLS = POW2 ? 8 * NT : NT;
    static constexpr int TMEM_BUDGET = (DEEP || D_COLS >= 256) ? 512 : 256;
    // An A stage holds G-th of a K block: 8 / G operand slices of 8 columns each. The unpack -> UMMA -> release
    // round trip of a stage costs ~1500 clocks of signalling latency, so the ring must hold several K blocks of
    // operand for the tensor pipe to stay busy: it takes everything D leaves of the 512 columns.
    static constexpr int G = 1;
    static constexpr int A_STAGE_COLS = 64 / G;
    static constexpr int A_FIT = ((TMEM_BUDGET - D_COLS) / A_STAGE_COLS) / (2 * G) * (2 * G);
    static constexpr int A_STAGES = A_FIT > 6 * G ? 6 * G : A_FIT;
    static constexpr int A_COL0 = D_COLS;
    static constexpr int TMEM_COLS = pow2_ceil(D_COLS + A_STAGE_COLS * A_STAGES);
    static constexpr int B_STAGE_BYTES = NT * 256;
    static constexpr bool ONE_PER_SM = TMEM_BUDGET == 512;
    static constexpr int B_STAGES = NT <= 32 ? 8 : (NT == 64 ? (ONE_PER_SM ? 6 : 4) : (NT == 128 ? (ONE_PER_SM ? 5 : 3) : 3));
    static constexpr int W_STAGES = NT == 256 ? 4 : ((NT == 128 && !ONE_PER_SM) ? 2 : 8);
    // Tiles of 256 columns are bound by UMMA execution even with one issuer; narrower ones use two.
    static constexpr int NMMA = NT == 256 ? 1 : 2;
    static constexpr int NBARS = 2 * W_STAGES + 2 * B_STAGES + 2 * A_STAGES + 2;
    static constexpr int MISC_BYTES = 512 /*barriers*/ + 512 /*alpha*/ + 1024 /*colsum*/ + 512 /*flags*/;
    // Epilogue staging aliases the activation and weight stages: one [NT][128] int32 tile, or -- K partitions in a
    // cluster -- up to (NT + 7 * 8) columns of partial sums received from the peers.
    static constexpr int STAGE_TILE_BYTES = (NT + 56) * 128 * 4;
    static_assert(128 * row_pitch_of(NT) * 4 <= STAGE_TILE_BYTES, "row-major staging");
    static constexpr int SMEM_USED = B_STAGES * B_STAGE_BYTES + W_STAGES * 4096 + MISC_BYTES + 1024 /*align*/;
    // Co-resident CTAs must not ask for more tensor memory than the SM has (a later tcgen05.alloc would
    // stall until an earlier CTA exits): request enough shared memory to cap residency at 512 / TMEM_COLS.
    static constexpr int SMEM_FLOOR = TMEM_COLS == 512 ? 117 * 1024 : 77 * 1024;
    static constexpr int SMEM_BYTES = SMEM_USED > SMEM_FLOOR ? SMEM_USED : SMEM_FLOOR;
    static constexpr int MIN_CTAS = TMEM_COLS <= 256 ? 2 : 1;
    // The two unpack sets take alternate K blocks. With even stage counts a stage (and its barriers) is always
    // served by the same set, so every waiter has seen the previous phase of the barrier it waits on; with an
    // odd count a set's first wait on a barrier would name phase 1 and pass before phase 0 has completed.
    static_assert(W_STAGES % 2 == 0 && A_STAGES % (2 * G) == 0, "stage counts shared by the two unpack sets must keep stage -> set fixed");
    static_assert(TMEM_COLS <= 512, "tensor memory budget");
    static_assert(NT % 16 == 0 && NT >= 16 && NT <= 256, "UMMA N");
    static_assert(NBARS * 8 <= 512, "barrier area");
    static_assert(STAGE_TILE_BYTES <= B_STAGES * B_STAGE_BYTES + W_STAGES * 4096, "staging must fit in the operand stages");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

template <int NT, bool POW2, bool DEEP>
__global__ void __launch_bounds__(kGemmThreads, Cfg<NT, POW2, DEEP>::MIN_CTAS) gemm_kernel(const __grid_constant__ CUtensorMap tmap_acts, const GemmParams p) {
    using C = Cfg<NT, POW2, DEEP>;
    BGEMM_TUNING_ONLY(const long long t_cta0 = clock64();)
    grid_launch_dependents();
    if (threadIdx.x == 0) BGEMM_STAMP(10);
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sB = smem;
    uint8_t* sW = sB + C::B_STAGES * C::B_STAGE_BYTES;
    uint8_t* misc = sW + C::W_STAGES * 4096;
    uint64_t* bars = reinterpret_cast<uint64_t*>(misc);
    float* s_alpha = reinterpret_cast<float*>(misc + 512);
    int* s_colsum = reinterpret_cast<int*>(misc + 1024);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(misc + 2048);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    int* last_flag = reinterpret_cast<int*>(tmem_holder + 2);

    const uint32_t w_full = smem_u32(bars);
    const uint32_t w_empty = w_full + 8 * C::W_STAGES;
    const uint32_t b_full = w_empty + 8 * C::W_STAGES;
    const uint32_t b_empty = b_full + 8 * C::B_STAGES;
    const uint32_t a_full = b_empty + 8 * C::B_STAGES;
    const uint32_t a_empty = a_full + 8 * C::A_STAGES;
    const uint32_t d_full = a_empty + 8 * C::A_STAGES;
    const uint32_t first_done = d_full + 8;       // K block 0 (which zeroes the accumulators) has been executed

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nt = blockIdx.x;
    const int split = blockIdx.y % p.split_k;     // == rank inside the cluster when p.cluster
    const int mt = blockIdx.y / p.split_k;
    const int batch = blockIdx.z;
    const int kb0 = (int)(((long long)p.kblocks * split) / p.split_k);
    const int kb1 = (int)(((long long)p.kblocks * (split + 1)) / p.split_k);
    const int nkb = kb1 - kb0;

    if (warp == 0) {
        // barrier i of the area: arrival count 4 for the two kinds that collect one arrival per unpack warp
        for (int i = lane; i < C::NBARS; i += 32) {
            const bool four = (i >= C::W_STAGES && i < 2 * C::W_STAGES) ||
                              (i >= 2 * C::W_STAGES + 2 * C::B_STAGES && i < 2 * C::W_STAGES + 2 * C::B_STAGES + C::A_STAGES);
            const bool per_issuer = i == C::NBARS - 2 ||                                              // d_full
                                    (i >= 2 * C::W_STAGES + C::B_STAGES && i < 2 * C::W_STAGES + 2 * C::B_STAGES);   // b_empty
            mbar_init(w_full + 8 * i, four ? 4 : (per_issuer ? C::NMMA : 1));
        }
        if (lane == 0) { *abort_flag = 0; *last_flag = 0; set_wait_budget(abort_flag, p.wait_budget); }
        mbar_fence_init();
    } else if (warp == kWarpB) {
        if (lane == 0) tma_prefetch_desc(&tmap_acts);
    } else if (warp == kWarpMma) {
        tmem_alloc(smem_u32(tmem_holder), C::TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Everything above touches no global memory, so under programmatic dependent launch it overlaps the tail of
    // the previous kernel in the stream; from here on that kernel's results are needed.
    grid_dependency_wait();
    const uint32_t tmem = *tmem_holder;
    const uint32_t tmem_d = tmem;
    const uint32_t tmem_a = tmem + C::A_COL0;
    if (tid == 0) BGEMM_STAMP(1);

    if (warp == kWarpW) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            const uint8_t* src = p.plane + (size_t)batch * p.plane_batch_bytes + ((size_t)mt * p.kblocks + kb0) * 4096;
            int issued = 0;
            BGEMM_TUNING_ONLY(long long tw = 0;)
            for (int i = 0; i < nkb; i++) {
                const int s = i % C::W_STAGES;
                bool okw = true;
                if (i >= C::W_STAGES) BGEMM_TIMED(tw, okw = mbar_wait(w_empty + 8 * s, ((i / C::W_STAGES) - 1) & 1, abort_flag, p.status, 11));
                if (!okw) break;
                if (kb0 + i == p.test_skip_kblock) continue;      // test hook: this K block never arrives, its consumers' waits run out
                mbar_arrive_expect_tx(w_full + 8 * s, 4096);
                bulk_g2s(smem_u32(sW + s * 4096), src + (size_t)i * 4096, 4096, w_full + 8 * s);
                if (i == 0) BGEMM_STAMP(2);
                issued = i + 1;
            }
            BGEMM_PUT(20, tw);
            if (*abort_flag) {  // drain own copies before the CTA may exit
                for (int i = issued - 1; i >= 0 && i >= issued - C::W_STAGES; i--) {
                    const long long t0 = clock64();
                    while (!mbar_test(w_full + 8 * (i % C::W_STAGES), (i / C::W_STAGES) & 1) && clock64() - t0 < wait_budget_of(abort_flag)) {}
                }
            }
        }
    } else if (warp == kWarpB) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            int issued = 0;
            BGEMM_TUNING_ONLY(long long tw = 0;)
            for (int i = 0; i < nkb; i++) {
                const int s = i % C::B_STAGES;
                bool okb = true;
                if (i >= C::B_STAGES) BGEMM_TIMED(tw, okb = mbar_wait(b_empty + 8 * s, ((i / C::B_STAGES) - 1) & 1, abort_flag, p.status, 12));
                if (!okb) break;
                mbar_arrive_expect_tx(b_full + 8 * s, C::B_STAGE_BYTES);
                const uint32_t dst = smem_u32(sB + s * C::B_STAGE_BYTES);
                tma_load_3d(dst, &tmap_acts, (kb0 + i) * 256, nt * NT, batch, b_full + 8 * s);
                tma_load_3d(dst + NT * 128, &tmap_acts, (kb0 + i) * 256 + 128, nt * NT, batch, b_full + 8 * s);
                issued = i + 1;
            }
            BGEMM_PUT(21, tw);
            if (*abort_flag) {
                for (int i = issued - 1; i >= 0 && i >= issued - C::B_STAGES; i--) {
                    const long long t0 = clock64();
                    while (!mbar_test(b_full + 8 * (i % C::B_STAGES), (i / C::B_STAGES) & 1) && clock64() - t0 < wait_budget_of(abort_flag)) {}
                }
            }
        }
    } else if (warp == kWarpMma || warp == kWarpMma2) {
        // ---------------- UMMA issuers: issuer `me` takes K blocks me, me + NMMA, ... ----------------
        const int me = warp == kWarpMma ? 0 : 1;
        if (lane == 0 && me < C::NMMA) {
            constexpr uint32_t idesc = umma_idesc_u8s8(NT);
            bool ok = true;
            BGEMM_TUNING_ONLY(long long twa = 0, twb = 0;)
            BGEMM_TUNING_ONLY(const long long tloop0 = clock64();)
            // Integer accumulation commutes, so the two issuers need no mutual order -- except that the UMMAs of K
            // block 0 overwrite the accumulators (accumulate = 0) and must run before anything is added.
            if (me == 1 && nkb > 1) ok = mbar_wait(first_done, 0, abort_flag, p.status, 18);
            for (int i = 0; i < nkb && ok; i++) {
                const int bs = i % C::B_STAGES;
                // Both issuers observe EVERY phase of every activation barrier and both release it (the owner of the K
                // block through tcgen05.commit after its UMMAs, the other with a plain arrive): the producer cannot
                // refill a stage -- and its barrier cannot advance -- before both have seen the phase, so a parity
                // wait can never be a phase behind. That keeps the stage count free of parity constraints.
                BGEMM_TIMED(twb, ok = mbar_wait(b_full + 8 * bs, (i / C::B_STAGES) & 1, abort_flag, p.status, 14));
                if (!ok) break;
                if ((i % C::NMMA) != me) { mbar_arrive(b_empty + 8 * bs); continue; }
                const uint32_t bbase = smem_u32(sB + bs * C::B_STAGE_BYTES);
#pragma unroll
                for (int g = 0; g < C::G && ok; g++) {
                    const int h = C::G * i + g, as = h % C::A_STAGES;
                    BGEMM_TIMED(twa, ok = mbar_wait(a_full + 8 * as, (h / C::A_STAGES) & 1, abort_flag, p.status, 13));
                    if (!ok) break;
                    tc_fence_after();
                    if (h == 0) BGEMM_STAMP(5);
#pragma unroll
                    for (int jj = 0; jj < 8 / C::G; jj++) {
                        const int j = (8 / C::G) * g + jj;
                        const uint64_t bdesc = umma_desc_sw128(bbase + (j >> 2) * (NT * 128) + (j & 3) * 32);
                        const uint32_t d = tmem_d + (POW2 ? j * NT : 0);
                        const uint32_t acc = POW2 ? (i > 0 ? 1u : 0u) : ((i | j) ? 1u : 0u);
                        umma_i8_ts(d, tmem_a + as * C::A_STAGE_COLS + jj * 8, bdesc, idesc, acc);
                    }
                    umma_commit(a_empty + 8 * as);
                }
                umma_commit(b_empty + 8 * bs);
                if (i == 0) umma_commit(first_done);
            }
            umma_commit(d_full);
            if (me == 0) { BGEMM_STAMP(6); BGEMM_PUT(16, twa); BGEMM_PUT(17, twb); BGEMM_PUT(24, clock64() - tloop0); }
        }
    } else {
        // ---------------- unpack: set 0 = warps 0-3 takes even K blocks, set 1 = warps 4-7 odd ones ----------------
        const int set = warp >> 2;
        const int r = (warp & 3) * 32 + lane;                 // weight row of the tile == tensor-memory lane
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        // per-row scales and column sums of this tile (needed by the epilogue only; their latency hides behind
        // the first weight load)
        if (tid < 128) {
            const int m = mt * 128 + tid;
            s_alpha[tid] = ((p.out_kind == BGEMM_OUT_F16_SCALED || (p.out_kind == kOutActs && p.alpha)) && m < p.M) ? __half2float(p.alpha[(size_t)batch * p.M + m]) : 1.f;
        }
        for (int i = tid; i < NT; i += kUnpackThreads) {
            const int n = nt * NT + i;
            s_colsum[i] = (p.epi && n < p.N) ? __ldg(p.colsum + (size_t)batch * p.N + n) : 0;
        }
        bool ok = true;
        BGEMM_TUNING_ONLY(long long tww = 0, twe = 0, tst = 0;)
        BGEMM_TUNING_ONLY(const long long tloop0 = clock64();)
        for (int i = set; i < nkb && ok; i += 2) {
            const int ws = i % C::W_STAGES;
            BGEMM_TIMED(tww, ok = mbar_wait(w_full + 8 * ws, (i / C::W_STAGES) & 1, abort_flag, p.status, 15));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (i == 0 && tid == 0) BGEMM_STAMP(3);
            const uint4 lo = *reinterpret_cast<const uint4*>(sW + ws * 4096 + r * 16);
            const uint4 hi = *reinterpret_cast<const uint4*>(sW + ws * 4096 + 2048 + r * 16);
            // The stage goes back to the producer, whose next bulk copy (async proxy) overwrites it: the proxy fence
            // orders these generic-proxy reads before it. Without it one warp's 32 rows were now and then computed from
            // the weights of the K block two ahead (two-stage ring, neighbour CTA saturating the load/store path).
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(w_empty + 8 * ws);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int g = 0; g < C::G; g++) {
                const int h = C::G * i + g, as = h % C::A_STAGES;
                if (h >= C::A_STAGES) BGEMM_TIMED(twe, ok = mbar_wait(a_empty + 8 * as, ((h / C::A_STAGES) - 1) & 1, abort_flag, p.status, 16));
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int jj = 0; jj < 8 / C::G; jj++) {
                    const int j = (8 / C::G) * g + jj;
                    uint32_t v[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) v[c] = POW2 ? (w[c] & (0x01010101u << j)) : ((w[c] >> j) & 0x01010101u);
                    tmem_st8(tmem_a + lane_base + as * C::A_STAGE_COLS + jj * 8, v);
                }
                BGEMM_TIMED(tst, tmem_wait_st());
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(a_full + 8 * as);
                if (h == 0 && tid == 0) BGEMM_STAMP(4);
            }
        }
        if (tid == 0) { BGEMM_PUT(18, tww); BGEMM_PUT(19, twe); BGEMM_PUT(25, clock64() - tloop0); BGEMM_PUT(26, tst); }
        if (tid == 128) { BGEMM_PUT(22, tww); BGEMM_PUT(23, twe); }
        ok = ok && mbar_wait(d_full, 0, abort_flag, p.status, 17);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        if (!ok) *abort_flag = 1;
        if (tid == 0) BGEMM_STAMP(7);
    }

    // ======================================= epilogue ==========================================================
    // Accumulators leave tensor memory as int32 [columns][128] tiles in shared memory (aliasing the operand stages,
    // which are idle by now). With K partitions in a cluster, column c of partition `split` is PUSHED into the
    // shared memory of the CTA that will store it (st.shared::cluster, slot `split`), so that after one cluster
    // barrier every CTA sums its own slots locally. With more partitions than a cluster holds, tiles go through a
    // global workspace and the last CTA to arrive sums them.
    const bool epi_thread = warp < 8;
    int* sP = reinterpret_cast<int*>(sB);
    const int per = p.cluster ? (((NT + p.split_k - 1) / p.split_k + 7) & ~7) : NT;      // columns stored by one CTA
    TileOut tout;
    tout.p = &p; tout.s_alpha = s_alpha; tout.s_colsum = s_colsum;
    tout.batch = batch; tout.m_base = mt * 128; tout.n_base = nt * NT;

    // [M, N] results without K partitions: staged row-major, stored as contiguous runs (see write_tile_rowmajor)
    const bool rowmajor = p.split_k == 1 && p.out_layout == BGEMM_LAYOUT_MN && p.out_kind != kOutActs;
    if (p.cluster) {   // every CTA of the cluster is past its mainloop: peers' operand stages may be overwritten
        __syncwarp();
        cluster_arrive_release();
        cluster_wait_acquire();
        if (tid == 0) BGEMM_STAMP(13);
    }
    if (epi_thread && !*abort_flag) {
        const int set = warp >> 2;
        const int r = (warp & 3) * 32 + lane;
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
        constexpr int HALF = NT / 2;                             // warps 0-3 take the lower half of the columns
        tc_fence_after();
#pragma unroll 1
        for (int n0 = set * HALF; n0 < (set + 1) * HALF; n0 += 8) {
            int acc[8];
            if (POW2) {
                uint32_t t[8][8];
#pragma unroll
                for (int j = 0; j < 8; j++) tmem_ld8(tmem_d + lane_base + j * NT + n0, t[j]);
                tmem_wait_ld();
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    acc[q] = 0;
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[q] += ((int)t[j][q]) >> j;
                }
            } else {
                uint32_t t[8];
                tmem_ld8(tmem_d + lane_base + n0, t);
                tmem_wait_ld();
#pragma unroll
                for (int q = 0; q < 8; q++) acc[q] = (int)t[q];
            }
            if (rowmajor) {
                int4* o = reinterpret_cast<int4*>(sP + r * row_pitch_of(NT) + n0);
                o[0] = make_int4(acc[0], acc[1], acc[2], acc[3]);
                o[1] = make_int4(acc[4], acc[5], acc[6], acc[7]);
            } else if (p.cluster) {
                const int dst = n0 / per;                        // the 8 columns of a chunk share their destination
                const uint32_t remote = mapa_shared(smem_u32(sP + ((split * per + (n0 - dst * per)) * 128 + r)), (uint32_t)dst);
#pragma unroll
                for (int q = 0; q < 8; q++) st_dsmem_s32(remote + (uint32_t)(q * 128 * 4), acc[q]);
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) sP[(n0 + q) * 128 + r] = acc[q];
            }
        }
        tc_fence_before();
    }
    if (tid == 0) BGEMM_STAMP(12);

    if (p.split_k == 1) {
        if (epi_thread) {
            named_bar_sync(1, kUnpackThreads);
            if (!*abort_flag) {
                if (rowmajor) write_tile_rowmajor<NT>(tout, sP, tid, kUnpackThreads);
                else write_tile<false>(tout, sP, 1, 0, 0, NT, tid, kUnpackThreads);
            }
        }
    } else if (p.cluster) {
        __syncwarp();
        cluster_arrive_release();      // the pushes of all peers are visible after this barrier; afterwards
        cluster_wait_acquire();        // nobody touches another CTA's shared memory again
        if (tid == 0) BGEMM_STAMP(14);
        if (epi_thread && !*abort_flag) {
            const int nbeg = min(NT, split * per), ncols = min(NT, nbeg + per) - nbeg;
            write_tile<false>(tout, sP, p.split_k, per * 128, nbeg, ncols, tid, kUnpackThreads);
        }
    } else if (epi_thread) {
        const int tile_id = (batch * p.mtiles + mt) * p.ntiles + nt;
        int* slab = p.ws_partial + ((size_t)tile_id * p.split_k + split) * (NT * 128);
        named_bar_sync(1, kUnpackThreads);
        if (!*abort_flag) {
            for (int i = tid; i < NT * 32; i += kUnpackThreads) reinterpret_cast<int4*>(slab)[i] = reinterpret_cast<const int4*>(sP)[i];
        }
        __threadfence();
        named_bar_sync(1, kUnpackThreads);
        if (tid == 0) {
            const unsigned ticket = atomicAdd(p.ws_counters + tile_id, 1u);
            const int last = (ticket == (unsigned)p.split_k - 1) ? 1 : 0;
            if (last) p.ws_counters[tile_id] = 0;  // leave the counter ready for the next launch
            *last_flag = last;
        }
        named_bar_sync(1, kUnpackThreads);
        if (*last_flag && !*abort_flag) {
            __threadfence();
            write_tile<true>(tout, p.ws_partial + (size_t)tile_id * p.split_k * (NT * 128), p.split_k, NT * 128, 0, NT, tid, kUnpackThreads);
        }
    }
    if (tid == 0) BGEMM_STAMP(8);
    tc_fence_before();
    __syncthreads();
    if (warp == kWarpMma) {
        if (*abort_flag && lane == 0) {   // a wait ran out: let the issued UMMAs finish before the columns are freed
            const long long t0 = clock64();
            while (!mbar_test(d_full, 0) && clock64() - t0 < wait_budget_of(abort_flag)) {}
        }
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
    if (tid == 0) { BGEMM_STAMP(9); BGEMM_STAMP(11); }
}

// ---- host side ----------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int sm_count() {
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cache[dev]) {
        int n = 0;
        cache[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return cache[dev];
}

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

template <int NT, bool POW2, bool DEEP>
static int launch_variant(cudaStream_t stream, const CUtensorMap& tmap, const GemmParams& p, dim3 grid) {
    using C = Cfg<NT, POW2, DEEP>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<NT, POW2, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned na = 0;
    if (p.cluster) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = (unsigned)p.split_k;
        attr[na].val.clusterDim.z = 1;
        na++;
    }
    if (programmatic_launch_enabled()) {
        // The kernel's prologue (barrier set-up, tensor-memory allocation) may start while the previous kernel of
        // the stream drains; it executes griddepcontrol.wait before its first global-memory access.
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = na ? attr : nullptr;
    cfg.numAttrs = na;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_kernel<NT, POW2, DEEP>, tmap, p);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// How many clusters of `split` CTAs of a kernel variant the device holds at once (-1: unknown, e.g. no device). A
// cluster lives inside one GPC, so large clusters leave SMs unused: sixteen clusters of eight do not all fit, and a
// launch that needs them runs in two waves (2048 x 8192 x 128: 18.3 us with 8 K partitions, 10.7 with 6).
template <int NT, bool POW2, bool DEEP>
static int resident_clusters_of(int split) {
    using C = Cfg<NT, POW2, DEEP>;
    if (cudaFuncSetAttribute(gemm_kernel<NT, POW2, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, (unsigned)split, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)split;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_kernel<NT, POW2, DEEP>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return n;
}

int max_resident_clusters(int NT, int split, bool deep) {
    static int cache[64][5][9][2];          // [device][tile width][cluster size][deep]: 0 = not asked yet
    static std::mutex lock;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || split < 2 || split > 8) {
        cudaGetLastError();
        return -1;
    }
    const int w = NT == 16 ? 0 : NT == 32 ? 1 : NT == 64 ? 2 : NT == 128 ? 3 : 4;
    std::lock_guard<std::mutex> g(lock);
    int& c = cache[dev][w][split][deep ? 1 : 0];
    if (c == 0) {
        int n;
        switch (NT) {
            case 16: n = deep ? resident_clusters_of<16, true, true>(split) : resident_clusters_of<16, true, false>(split); break;
            case 32: n = resident_clusters_of<32, true, true>(split); break;
            case 64: n = deep ? resident_clusters_of<64, false, true>(split) : resident_clusters_of<64, false, false>(split); break;
            case 128: n = deep ? resident_clusters_of<128, false, true>(split) : resident_clusters_of<128, false, false>(split); break;
            default: n = resident_clusters_of<256, false, true>(split); break;
        }
        c = n > 0 ? n : -1;
    }
    return c;
}

// Tuning overrides (read once): BGEMM_FORCE_NT = 16|32|64|128|256 forces the tile width, BGEMM_FORCE_DEEP = 0|1 the
// occupancy variant. Unset in normal use.
static int env_int(const char* name) {
    const char* e = std::getenv(name);
    return e ? std::atoi(e) : -1;
}
static int forced_nt() { static const int v = env_int("BGEMM_FORCE_NT"); return v; }
static int forced_deep() { static const int v = env_int("BGEMM_FORCE_DEEP"); return v; }
static int forced_persist() { static const int v = env_int("BGEMM_PERSIST"); return v; }   // 0: never the persistent kernel, 1: whenever it applies
// Fewest K blocks per tile for the persistent kernel (tuning override: BGEMM_PERSIST_MIN_KB).
static int persist_min_kblocks() { static const int v = env_int("BGEMM_PERSIST_MIN_KB"); return v > 0 ? v : 2; }

int gemm_tile_n(long long M, long long N, long long K, long long batch) {
    const int f = forced_nt();
    if (f == 16 || f == 32 || f == 64 || f == 128 || f == 256) return f;
    if (N <= 16) return 16;
    if (N <= 32) return 32;
    if (N <= 64) return 64;
    // 65-256 activation rows on few row tiles: 64-column tiles, all resident at once, with half as many K partitions each
    // are faster than 128-column ones (half the partial sums to exchange per CTA, or none; 4096 x 4096 x 128: 9.35 against
    // 9.87 us, 2048 x 4096 x 128: 7.9 against 9.2, 4096 x 1024 x 256: 6.75 against 8.5, 1024 x 4096 x 256: 7.8 against 9.2;
    // level at 4096 x 4096 x 256) as long as the K range per partition stays short (4096 x 8192 x 128: 12.5 against 11.7).
    if (N <= 256 && batch == 1 && (M + 127) / 128 * ((N + 63) / 64) <= sm_count() && (K + 255) / 256 <= 16) return 64;
    // 128-wide tiles with two CTAs per SM and two UMMA issuers measured faster than 256-wide ones at every N
    // (686 vs 733 us at 28672 x 8192 x 4096); the 256-wide variant stays available through BGEMM_FORCE_NT.
    return 128;
}

int launch_gemm(cudaStream_t stream, GemmParams p, const int8_t* acts, long long act_ld, long long batch) {
    // Up to 16 activation rows: pure weight streaming (no tensor-memory set-up, no 128-row tile, no cluster reduction).
    // A single row of ternary activations goes to the CUDA-core popcount kernel (28672 x 8192: 10.2 us against 11.6),
    // everything else to the register-fed mma.sync kernel (N = 2 / 4 / 8 / 16: 11.7 / 11.8 / 12.1 / 17.5 us against
    // 12.3 / 15.3 / 19.8 / 19.9 for the kernels behind it), which falls back to the former where it does not apply.
    // BGEMM_STREAM_MIN_N / BGEMM_STREAM_MAX_N / BGEMM_SKINNY_MAX_N move the limits.
    const bool single_ternary_row = p.N == 1 && p.epi && !p.acts_general && stream_min_n() <= 1;
    if (single_ternary_row && skinny_supported(p, batch, true)) return launch_gemm_skinny(stream, p, acts, act_ld, batch);
    if (stream_supported(p, batch)) return launch_gemm_stream(stream, p, acts, act_ld, batch, p.weights_static != 0);
    if (skinny_supported(p, batch, !p.acts_general)) return launch_gemm_skinny(stream, p, acts, act_ld, batch);
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return BGEMM_ERR_DRIVER;
    int NT = gemm_tile_n(p.M, p.N, p.K, batch);
    // One partial wave: with 128-wide tiles on more than one but at most two CTAs per SM, some SMs run two tiles side by
    // side while the others run one, and the launch lasts as long as the pairs (3584 x 8192 x 1024, the 8-GPU shard of the
    // 28672-row layer: 32.5 us); 256-wide tiles, one CTA per SM, finish sooner when they all fit at once (28.9 us).
    if (NT == 128 && p.split_k == 1 && batch == 1 && forced_nt() < 0) {
        const long long t128 = (long long)p.mtiles * ((p.N + 127) / 128), t256 = (long long)p.mtiles * ((p.N + 255) / 256);
        if (t128 > sm_count() && t128 <= 2LL * sm_count() && t256 <= sm_count() && p.N % 256 == 0) NT = 256;
    }
    // 17-32 activation rows on more row tiles than SMs: the 32-column variant always takes a whole SM per CTA and would
    // run in several waves; 64-column tiles, two CTAs per SM (or the persistent kernel), are faster although half of their
    // columns are padding (28672 x 8192 x 32: 25.4 against 32.9 us; 28672 x 1024 x 32: 7.6 against 12.1). In one wave
    // the 32-column variant stays 3-6 % ahead.
    if (NT == 32 && p.split_k == 1 && (long long)p.mtiles * batch > sm_count() && forced_nt() < 0) NT = 64;
    // Wide activation matrices: 256 x 256 tiles on CTA pairs (each CTA loads boxes of 128 activation rows).
    const bool pair = pair_supported(p, batch);
    if (pair) NT = 256;
    p.ntiles = (int)((p.N + NT - 1) / NT);

    CUtensorMap tmap;
    cuuint64_t dims[3] = {(cuuint64_t)act_ld, (cuuint64_t)p.N, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)act_ld, (cuuint64_t)act_ld * (cuuint64_t)p.N};
    cuuint32_t box[3] = {128u, (cuuint32_t)(pair ? 128 : NT), 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(acts), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return BGEMM_ERR_DRIVER;
    if (pair) return launch_gemm_pair(stream, &tmap, p, batch);

    // A pool of narrow problems (one tile across N, many more tiles than SMs, no K partitioning): one persistent CTA
    // per SM walks over the tiles and overlaps every tile's epilogue with the next tile's mainloop (measured 2.46 vs
    // 2.27 POP/s on 95 x [4096 x 4096 x 128]). The tile-per-CTA kernel keeps the launches whose tiles are all resident
    // at once at two CTAs per SM: there the persistent kernel runs two tiles in a row on some SMs and one on the others
    // (28672 x 8192, 224 tiles: N = 128 33.0 against 34.2 us, N = 64 26.1 against 29.0).
    // With several tiles across N the persistent kernel is ahead at 12-16 K blocks per tile (16384 x 4096 x 512: 34.1
    // against 36.9 us; 16 x [4096 x 4096 x 256]: 57 against 64), level or slightly behind at 32 (28672 x 8192 x 256: 58.7
    // against 57.0) and behind with short K (8192 x 2048 x 1024: 27.8 against 25.0).
    const long long total_tiles = (long long)p.ntiles * p.mtiles * batch;
    const bool many_tiles = total_tiles > 2LL * sm_count();
    const int persist = forced_persist() >= 0 ? forced_persist()
                                              : (many_tiles && (p.ntiles == 1 || (p.kblocks >= 12 && p.kblocks < 32)) ? 1 : 0);
    if (persist && p.split_k == 1 && persistent_supported(NT) && total_tiles > sm_count() && p.kblocks >= persist_min_kblocks() &&
        persistent_kblocks_ok(NT, p.kblocks))
        return launch_gemm_persistent(stream, &tmap, p, NT, total_tiles, sm_count());

    dim3 grid((unsigned)p.ntiles, (unsigned)(p.mtiles * p.split_k), (unsigned)batch);
    // At most one CTA per SM in the whole launch: give each CTA the full tensor memory and a deeper pipeline.
    const bool deep = forced_deep() >= 0 ? forced_deep() != 0 : (long long)grid.x * grid.y * grid.z <= sm_count();
    switch (NT) {
        case 16: return deep ? launch_variant<16, true, true>(stream, tmap, p, grid) : launch_variant<16, true, false>(stream, tmap, p, grid);
        case 32: return launch_variant<32, true, true>(stream, tmap, p, grid);
        case 64: return deep ? launch_variant<64, false, true>(stream, tmap, p, grid) : launch_variant<64, false, false>(stream, tmap, p, grid);
        case 128: return deep ? launch_variant<128, false, true>(stream, tmap, p, grid) : launch_variant<128, false, false>(stream, tmap, p, grid);
        default: return launch_variant<256, false, true>(stream, tmap, p, grid);
    }
}

}  // namespace bgemm
