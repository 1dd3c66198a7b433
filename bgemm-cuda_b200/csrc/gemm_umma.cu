// Binary-weight GEMM mainloop for sm_100a: packed 1-bit weights are unpacked on chip to u8 and fed to
// tcgen05.mma kind::i8 as the A operand straight from tensor memory; int8 activations arrive by TMA.
//
// Replaces PACK_BGEMM_Kernel (lowbit_kernel/csrc/include/kernel_matmul.cuh:370-547) and the separate
// SplitK_Reduction launch (kernel_reduction.cuh:29-48) of the reference. The legacy b1 mma.sync path
// the reference uses runs at ~0.4 POP/s on B200 (measured), an order of magnitude below kind::i8.
//
// One CTA computes a 128(M) x NT(N) tile over a K range [kb0, kb1) of 256-column blocks.
//   warps 0-3  unpack: thread r owns weight row r of the tile; per K block it reads its 32 packed bytes
//              from shared memory, expands them to 8 x (128 x 32) u8 operand slices with one or two
//              logic ops per 4 elements, and writes them to tensor memory (tcgen05.st). Afterwards the
//              same warps run the epilogue (tcgen05.ld, split-K reduction, scale, store).
//   warp 4     allocates tensor memory; one lane issues 8 UMMAs (128 x NT x 32) per K block.
//   warp 5     one lane streams the packed weight tiles (4 KB each, contiguous) with cp.async.bulk.
//   warp 6     one lane loads the activation tiles [NT x 256 B] with two 128B-swizzled TMA boxes.
//
// POW2 variant (NT <= 32, weight-streaming shapes): slice j keeps the weight bit at byte value 2^j
// (a single AND per 4 elements) and accumulates into its own accumulator D_j; the epilogue adds
// D_j >> j. The plain variant shifts the bit down to {0,1} and uses one accumulator.
//
// With D = sum_k bit_w(k) * x(k):  XOR / BWTA results are colsum_x[n] - 2 D, AND / ATTN results are D.
#include <cuda_fp16.h>

#include "internal.h"
#include "ptx.cuh"

namespace bgemm {

constexpr int kUnpackThreads = 128;
constexpr int kGemmThreads = 224;

__host__ __device__ constexpr int pow2_ceil(int v) {
    int p = 32;
    while (p < v) p <<= 1;
    return p;
}

template <int NT, bool POW2>
struct Cfg {
    static constexpr int D_COLS = POW2 ? 8 * NT : NT;
    static constexpr int A_STAGES = POW2 ? (NT == 16 ? 2 : 4) : (NT == 64 ? 3 : (NT == 128 ? 2 : 4));
    static constexpr int A_COL0 = D_COLS;
    static constexpr int TMEM_COLS = pow2_ceil(D_COLS + 64 * A_STAGES);
    static constexpr int B_STAGE_BYTES = NT * 256;
    static constexpr int B_STAGES = NT <= 32 ? 4 : 3;
    static constexpr int W_STAGES = NT <= 32 ? 6 : (NT == 128 ? 3 : 4);
    static constexpr int NBARS = 2 * W_STAGES + 2 * B_STAGES + 2 * A_STAGES + 1;
    static constexpr int SMEM_USED = B_STAGES * B_STAGE_BYTES + W_STAGES * 4096 + 1024 /*barriers, flags*/ + 1024 /*align*/;
    // Co-resident CTAs must not ask for more tensor memory than the SM has (a later tcgen05.alloc would
    // stall until an earlier CTA exits): request enough shared memory to cap residency at 512 / TMEM_COLS.
    static constexpr int SMEM_FLOOR = TMEM_COLS == 512 ? 117 * 1024 : 77 * 1024;
    static constexpr int SMEM_BYTES = SMEM_USED > SMEM_FLOOR ? SMEM_USED : SMEM_FLOOR;
    static_assert(TMEM_COLS <= 512, "tensor memory budget");
    static_assert(NT % 16 == 0 && NT >= 16 && NT <= 256, "UMMA N");
};

__device__ __forceinline__ void store_result(const GemmParams& p, int batch, int m, int n, int acc) {
    if (m >= p.M || n >= p.N) return;
    const int val = p.epi ? (__ldg(p.colsum + (size_t)batch * p.N + n) - 2 * acc) : acc;
    const size_t idx = (size_t)batch * p.M * p.N + (p.out_layout == BGEMM_LAYOUT_NM ? (size_t)n * p.M + m : (size_t)m * p.N + n);
    if (p.out_kind == BGEMM_OUT_I32) {
        reinterpret_cast<int*>(p.out)[idx] = val;
    } else if (p.out_kind == BGEMM_OUT_F16) {
        reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn((float)val);
    } else {
        const float a = __half2float(p.alpha[(size_t)batch * p.M + m]);
        reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn((float)val * a);
    }
}

template <int NT, bool POW2>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_kernel(const __grid_constant__ CUtensorMap tmap_acts, const GemmParams p) {
    using C = Cfg<NT, POW2>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sB = smem;
    uint8_t* sW = sB + C::B_STAGES * C::B_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sW + C::W_STAGES * 4096);
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + C::NBARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    int* last_flag = reinterpret_cast<int*>(tmem_holder + 2);

    const uint32_t w_full = smem_u32(bars);
    const uint32_t w_empty = w_full + 8 * C::W_STAGES;
    const uint32_t b_full = w_empty + 8 * C::W_STAGES;
    const uint32_t b_empty = b_full + 8 * C::B_STAGES;
    const uint32_t a_full = b_empty + 8 * C::B_STAGES;
    const uint32_t a_empty = a_full + 8 * C::A_STAGES;
    const uint32_t d_full = a_empty + 8 * C::A_STAGES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nt = blockIdx.x;
    const int split = blockIdx.y % p.split_k;
    const int mt = blockIdx.y / p.split_k;
    const int batch = blockIdx.z;
    const int kb0 = (int)(((long long)p.kblocks * split) / p.split_k);
    const int kb1 = (int)(((long long)p.kblocks * (split + 1)) / p.split_k);
    const int nkb = kb1 - kb0;

    if (tid == 0) {
        for (int i = 0; i < C::W_STAGES; i++) { mbar_init(w_full + 8 * i, 1); mbar_init(w_empty + 8 * i, 4); }
        for (int i = 0; i < C::B_STAGES; i++) { mbar_init(b_full + 8 * i, 1); mbar_init(b_empty + 8 * i, 1); }
        for (int i = 0; i < C::A_STAGES; i++) { mbar_init(a_full + 8 * i, 4); mbar_init(a_empty + 8 * i, 1); }
        mbar_init(d_full, 1);
        *abort_flag = 0;
        *last_flag = 0;
        mbar_fence_init();
    }
    if (warp == 6 && lane == 0) tma_prefetch_desc(&tmap_acts);
    if (warp == 4) tmem_alloc(smem_u32(tmem_holder), C::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_holder;
    const uint32_t tmem_d = tmem;
    const uint32_t tmem_a = tmem + C::A_COL0;

    if (warp == 5) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            const uint8_t* src = p.plane + (size_t)batch * p.plane_batch_bytes + ((size_t)mt * p.kblocks + kb0) * 4096;
            int issued = 0;
            for (int i = 0; i < nkb; i++) {
                const int s = i % C::W_STAGES;
                if (i >= C::W_STAGES && !mbar_wait(w_empty + 8 * s, ((i / C::W_STAGES) - 1) & 1, abort_flag, p.status, 11)) break;
                mbar_arrive_expect_tx(w_full + 8 * s, 4096);
                bulk_g2s(smem_u32(sW + s * 4096), src + (size_t)i * 4096, 4096, w_full + 8 * s);
                issued = i + 1;
            }
            if (*abort_flag) {  // drain own copies before the CTA may exit
                for (int i = issued - 1; i >= 0 && i >= issued - C::W_STAGES; i--) {
                    const long long t0 = clock64();
                    while (!mbar_test(w_full + 8 * (i % C::W_STAGES), (i / C::W_STAGES) & 1) && clock64() - t0 < kWaitBudgetClocks) {}
                }
            }
        }
    } else if (warp == 6) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < nkb; i++) {
                const int s = i % C::B_STAGES;
                if (i >= C::B_STAGES && !mbar_wait(b_empty + 8 * s, ((i / C::B_STAGES) - 1) & 1, abort_flag, p.status, 12)) break;
                mbar_arrive_expect_tx(b_full + 8 * s, C::B_STAGE_BYTES);
                const uint32_t dst = smem_u32(sB + s * C::B_STAGE_BYTES);
                tma_load_3d(dst, &tmap_acts, (kb0 + i) * 256, nt * NT, batch, b_full + 8 * s);
                tma_load_3d(dst + NT * 128, &tmap_acts, (kb0 + i) * 256 + 128, nt * NT, batch, b_full + 8 * s);
                issued = i + 1;
            }
            if (*abort_flag) {
                for (int i = issued - 1; i >= 0 && i >= issued - C::B_STAGES; i--) {
                    const long long t0 = clock64();
                    while (!mbar_test(b_full + 8 * (i % C::B_STAGES), (i / C::B_STAGES) & 1) && clock64() - t0 < kWaitBudgetClocks) {}
                }
            }
        }
    } else if (warp == 4) {
        // ---------------- UMMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_u8s8(NT);
            bool ok = true;
            for (int i = 0; i < nkb && ok; i++) {
                const int as = i % C::A_STAGES, bs = i % C::B_STAGES;
                ok = mbar_wait(a_full + 8 * as, (i / C::A_STAGES) & 1, abort_flag, p.status, 13) &&
                     mbar_wait(b_full + 8 * bs, (i / C::B_STAGES) & 1, abort_flag, p.status, 14);
                if (!ok) break;
                tc_fence_after();
                const uint32_t bbase = smem_u32(sB + bs * C::B_STAGE_BYTES);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const uint64_t bdesc = umma_desc_sw128(bbase + (j >> 2) * (NT * 128) + (j & 3) * 32);
                    const uint32_t d = tmem_d + (POW2 ? j * NT : 0);
                    const uint32_t acc = POW2 ? (i > 0 ? 1u : 0u) : ((i | j) ? 1u : 0u);
                    umma_i8_ts(d, tmem_a + as * 64 + j * 8, bdesc, idesc, acc);
                }
                umma_commit(a_empty + 8 * as);
                umma_commit(b_empty + 8 * bs);
            }
            umma_commit(d_full);
        }
    } else {
        // ---------------- unpack (warps 0-3), then epilogue ----------------
        const int r = tid;  // weight row of the tile == tensor-memory lane
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        bool ok = true;
        for (int i = 0; i < nkb && ok; i++) {
            const int ws = i % C::W_STAGES, as = i % C::A_STAGES;
            ok = mbar_wait(w_full + 8 * ws, (i / C::W_STAGES) & 1, abort_flag, p.status, 15);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const uint4 lo = *reinterpret_cast<const uint4*>(sW + ws * 4096 + r * 16);
            const uint4 hi = *reinterpret_cast<const uint4*>(sW + ws * 4096 + 2048 + r * 16);
            __syncwarp();
            if (lane == 0) mbar_arrive(w_empty + 8 * ws);
            if (i >= C::A_STAGES) ok = mbar_wait(a_empty + 8 * as, ((i / C::A_STAGES) - 1) & 1, abort_flag, p.status, 16);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                uint32_t v[8];
#pragma unroll
                for (int c = 0; c < 8; c++) v[c] = POW2 ? (w[c] & (0x01010101u << j)) : ((w[c] >> j) & 0x01010101u);
                tmem_st8(tmem_a + lane_base + as * 64 + j * 8, v);
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full + 8 * as);
        }

        // ---- epilogue ----
        ok = ok && mbar_wait(d_full, 0, abort_flag, p.status, 17);
        ok = __all_sync(0xffffffffu, ok);
        tc_fence_after();
        const int m = mt * 128 + r;
        const int tile_id = (batch * p.mtiles + mt) * p.ntiles + nt;
        int* slab = p.ws_partial ? p.ws_partial + ((size_t)tile_id * p.split_k + split) * (NT * 128) : nullptr;
        if (ok) {
            constexpr int CH = 8;
#pragma unroll 1
            for (int n0 = 0; n0 < NT; n0 += CH) {
                int acc[CH];
                if (POW2) {
#pragma unroll
                    for (int q = 0; q < CH; q++) acc[q] = 0;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        uint32_t t[8];
                        tmem_ld8(tmem_d + lane_base + j * NT + n0, t);
                        tmem_wait_ld();
#pragma unroll
                        for (int q = 0; q < CH; q++) acc[q] += ((int)t[q]) >> j;
                    }
                } else {
                    uint32_t t[8];
                    tmem_ld8(tmem_d + lane_base + n0, t);
                    tmem_wait_ld();
#pragma unroll
                    for (int q = 0; q < CH; q++) acc[q] = (int)t[q];
                }
                if (p.split_k == 1) {
#pragma unroll
                    for (int q = 0; q < CH; q++) store_result(p, batch, m, nt * NT + n0 + q, acc[q]);
                } else {
#pragma unroll
                    for (int q = 0; q < CH; q++) slab[(n0 + q) * 128 + r] = acc[q];
                }
            }
        }
        if (p.split_k > 1) {
            // The last CTA of this tile to arrive sums every partial slab and stores the result.
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
                const int* base = p.ws_partial + (size_t)tile_id * p.split_k * (NT * 128);
#pragma unroll 1
                for (int n = 0; n < NT; n++) {
                    int acc = 0;
                    for (int s = 0; s < p.split_k; s++) acc += __ldcg(base + (size_t)s * (NT * 128) + n * 128 + r);
                    store_result(p, batch, m, nt * NT + n, acc);
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, C::TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

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

template <int NT, bool POW2>
static int launch_variant(cudaStream_t stream, const CUtensorMap& tmap, const GemmParams& p, dim3 grid) {
    using C = Cfg<NT, POW2>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<NT, POW2>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    gemm_kernel<NT, POW2><<<grid, kGemmThreads, C::SMEM_BYTES, stream>>>(tmap, p);
    count_launch();
    return (int)cudaGetLastError();
}

int gemm_tile_n(long long N) {
    if (N <= 16) return 16;
    if (N <= 32) return 32;
    if (N <= 64) return 64;
    if (N <= 128) return 128;
    // widest tile unless it would leave most of a tile empty
    return (N % 256 == 0 || N > 1024) ? 256 : 128;
}

int launch_gemm(cudaStream_t stream, GemmParams p, const int8_t* acts, long long act_ld, long long batch) {
    EncodeTiledFn encode = get_encode_fn();
    if (!encode) return BGEMM_ERR_DRIVER;
    const int NT = gemm_tile_n(p.N);
    p.ntiles = (int)((p.N + NT - 1) / NT);

    CUtensorMap tmap;
    cuuint64_t dims[3] = {(cuuint64_t)act_ld, (cuuint64_t)p.N, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)act_ld, (cuuint64_t)act_ld * (cuuint64_t)p.N};
    cuuint32_t box[3] = {128u, (cuuint32_t)NT, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(acts), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return BGEMM_ERR_DRIVER;

    dim3 grid((unsigned)p.ntiles, (unsigned)(p.mtiles * p.split_k), (unsigned)batch);
    switch (NT) {
        case 16: return launch_variant<16, true>(stream, tmap, p, grid);
        case 32: return launch_variant<32, true>(stream, tmap, p, grid);
        case 64: return launch_variant<64, false>(stream, tmap, p, grid);
        case 128: return launch_variant<128, false>(stream, tmap, p, grid);
        default: return launch_variant<256, false>(stream, tmap, p, grid);
    }
}

}  // namespace bgemm
