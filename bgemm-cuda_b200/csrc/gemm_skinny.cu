// Weight-streaming kernel for very few activation rows (built for N <= 8, dispatched for N <= 4: single-token and
// small-batch decode shapes).
// At N <= 8 the product is pure HBM streaming of the packed weight plane (one bit per weight), and the tensor-core
// path pays for a 16-column UMMA tile, tensor-memory set-up and a cluster reduction that together cost several
// times the streaming time (28672 x 8192: 24 us against 4.5 us of HBM time). This kernel keeps the work on the
// CUDA cores, where it is cheap enough to hide behind the loads. A lane owns one weight row and fetches its 32 packed
// bytes of a 256-column K block with two coalesced 16-byte asynchronous copies (the tiled plane keeps 128 rows x 16 B
// contiguous) into a ring in shared memory that only this lane reads back: up to 192 KB per SM (12 K blocks per lane
// with 16 warps, 6 with 32) are in flight from the first instruction on, and cp.async group counting is all the
// synchronisation it needs.
//
//   popc path   activations in {-1, 0, +1} and a result of the form colsum - 2 D (ops XOR and BWTA): the CTA first
//               turns the int8 activations into two bit planes in the weight plane's own bit order (non-zero, negative);
//               then  sum_k sign(w) x = popc(nz) - 2 popc(nz & (w ^ neg)),  one LOP3 + POPC + add per 32 weights.
//   dp4a path   any int8 activations, any op: bit j of every byte is isolated with one AND (byte value 0 or 2^j) and four
//               weights meet four activations in one dp4a (u8 x s8 -> s32) into accumulator j; the end adds acc_j >> j.
//
// Which path runs is decided in the kernel, from the activations themselves (every CTA scans them while it stages
// them), so a result never depends on what the caller promised. Both are int32-exact and bit-identical to the
// tensor-core kernels. The dp4a path is ALU-bound (8 dp4a per 32 weights and activation row) and only pays for
// N <= 2; the dispatcher therefore sends N = 3..8 here only for ops whose activations are ternary by contract.
//
// Replaces the same reference functions as gemm_umma.cu (PACK_BGEMM_Kernel, kernel_matmul.cuh:370-547, which does
// not accept N < 32 at all) for the shapes named above.
//
// One CTA of 16 or 32 warps per SM walks over a contiguous range of 32-row groups, so the activations are turned into
// planes once per CTA; `ks` warps share the K blocks of a group and meet in shared memory.
#include <cuda_fp16.h>

#include <cstdlib>

#include "internal.h"
#include "ptx.cuh"

namespace bgemm {

constexpr int kSkinnyMaxSmem = 224 * 1024;

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// One K block of one weight row against NN activation rows, dp4a path. `w` = the row's 32 packed bytes; bit (8 b + j)
// of word c is the weight of column 32 j + 4 c + b of the block, so the four bytes of (w[c] & (0x01010101 << j)) line
// up with the four int8 activations at byte offset 32 j + 4 c. `x_block` may be shared or global memory.
template <int NN>
__device__ __forceinline__ void skinny_block_dp4a(const uint4& lo, const uint4& hi, const int8_t* x_block, long long x_pitch, int (&acc)[NN][8]) {
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int j = 0; j < 8; j++) {
        uint32_t a[8];
#pragma unroll
        for (int c = 0; c < 8; c++) a[c] = w[c] & (0x01010101u << j);
#pragma unroll
        for (int n = 0; n < NN; n++) {
            const uint4 x0 = *reinterpret_cast<const uint4*>(x_block + (size_t)n * x_pitch + 32 * j);
            const uint4 x1 = *reinterpret_cast<const uint4*>(x_block + (size_t)n * x_pitch + 32 * j + 16);
            int s = acc[n][j];
            s = dp4a_u8s8(a[0], x0.x, s); s = dp4a_u8s8(a[1], x0.y, s); s = dp4a_u8s8(a[2], x0.z, s); s = dp4a_u8s8(a[3], x0.w, s);
            s = dp4a_u8s8(a[4], x1.x, s); s = dp4a_u8s8(a[5], x1.y, s); s = dp4a_u8s8(a[6], x1.z, s); s = dp4a_u8s8(a[7], x1.w, s);
            acc[n][j] = s;
        }
    }
}

// Carry-save adder over bit columns: a + b + c = 2 h + l in every bit position.
__device__ __forceinline__ void skinny_csa(uint32_t& h, uint32_t& l, uint32_t a, uint32_t b, uint32_t c) {
    const uint32_t u = a ^ b;
    h = (a & b) | (u & c);
    l = u ^ c;
}
// Running count of set bits kept bit-sliced (ones, twos, fours) so that a K block of eight words costs one POPC (of
// the eights that fall out) instead of eight: POPC runs at a quarter of the logic rate and bounded the kernel.
struct SkinnyCount {
    uint32_t ones, twos, fours;
    int eights;
    __device__ __forceinline__ void reset() { ones = twos = fours = 0u; eights = 0; }
    __device__ __forceinline__ int total() const { return 8 * eights + 4 * __popc(fours) + 2 * __popc(twos) + __popc(ones); }
};

// The same K block on the popc path. `planes` = this block's [NN][16] words in shared memory: 8 non-zero words, then
// 8 negative words, bit for bit in the order of the weight words. cnt[n] counts the products that are -1.
template <int NN>
__device__ __forceinline__ void skinny_block_popc(const uint4& lo, const uint4& hi, const uint32_t* planes, int plane_pitch, SkinnyCount (&cnt)[NN]) {
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int n = 0; n < NN; n++) {
        const uint4* q = reinterpret_cast<const uint4*>(planes + (size_t)n * plane_pitch);
        const uint4 z0 = q[0], z1 = q[1], g0 = q[2], g1 = q[3];
        const uint32_t nz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
        const uint32_t ng[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        uint32_t t[8];
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = (w[i] ^ ng[i]) & nz[i];
        SkinnyCount& s = cnt[n];
        // 8 new words + the running ones -> ones, and carries up the levels; only one adder per level depends on
        // the running state, the rest of the tree is independent work
        uint32_t c1, c2, c3, c4, l1, l2, l3, f1, f2, m1, e;
        skinny_csa(c1, l1, t[0], t[1], t[2]);
        skinny_csa(c2, l2, t[3], t[4], t[5]);
        skinny_csa(c3, l3, l1, l2, t[6]);
        skinny_csa(c4, s.ones, s.ones, l3, t[7]);
        skinny_csa(f1, m1, c1, c2, c3);
        skinny_csa(f2, s.twos, s.twos, m1, c4);
        skinny_csa(e, s.fours, s.fours, f1, f2);
        s.eights += __popc(e);
    }
}

// Four int8 activations of one row at column k (a multiple of 4); columns from K on read as zero.
__device__ __forceinline__ uint32_t skinny_x4(const int8_t* row, int k, int K) {
    if (k >= K) return 0u;
    uint32_t v = *reinterpret_cast<const uint32_t*>(row + k);
    if (k + 4 > K) v &= 0xffffffffu >> (8 * (k + 4 - K));
    return v;
}
__device__ __forceinline__ bool skinny_is_ternary(uint32_t x4) {      // every byte in {0xff, 0x00, 0x01}
    return __vcmpgtu4(__vadd4(x4, 0x01010101u), 0x02020202u) == 0u;
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kSkinnyMaxWarps = 32;            // CTAs have 16 or 32 warps = (groups in flight) x (K shares)                // 16 warps = (groups in flight) x (K shares)
constexpr int kSkinnyPiece = 8 * 1024;             // columns staged per pass and row by the N > 2 variants

// `ks` warps share the K blocks of one 32-row group (ks a power of two up to W); the CTA works on W / ks groups at a
// time and owns the contiguous range of groups [groups * b / gridDim.x, groups * (b + 1) / gridDim.x).
template <int NN, int D, int W>
__global__ void __launch_bounds__(32 * W) gemm_skinny_kernel(const GemmParams p, const int8_t* __restrict__ acts, long long act_ld,
                                                                     int groups, int ks, int weights_static) {
    constexpr int T = 32 * W;                    // threads of the CTA
    constexpr bool STAGE = NN <= 2;              // whole int8 activations stay in shared memory (they feed the dp4a path)
    grid_launch_dependents();
    extern __shared__ __align__(16) uint8_t skinny_smem[];
    const int x_pitch = p.kblocks * 256;                                    // == act_ld
    uint32_t* planes = reinterpret_cast<uint32_t*>(skinny_smem);            // [kblocks][NN][8 nz + 8 neg]
    int* red = reinterpret_cast<int*>(planes + (size_t)p.kblocks * NN * 16); // [warps][NN][32]
    int* s_pn = red + W * NN * 32;                                         // [8] non-zero activations per row
    int8_t* sx = reinterpret_cast<int8_t*>(s_pn + 8);                       // [NN][x_pitch] (STAGE) or [NN][piece]
    const int piece = STAGE ? x_pitch : (x_pitch < kSkinnyPiece ? x_pitch : kSkinnyPiece);   // columns staged per pass, all rows at once
    // Weight ring: D slots of 32 bytes per lane, [slot][lo | hi][thread]. A lane only ever reads what it copied itself,
    // so cp.async group accounting is all the synchronisation the ring needs.
    uint4* ring = reinterpret_cast<uint4*>(sx + (size_t)NN * piece);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int batch = blockIdx.y;
    const int gs = W / ks;            // groups in flight
    const int team = warp / ks, share = warp - team * ks;
    const int kb0 = (int)(((long long)p.kblocks * share) / ks);
    const int kb1 = (int)(((long long)p.kblocks * (share + 1)) / ks);
    const int g_begin = (int)(((long long)groups * blockIdx.x) / gridDim.x);
    const int g_end = (int)(((long long)groups * (blockIdx.x + 1)) / gridDim.x);
    if (tid < 8) s_pn[tid] = 0;
    const int8_t* src = acts + (size_t)batch * p.N * act_ld;
    const uint8_t* plane = p.plane + (size_t)batch * p.plane_batch_bytes;

    // The warp's work is a sequence of units (group, K block). D of them are in flight per lane at any time, as
    // 16-byte asynchronous copies into the lane's ring slots: with D = 12 that is 192 KB per SM, the SM's whole share
    // of a 28672 x 8192 plane, so the loads of a launch all leave at its start.
    auto advance = [&](int& g, int& kb) {
        if (++kb >= kb1) { kb = kb0; g += gs; }
    };
    // Address of this lane's 16 bytes ("lo" half; "hi" is 2048 further) of unit (g, kb). The loop below keeps a running
    // pointer instead (next K block: + 4096) and only comes back here when the group changes.
    auto unit_ptr = [&](int g, int kb) {
        return plane + ((size_t)(g >> 2) * p.kblocks + kb) * 4096 + (size_t)((g & 3) * 32 + lane) * 16;
    };
    constexpr uint32_t kSlotBytes = 2u * T * 16u;
    const uint32_t ring_addr = smem_u32(ring + tid);
    auto issue = [&](int slot, bool live, const uint8_t* w) {   // always closes a group: one group per unit
        if (live) {
            cp_async16(ring_addr + slot * kSlotBytes, w);
            cp_async16(ring_addr + slot * kSlotBytes + kSlotBytes / 2, w + 2048);
        }
        cp_async_commit();
    };
    int gc = g_begin + team, kc = kb0;           // unit being computed
    int gl = gc, kl = kc;                        // next unit to load
    const uint8_t* wl = unit_ptr(gl, kl);        // where unit (gl, kl) lives
    auto next_load = [&]() {                     // (gl, kl, wl) -> the following unit
        wl += 4096;
        if (++kl >= kb1) { kl = kb0; gl += gs; wl = unit_ptr(gl, kl); }
    };
    // With the caller's promise that the plane was complete before the previous kernel of the stream was launched
    // (bgemm_gemm_static_weights) the ring is filled ahead of the dependency wait, i.e. while that kernel still runs.
    if (weights_static) {
#pragma unroll 1
        for (int d = 0; d < D; d++) { issue(d, gl < g_end, wl); next_load(); }
    }
    grid_dependency_wait();
    // The (small) activation loads go first: issued behind two thirds of the weight traffic they would come back last
    // and hold up the whole CTA.
    auto load_x = [&](int i, int base, int chunks) {
        const int n = i / chunks, k0 = base + (i - n * chunks) * 16;
        return (n < p.N && k0 < p.K) ? *reinterpret_cast<const uint4*>(src + (size_t)n * act_ld + k0) : make_uint4(0u, 0u, 0u, 0u);
    };
    constexpr int XR = NN;                       // activation chunks per thread fetched ahead (covers K <= 8192)
    uint4 xv[XR];
#pragma unroll
    for (int r = 0; r < XR; r++) {
        const int i = tid + r * T;
        xv[r] = i < NN * (piece / 16) ? load_x(i, 0, piece / 16) : make_uint4(0u, 0u, 0u, 0u);
    }
    if (!weights_static) {
#pragma unroll 1
        for (int d = 0; d < D; d++) { issue(d, gl < g_end, wl); next_load(); }
    }

    // ---- activations: int8 -> shared memory piece by piece (coalesced), checked for values outside {-1, 0, +1}, and
    //      turned into bit planes in the weight plane's bit order. Rows beyond N and columns beyond K become zero.
    bool tern = true;
    {
        int nonzero[NN];
#pragma unroll
        for (int n = 0; n < NN; n++) nonzero[n] = 0;
        for (int base = 0; base < x_pitch; base += piece) {
            const int len = x_pitch - base < piece ? x_pitch - base : piece;
            const int chunks = len / 16;
            auto put_x = [&](int i, uint4 v) {
                const int n = i / chunks, k0 = base + (i - n * chunks) * 16;
                if (k0 + 16 > p.K) {                                            // columns from K on read as zero
                    uint32_t* q = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                    for (int b = 0; b < 16; b++)
                        if (k0 + b >= p.K) q[b >> 2] &= ~(0xffu << (8 * (b & 3)));
                }
                tern = tern && skinny_is_ternary(v.x) && skinny_is_ternary(v.y) && skinny_is_ternary(v.z) && skinny_is_ternary(v.w);
                *reinterpret_cast<uint4*>(sx + (size_t)n * piece + (k0 - base)) = v;
            };
            int i = tid;
            if (base == 0) {                                                    // fetched ahead
#pragma unroll
                for (int r = 0; r < XR; r++, i += T)
                    if (i < NN * chunks) put_x(i, xv[r]);
            }
            for (; i < NN * chunks; i += T) put_x(i, load_x(i, base, chunks));
            __syncthreads();
            const int words = len / 32;                                         // items per row: word c of K block kb, both planes
#pragma unroll
            for (int n = 0; n < NN; n++) {
                for (int i = tid; i < words; i += T) {
                    const int c = i & 7, kbl = i >> 3, kb = base / 256 + kbl;
                    uint32_t nzw = 0u, ngw = 0u;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const uint32_t x4 = *reinterpret_cast<const uint32_t*>(sx + (size_t)n * piece + kbl * 256 + 32 * j + 4 * c);
                        nzw |= (__vcmpne4(x4, 0u) & 0x01010101u) << j;
                        ngw |= ((x4 >> 7) & 0x01010101u) << j;
                    }
                    planes[((size_t)kb * NN + n) * 16 + c] = nzw;
                    planes[((size_t)kb * NN + n) * 16 + 8 + c] = ngw;
                    nonzero[n] += __popc(nzw);
                }
            }
            if (!STAGE) __syncthreads();                                        // the staging buffer is reused
        }
#pragma unroll
        for (int n = 0; n < NN; n++) {
            const int t = __reduce_add_sync(0xffffffffu, nonzero[n]);
            if (lane == 0 && t) atomicAdd(&s_pn[n], t);
        }
    }
    const bool popc_path = __syncthreads_and(tern) != 0 && p.epi != 0;

    // Sums of the team's K shares meet in shared memory; the team's threads then convert and store 32 rows x N results.
    auto reduce_store = [&](int g) {
        const int mt = g >> 2, quarter = g & 3;
        // a team of one warp needs no barrier; ids 1..8 serve teams of two warps or more
        if (ks > 1) named_bar_sync(1 + team, ks * 32); else __syncwarp();
        for (int t = share * 32 + lane; t < NN * 32; t += ks * 32) {
            const int n = t >> 5, l = t & 31;
            int d = 0;
            for (int w = 0; w < ks; w++) d += red[((team * ks + w) * NN + n) * 32 + l];
            const int m = mt * 128 + quarter * 32 + l;
            if (n < p.N && m < p.M) {
                const int val = popc_path ? s_pn[n] - 2 * d : (p.epi ? __ldg(p.colsum + (size_t)batch * p.N + n) - 2 * d : d);
                const size_t idx = (size_t)batch * p.M * p.N + (p.out_layout == BGEMM_LAYOUT_NM ? (size_t)n * p.M + m : (size_t)m * p.N + n);
                if (p.out_kind == BGEMM_OUT_I32) {
                    reinterpret_cast<int*>(p.out)[idx] = val;
                } else {
                    const float f = p.out_kind == BGEMM_OUT_F16 ? (float)val : (float)val * __half2float(p.alpha[(size_t)batch * p.M + m]);
                    reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn(f);
                }
            }
        }
        if (ks > 1) named_bar_sync(1 + team, ks * 32); else __syncwarp();
    };

    if (popc_path || STAGE) {
        SkinnyCount cnt[NN];
        int acc[STAGE ? NN : 1][8];                                         // dp4a path only
#pragma unroll
        for (int n = 0; n < NN; n++) cnt[n].reset();
#pragma unroll
        for (int n = 0; n < (STAGE ? NN : 1); n++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[n][j] = 0;
        int slot = 0;
        while (gc < g_end) {
            cp_async_wait<D - 1>();                                         // the oldest of the D units in flight has landed
            const uint4* rs = ring + tid + slot * (2 * T);
            const uint4 lo = rs[0], hi = rs[T];
            if (popc_path) {
                skinny_block_popc<NN>(lo, hi, planes + (size_t)kc * NN * 16, 16, cnt);
            } else if (STAGE) {
                skinny_block_dp4a<STAGE ? NN : 1>(lo, hi, sx + (size_t)kc * 256, x_pitch, acc);
            }
            // The slot's words have been consumed (the arithmetic above waited for them), so the slot may be
            // overwritten: its next unit leaves before this warp may wait at the team's barrier.
            issue(slot, gl < g_end, wl);
            next_load();
            slot = slot + 1 == D ? 0 : slot + 1;
            if (kc + 1 >= kb1) {                                            // the group is complete
#pragma unroll
                for (int n = 0; n < NN; n++) {
                    int d;
                    if (popc_path) {
                        d = cnt[n].total();
                        cnt[n].reset();
                    } else {                                                // acc_j holds 2^j x (its share): exact shifts
                        d = 0;
#pragma unroll
                        for (int j = 0; j < 8; j++) { d += acc[STAGE ? n : 0][j] >> j; acc[STAGE ? n : 0][j] = 0; }
                    }
                    red[(warp * NN + n) * 32 + lane] = d;
                }
                reduce_store(gc);
            }
            advance(gc, kc);
        }
    } else {
        // N = 3..8 with activations that are not ternary after all: correct, not fast. One activation row at a time
        // straight from global memory (columns beyond K meet weight bits that the prepack left at zero); the weights
        // are read again for every row, which keeps this branch out of the register budget of the popc path.
        for (int g = g_begin + team; g < g_end; g += gs) {
            const uint8_t* wrow = plane + (size_t)(g >> 2) * p.kblocks * 4096 + (size_t)((g & 3) * 32 + lane) * 16;
#pragma unroll 1
            for (int n = 0; n < NN; n++) {
                int one[1][8];
#pragma unroll
                for (int j = 0; j < 8; j++) one[0][j] = 0;
                if (n < p.N) {
                    for (int kb = kb0; kb < kb1; kb++) {
                        const uint4 l = __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)kb * 4096));
                        const uint4 h = __ldg(reinterpret_cast<const uint4*>(wrow + (size_t)kb * 4096 + 2048));
                        skinny_block_dp4a<1>(l, h, src + (size_t)n * act_ld + (size_t)kb * 256, act_ld, one);
                    }
                }
                int d = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) d += one[0][j] >> j;
                red[(warp * NN + n) * 32 + lane] = d;
            }
            reduce_store(g);
        }
    }
    cp_async_wait<0>();                          // nothing of this thread's is in flight when it leaves
}

static size_t skinny_smem_bytes(int NN, int kblocks) {      // everything but the weight ring
    const size_t stage = (size_t)NN * (NN <= 2 ? (size_t)kblocks * 256 : ((size_t)kblocks * 256 < (size_t)kSkinnyPiece ? (size_t)kblocks * 256 : (size_t)kSkinnyPiece));
    return (size_t)kblocks * NN * 64 + (size_t)kSkinnyMaxWarps * NN * 32 * sizeof(int) + 32 + stage;
}
constexpr size_t kSkinnyRingBytes = 192 * 1024;        // ring of the deepest variants: 12 K blocks x 16 warps or 6 x 32 warps

template <int NN, int D, int W>
static int launch_skinny_variant(cudaStream_t stream, const GemmParams& p, const int8_t* acts, long long act_ld, long long batch, long long ctas) {
    const size_t smem = skinny_smem_bytes(NN, p.kblocks) + (size_t)D * W * 32 * 32;
    const long long groups = (long long)p.mtiles * 4;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return BGEMM_ERR_DRIVER;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<NN, D, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSkinnyMaxSmem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    // K shares per group: at least four K blocks per warp while that leaves every team of the launch a group to work on
    int ks = 1;
    while (ks < W && p.kblocks / (ks * 2) >= 4) ks *= 2;
    while (ks < W && ks * 2 <= p.kblocks && groups < ctas * (W / ks)) ks *= 2;
    // teams of two or more warps meet at named barriers 1..15: at most 8 teams then (a team of one warp needs none)
    if (ks > 1 && W / ks > 8) ks = W / 8 <= p.kblocks ? W / 8 : 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, (unsigned)batch, 1);
    cfg.blockDim = dim3(32u * W, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (programmatic_launch_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<NN, D, W>, p, acts, act_ld, (int)groups, ks, p.weights_static);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// Largest N served here (tuning override: BGEMM_SKINNY_MAX_N, 0 switches the kernel off). Measured against the
// tensor-core path (24 us at any N <= 16 for 28672 x 8192): N = 1 / 2 / 4 take 9.5 / 13.5 / 15.4 us here, N = 8 takes 26 us.
static int skinny_max_n() {
    static const int v = [] {
        const char* e = std::getenv("BGEMM_SKINNY_MAX_N");
        const int n = e ? std::atoi(e) : 4;
        return n < 0 ? 0 : (n > 8 ? 8 : n);
    }();
    return v;
}

bool skinny_supported(const GemmParams& p, long long batch, bool ternary_acts_expected) {
    if (p.N > skinny_max_n() || p.out_kind == kOutActs || batch > 65535) return false;
    // this kernel writes one result with the default pitch only
    if (p.n_out_more > 0 || p.ldo != (p.out_layout == BGEMM_LAYOUT_NM ? p.M : p.N)) return false;
    // N = 3..8 pays only on the popc path: ops of the form colsum - 2 D whose activations are ternary by contract
    if (p.N > 2 && !(p.epi && ternary_acts_expected)) return false;
    const int NN = p.N <= 1 ? 1 : (p.N <= 2 ? 2 : (p.N <= 4 ? 4 : 8));
    // the activation planes must fit in shared memory, and accumulator 7 (weights of 128) must stay inside int32
    return skinny_smem_bytes(NN, p.kblocks) + kSkinnyRingBytes / 3 <= (size_t)kSkinnyMaxSmem && p.K <= 65536;
}

// One CTA per SM (the ring takes most of its shared memory), fewer per problem with a batch in grid.y. CTAs with
// plenty to stream (128 KB of plane or more each) get 32 warps, which hide the arithmetic's dependent chains better
// (28672 x 8192 x 1: 9.5 against 11.1 us); smaller problems get 16, whose fixed costs are lower (4096 x 4096 x 1: 3.1
// against 4.1 us). The ring is as deep as fits beside the activation planes: 192, 128 or 64 KB.
template <int NN>
static int launch_skinny_depth(cudaStream_t stream, const GemmParams& p, const int8_t* acts, long long act_ld, long long batch) {
    const long long groups = (long long)p.mtiles * 4;
    long long ctas = (sm_count() + batch - 1) / batch;
    if (ctas > groups) ctas = groups;
    const size_t base = skinny_smem_bytes(NN, p.kblocks);
    const int depth = base + kSkinnyRingBytes <= (size_t)kSkinnyMaxSmem ? 3 : (base + kSkinnyRingBytes * 2 / 3 <= (size_t)kSkinnyMaxSmem ? 2 : 1);
    const bool wide = (double)p.plane_batch_bytes / (double)ctas >= 128.0 * 1024.0;
    if (wide) {
        if (depth == 3) return launch_skinny_variant<NN, 6, 32>(stream, p, acts, act_ld, batch, ctas);
        if (depth == 2) return launch_skinny_variant<NN, 4, 32>(stream, p, acts, act_ld, batch, ctas);
        return launch_skinny_variant<NN, 2, 32>(stream, p, acts, act_ld, batch, ctas);
    }
    if (depth == 3) return launch_skinny_variant<NN, 12, 16>(stream, p, acts, act_ld, batch, ctas);
    if (depth == 2) return launch_skinny_variant<NN, 8, 16>(stream, p, acts, act_ld, batch, ctas);
    return launch_skinny_variant<NN, 4, 16>(stream, p, acts, act_ld, batch, ctas);
}

int launch_gemm_skinny(cudaStream_t stream, const GemmParams& p, const int8_t* acts, long long act_ld, long long batch) {
    if (p.N <= 1) return launch_skinny_depth<1>(stream, p, acts, act_ld, batch);
    if (p.N <= 2) return launch_skinny_depth<2>(stream, p, acts, act_ld, batch);
    if (p.N <= 4) return launch_skinny_depth<4>(stream, p, acts, act_ld, batch);
    return launch_skinny_depth<8>(stream, p, acts, act_ld, batch);
}

}  // namespace bgemm
