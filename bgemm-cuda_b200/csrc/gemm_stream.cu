// Weight-streaming kernel for few activation rows (N <= 16: decode and small-batch shapes), on the legacy int8
// tensor path (mma.sync m16n8k32, u8 x s8 -> s32) fed straight from registers.
//
// At these N the product is HBM streaming of the packed weight plane (one bit per weight). The tcgen05 kernels pay
// for a 128-row tile, tensor-memory set-up and an unpack -> tensor memory -> UMMA round trip per K block that cost
// several times the streaming time; here a warp owns a 32-row group of weights for a range of K blocks, fetches the
// group's 1 KB of a K block with 16-byte asynchronous copies into a private ring in shared memory (several K blocks
// in flight per warp, no barrier involved), turns bit j of every byte into the u8 value 2^j (even j) or 2^(j-1) (odd j,
// from the word shifted right by one) with ONE logic operation per four weights (A fragments: two 16-row fragments per
// warp), and multiplies by the int8 activations (B fragments, ldmatrix from shared memory) into accumulator set j / 2;
// the end adds acc_s >> 2s. Results are int32-exact for any int8 activations (|x| <= 128; K <= 65536 is the limit this
// library keeps for narrow tiles) and bit-identical to the tensor-memory kernels'.
//
// Work split: a CTA owns a contiguous range of 32-row groups; its warps cut the (group, K block) units of the range
// into equal contiguous pieces, add their partial sums into shared memory when they leave a group, and after one
// barrier the CTA converts and stores its rows. Two CTAs of eight warps share an SM where the activations leave room,
// so that under programmatic dependent launch the CTAs of the next launch take over SMs one by one.
//
// `weights_static`: the caller promises that the plane was complete before the previous kernel of the stream was
// launched (weights prepacked at load time). The ring is then filled BEFORE griddepcontrol.wait, i.e. while the
// previous kernel still runs; everything else (activations, column sums, scales, output) is touched after the wait.
//
// Replaces the same reference functions as gemm_umma.cu (PACK_BGEMM_Kernel, lowbit_kernel/csrc/include/
// kernel_matmul.cuh:370-547, which refuses N < 32 altogether: fp6_linear.cu:288-290) for the shapes named above.
#include <cuda_fp16.h>

#include <cstdlib>

#include "internal.h"
#include "ptx.cuh"

namespace bgemm {

namespace {

constexpr int kStreamMaxSmem = 224 * 1024;
constexpr int kGroupsPerPass = 8;             // 32-row groups whose sums a CTA holds in shared memory at a time

__device__ __forceinline__ void st_cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void st_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void st_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Four 8 x 16-byte matrices from shared memory: lane l supplies the address of row l % 8 of matrix l / 8 and receives,
// from each matrix, the four bytes 4 (l % 4) .. of row l / 4 -- exactly the operand fragments of mma.m16n8k32.
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
// D (16 x 8, s32) += A (16 x 32, u8, row) * B (32 x 8, s8, col)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D (16 x 8, f32) += A (16 x 16, f16, row) * B (16 x 8, f16, col)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Two weight bits of a packed word -> a pair of fp16 values -1.0 / +1.0 (bit set = negative). `shift` moves the bit of the
// low half to bit 15; its partner sits 16 bits higher and lands on bit 31. One shift and one three-input logic operation.
__device__ __forceinline__ uint32_t pm1_pair(uint32_t w, int shift) { return ((w << shift) & 0x80008000u) | 0x3C003C00u; }

struct StreamArgs {
    const int8_t* acts;
    long long act_ld;
    const __half* x16;       // fp16 activations [N, K] (binary weight x fp16 activation variant), row pitch x_ld elements
    long long x_ld;
    int groups;              // 32-row groups of one problem (4 per row tile)
    int weights_static;      // fill the ring before the dependency wait
};

// Shared memory: [x rows: N x (Kpad + 16)] [ring: W x D x 1 KB] [sums: kGroupsPerPass x NPAD x 32 int] [row scales] [column sums] [mbarrier, flags]
// F16: the activations are fp16 values (not prepared int8 rows) and the sums are fp32: weight bits become fp16 -1 / +1
// pairs and meet the activations in mma.m16n8k16 (one column tile, N <= 8).
template <int NTILES, int W, int D, bool F16 = false>
__global__ void __launch_bounds__(32 * W, W <= 8 ? 2 : 1) gemm_stream_kernel(const GemmParams p, const StreamArgs a) {
    static_assert(!F16 || NTILES == 1, "the fp16-activation variant has one column tile");
    constexpr int NPAD = 8 * NTILES;
    // Bit slice j of a packed byte is isolated where it stands (value 2^j) for even j, and one position lower in the
    // word shifted right by one (value 2^(j-1)) for odd j: slices 2s and 2s + 1 then share the scale 4^s and one
    // accumulator set, four sets in all; the end adds acc_s >> 2s (exact: set s holds 4^s times its share of the sum).
    constexpr int SETS = F16 ? 1 : 4;
    constexpr int T = 32 * W;
    grid_launch_dependents();
    extern __shared__ __align__(128) uint8_t stream_smem[];
    // activation rows in shared memory: int8 rows of pitch Kpad + 16 (ldmatrix rows of 16 bytes fall on distinct banks),
    // fp16 rows of pitch 2 Kpad + 32 (the 8-byte loads of a half-warp fall on distinct banks)
    const int kpad = p.kblocks * 256, pitch = F16 ? 2 * kpad + 32 : kpad + 16;
    uint8_t* xs = stream_smem;
    uint8_t* ring = xs + (((size_t)p.N * pitch + 127) & ~(size_t)127);
    int* sums = reinterpret_cast<int*>(ring + (size_t)W * D * 1024);
    float* scale_s = reinterpret_cast<float*>(sums + kGroupsPerPass * NPAD * 32);     // per-row scales of the pass's rows
    int* colsum_s = reinterpret_cast<int*>(scale_s + kGroupsPerPass * 32);            // [16] column sums
    uint64_t* bar = reinterpret_cast<uint64_t*>(colsum_s + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 1) + 1;  // flag at byte 12, wait budget at bytes 24..31 (8-byte aligned)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int batch = blockIdx.y;
    const uint8_t* plane = p.plane + (size_t)batch * p.plane_batch_bytes;
    const int g_begin = (int)(((long long)a.groups * blockIdx.x) / gridDim.x);
    const int g_end = (int)(((long long)a.groups * (blockIdx.x + 1)) / gridDim.x);
    const int nkb = p.kblocks;

    if (tid == 0) {
        mbar_init(smem_u32(bar), 1);
        *abort_flag = 0;
        set_wait_budget(abort_flag, p.wait_budget);
        mbar_fence_init();
    }
    for (int i = tid; i < kGroupsPerPass * NPAD * 32; i += T) sums[i] = 0;

    // ---- the warp's sequence of units: for every pass (kGroupsPerPass groups of the CTA's range) the contiguous piece
    //      [U w / W, U (w + 1) / W) of the pass's U = groups x K blocks units, unit u = (group u / nkb, K block u % nkb).
    //      Cursors step through it with additions only (one division per pass).
    struct Cursor {
        int pass_g0;          // first group of the pass; >= g_end: the warp's work is over
        int gl, kb;           // current unit: group (pass-local) and K block
        int left;             // units left in this warp's piece of the pass
        const uint8_t* ptr;   // this lane's 16 bytes of the current unit (used by the load cursor)
    };
    auto unit_ptr = [&](int g, int kb) { return plane + ((size_t)(g >> 2) * nkb + kb) * 4096 + (size_t)((g & 3) * 32 + lane) * 16; };
    auto open_pass = [&](Cursor& c, int g0) {
        c.pass_g0 = g0;
        c.left = 0;
        if (g0 >= g_end) return;
        const int ng = min(kGroupsPerPass, g_end - g0);
        const int U = ng * nkb, u0 = (int)((long long)U * warp / W), u1 = (int)((long long)U * (warp + 1) / W);
        c.left = u1 - u0;
        c.gl = u0 / nkb;
        c.kb = u0 - c.gl * nkb;
        c.ptr = unit_ptr(g0 + c.gl, c.kb);
    };
    // make the cursor point at a unit, skipping empty pieces; false when the warp's work is over
    auto settle = [&](Cursor& c) {
        while (c.pass_g0 < g_end && c.left == 0) open_pass(c, c.pass_g0 + kGroupsPerPass);
        return c.pass_g0 < g_end;
    };
    auto step = [&](Cursor& c) {
        c.left--;
        c.ptr += 4096;
        if (++c.kb == nkb) { c.kb = 0; c.gl++; c.ptr = unit_ptr(c.pass_g0 + c.gl, 0); }
    };
    const uint32_t ring_addr = smem_u32(ring + (size_t)warp * D * 1024) + lane * 16;
    auto issue = [&](uint32_t slot_addr, Cursor& c) {  // always closes a group: one cp.async group per unit
        if (settle(c)) {
            st_cp_async16(slot_addr, c.ptr);
            st_cp_async16(slot_addr + 512, c.ptr + 2048);
            step(c);
        }
        st_cp_async_commit();
    };

    Cursor cl, cc;                       // load cursor runs D units ahead of the compute cursor
    open_pass(cl, g_begin);
    open_pass(cc, g_begin);
    if (a.weights_static) {
#pragma unroll 1
        for (int d = 0; d < D; d++) issue(ring_addr + d * 1024, cl);
    }
    __syncthreads();                     // barrier initialised, sums zeroed
    // From here on the previous kernel's results are needed (activations, column sums) or its reads must be over (output).
    grid_dependency_wait();
    if (!a.weights_static) {
#pragma unroll 1
        for (int d = 0; d < D; d++) issue(ring_addr + d * 1024, cl);
    }
    if (F16) {
        // fp16 activations: every group of four columns (e0, e1, e2, e3) is stored as (e0, e2, e1, e3), the order in which
        // the weight bits of a packed word pair up (bits 16 apart); columns from K on are zero.
        const bool vec = (reinterpret_cast<uintptr_t>(a.x16) & 15) == 0 && (a.x_ld & 7) == 0;
        const int chunks = kpad / 8;
        for (int i = tid; i < p.N * chunks; i += T) {
            const int n = i / chunks, k0 = (i - n * chunks) * 8;
            const __half* src = a.x16 + (size_t)n * a.x_ld + k0;
            uint4 v;
            if (vec && k0 + 8 <= p.K) {
                v = *reinterpret_cast<const uint4*>(src);
            } else {
                __align__(16) __half e[8];
#pragma unroll
                for (int q = 0; q < 8; q++) e[q] = k0 + q < p.K ? src[q] : __ushort_as_half(0);
                v = *reinterpret_cast<const uint4*>(e);
            }
            uint4 o;
            o.x = __byte_perm(v.x, v.y, 0x5410); o.y = __byte_perm(v.x, v.y, 0x7632);
            o.z = __byte_perm(v.z, v.w, 0x5410); o.w = __byte_perm(v.z, v.w, 0x7632);
            *reinterpret_cast<uint4*>(xs + (size_t)n * pitch + (size_t)k0 * 2) = o;
        }
    } else if (tid == 0) {               // activations: one bulk copy per row into the padded rows of xs
        mbar_arrive_expect_tx(smem_u32(bar), (uint32_t)p.N * (uint32_t)kpad);
        const int8_t* src = a.acts + (size_t)batch * p.N * a.act_ld;
        for (int n = 0; n < p.N; n++) bulk_g2s(smem_u32(xs + (size_t)n * pitch), src + (size_t)n * a.act_ld, (uint32_t)kpad, smem_u32(bar));
    }
    // What the epilogue needs from global memory is staged now, so that its latency hides behind the main loop.
    auto stage_epilogue = [&](int pass_g0) {
        for (int i = tid; i < kGroupsPerPass * 32; i += T) {
            const int m = pass_g0 * 32 + i;
            const bool scaled = F16 ? p.alpha != nullptr : p.out_kind == BGEMM_OUT_F16_SCALED;
            scale_s[i] = (scaled && m < p.M) ? __half2float(p.alpha[(size_t)batch * p.M + m]) : 1.f;
        }
        if (tid < 16) colsum_s[tid] = (p.epi && tid < p.N) ? __ldg(p.colsum + (size_t)batch * p.N + tid) : 0;
    };
    stage_epilogue(g_begin);
    bool ok = true;
    if (F16) {
        __syncthreads();                 // the activation rows are in place
    } else {
        ok = mbar_wait(smem_u32(bar), 0, abort_flag, p.status, 31);
        ok = __all_sync(0xffffffffu, ok);
    }

    // B-operand addressing: lane l supplies row (l % 8) of matrix (l / 8); matrix m of a load = 16 bytes at k offset 16 m
    uint32_t xrow[NTILES];
#pragma unroll
    for (int t = 0; t < NTILES; t++) {
        int n = 8 * t + (lane & 7);
        if (n >= p.N) n = p.N - 1;                       // columns beyond N: any valid row, their results are dropped
        xrow[t] = smem_u32(xs + (size_t)n * pitch) + 16 * (lane >> 3);
    }
    // fp16 variant: lane (g, tig) reads, for column g, the permuted four-column group of packed word tig (or 4 + tig)
    uint32_t xrow16 = 0;
    if (F16) {
        int n = lane >> 2;
        if (n >= p.N) n = p.N - 1;
        xrow16 = smem_u32(xs + (size_t)n * pitch) + 8 * (lane & 3);
    }

    int acc[2][SETS][NTILES][4];
    float facc[2][4];                    // fp16 variant
    auto zero_acc = [&]() {
        if (F16) {
#pragma unroll
            for (int f = 0; f < 2; f++)
#pragma unroll
                for (int i = 0; i < 4; i++) facc[f][i] = 0.f;
            return;
        }
#pragma unroll
        for (int f = 0; f < 2; f++)
#pragma unroll
            for (int j = 0; j < SETS; j++)
#pragma unroll
                for (int t = 0; t < NTILES; t++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[f][j][t][i] = 0;
    };
    // add the warp's sums of group `gl` (pass-local) into the CTA's shared sums [gl][n][row]
    auto flush = [&](int gl) {
        const int g = lane >> 2, tig = lane & 3;
        if (F16) {
#pragma unroll
            for (int f = 0; f < 2; f++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int n = 2 * tig + (i & 1), row = 16 * f + g + 8 * (i >> 1);
                    atomicAdd(reinterpret_cast<float*>(sums) + (gl * NPAD + n) * 32 + row, facc[f][i]);
                }
            zero_acc();
            return;
        }
#pragma unroll
        for (int f = 0; f < 2; f++)
#pragma unroll
            for (int t = 0; t < NTILES; t++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    int v = 0;
#pragma unroll
                    for (int j = 0; j < SETS; j++) v += acc[f][j][t][i] >> (2 * j);      // set j holds 4^j x its share: exact
                    const int n = 8 * t + 2 * tig + (i & 1), row = 16 * f + g + 8 * (i >> 1);
                    atomicAdd(&sums[(gl * NPAD + n) * 32 + row], v);
                }
        zero_acc();
    };
    zero_acc();

    int slot = 0;
    uint32_t slot_addr = ring_addr;
    int cur_pass = g_begin;              // pass whose sums are in shared memory
#pragma unroll 1
    while (true) {
        const bool mine = ok && settle(cc);
        // ---- pass boundary: every warp arrives here once per pass of the CTA's range (also warps without units) ----
        const int my_pass = mine ? cc.pass_g0 : g_end;
        while (cur_pass < g_end && my_pass > cur_pass) {
            __syncthreads();             // all partial sums of the pass are in `sums`
            if (ok) {
                const int ng = min(kGroupsPerPass, g_end - cur_pass);
                for (int i = tid; i < ng * NPAD * 32; i += T) {
                    const int row = i & 31, n = (i >> 5) % NPAD, gl = i / (32 * NPAD);
                    const int m = (cur_pass + gl) * 32 + row;
                    const int d = sums[i];
                    sums[i] = 0;
                    if (F16) {
                        if (n < p.N && m < p.M) {
                            const float val = __int_as_float(d) * scale_s[gl * 32 + row];
                            const size_t idx = p.out_layout == BGEMM_LAYOUT_NM ? (size_t)n * p.ldo + m : (size_t)m * p.ldo + n;
                            if (p.out_kind == BGEMM_OUT_F32) reinterpret_cast<float*>(p.out)[idx] = val;
                            else reinterpret_cast<__half*>(p.out)[idx] = __float2half_rn(val);
                        }
                        continue;
                    }
                    if (n < p.N && m < p.M) {
                        const int val = p.epi ? colsum_s[n] - 2 * d : d;
                        const size_t idx = (size_t)batch * p.M * p.N + (p.out_layout == BGEMM_LAYOUT_NM ? (size_t)n * p.ldo + m : (size_t)m * p.ldo + n);
                        const __half hv = __float2half_rn((float)val * scale_s[gl * 32 + row]);
                        for (int dst = 0; dst <= p.n_out_more; dst++) {       // further destinations: peer-mapped copies of the result
                            void* o = dst == 0 ? p.out : p.out_more[dst - 1];
                            if (p.out_kind == BGEMM_OUT_I32) reinterpret_cast<int*>(o)[idx] = val;
                            else reinterpret_cast<__half*>(o)[idx] = hv;
                        }
                    }
                }
            }
            cur_pass += kGroupsPerPass;
            if (cur_pass < g_end) {      // a further pass: its scales replace this one's once everybody has used them
                __syncthreads();
                stage_epilogue(cur_pass);
            }
            __syncthreads();             // `sums` is zero again (and the scales are in place) for the next pass
        }
        if (!mine) break;

        const int gl = cc.gl;
        const uint32_t xo = (uint32_t)cc.kb * 256u;
        st_cp_async_wait<D - 1>();       // the oldest of the D units in flight has landed (this lane's part ...)
        __syncwarp();                    // ... and every other lane's part of it
        uint32_t lo[4], hi[4];
        ldsm_x4(slot_addr, lo);          // word (lane % 4) of rows lane / 4 + {0, 8, 16, 24}
        ldsm_x4(slot_addr + 512, hi);    // word 4 + (lane % 4) of the same rows
        uint32_t lo1[4], hi1[4];         // the same words one bit lower, for the odd slices
#pragma unroll
        for (int i = 0; i < 4; i++) { lo1[i] = lo[i] >> 1; hi1[i] = hi[i] >> 1; }
        issue(slot_addr, cl);            // the slot's words are on their way to registers: its next unit may leave
        slot_addr += 1024;
        if (++slot == D) { slot = 0; slot_addr = ring_addr; }
        if (F16) {
            const uint32_t xo16 = xrow16 + xo * 2;
#pragma unroll
            for (int j = 0; j < 8; j++) {
#pragma unroll
                for (int h = 0; h < 2; h++) {            // packed words tig (h = 0) and 4 + tig (h = 1): 16 columns per step
                    uint32_t b0, b1;
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(xo16 + (32 * j + 16 * h) * 2));
#pragma unroll
                    for (int f = 0; f < 2; f++) {
                        const uint32_t w0 = h ? hi[2 * f] : lo[2 * f], w1 = h ? hi[2 * f + 1] : lo[2 * f + 1];
                        // columns (0, 2) of the word's group: bits j and 16 + j; columns (1, 3): bits 8 + j and 24 + j
                        mma_f16(facc[f], pm1_pair(w0, 15 - j), pm1_pair(w1, 15 - j), pm1_pair(w0, 7 - j), pm1_pair(w1, 7 - j), b0, b1);
                    }
                }
            }
        } else
#pragma unroll
        for (int jp = 0; jp < 4; jp++) {                 // two slices (32 columns each) per B load
            uint32_t b[NTILES][4];
#pragma unroll
            for (int t = 0; t < NTILES; t++) ldsm_x4(xrow[t] + xo + jp * 64, b[t]);
#pragma unroll
            for (int h = 0; h < 2; h++) {
#pragma unroll
                for (int f = 0; f < 2; f++) {
                    // j = 2 jp + h: even slices from the words as they are, odd ones from the shifted words, both at bit 2 jp
                    const uint32_t m = 0x01010101u << (2 * jp);
                    const uint32_t a0 = (h ? lo1[2 * f] : lo[2 * f]) & m, a1 = (h ? lo1[2 * f + 1] : lo[2 * f + 1]) & m;
                    const uint32_t a2 = (h ? hi1[2 * f] : hi[2 * f]) & m, a3 = (h ? hi1[2 * f + 1] : hi[2 * f + 1]) & m;
#pragma unroll
                    for (int t = 0; t < NTILES; t++) mma_u8s8(acc[f][jp][t], a0, a1, a2, a3, b[t][2 * h], b[t][2 * h + 1]);
                }
            }
        }
        step(cc);
        // the warp leaves the group (its piece ends, or the next unit belongs to another group): hand the sums over
        if (cc.left == 0 || cc.gl != gl) flush(gl);
    }
    st_cp_async_wait<0>();               // nothing of this thread's is in flight when it leaves
}

size_t stream_smem_bytes(int N, int kblocks, int NTILES, int W, int D) {
    const size_t x = ((size_t)N * ((size_t)kblocks * 256 + 16) + 127) & ~(size_t)127;
    return x + (size_t)W * D * 1024 + (size_t)kGroupsPerPass * 8 * NTILES * 32 * sizeof(int) + (size_t)kGroupsPerPass * 32 * sizeof(float) + 64 + 64;
}

template <int NTILES, int W, int D>
int launch_stream_variant(cudaStream_t stream, const GemmParams& p, const StreamArgs& a, long long batch) {
    const size_t smem = stream_smem_bytes(p.N, p.kblocks, NTILES, W, D);
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return BGEMM_ERR_DRIVER;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NTILES, W, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamMaxSmem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    // CTAs: as many as the GPU holds at once (one or two per SM), fewer per problem with a batch in grid.y, and never
    // more than the problem has groups.
    static const int forced_per_sm = [] { const char* e = std::getenv("BGEMM_STREAM_CTAS_PER_SM"); return e ? std::atoi(e) : 0; }();   // tuning override
    const int per_sm = (W <= 8 && smem <= 110 * 1024 && forced_per_sm != 1) ? 2 : 1;
    long long ctas = ((long long)sm_count() * per_sm + batch - 1) / batch;
    if (ctas > a.groups) ctas = a.groups;
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<NTILES, W, D>, p, a);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

size_t stream16_smem_bytes(int N, int kblocks, int W, int D) {
    const size_t x = ((size_t)N * ((size_t)kblocks * 512 + 32) + 127) & ~(size_t)127;
    return x + (size_t)W * D * 1024 + (size_t)kGroupsPerPass * 8 * 32 * sizeof(float) + (size_t)kGroupsPerPass * 32 * sizeof(float) + 64 + 64;
}

template <int W, int D>
int launch_stream16_variant(cudaStream_t stream, const GemmParams& p, const StreamArgs& a) {
    const size_t smem = stream16_smem_bytes(p.N, p.kblocks, W, D);
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return BGEMM_ERR_DRIVER;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<1, W, D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamMaxSmem);
        if (e != cudaSuccess) return (int)e;
        configured[dev] = true;
    }
    const int per_sm = (W <= 8 && smem <= 110 * 1024) ? 2 : 1;
    long long ctas = (long long)sm_count() * per_sm;
    if (ctas > a.groups) ctas = a.groups;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas, 1, 1);
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<1, W, D, true>, p, a);
    count_launch();
    return (int)(e != cudaSuccess ? e : cudaGetLastError());
}

// Largest N served here (tuning override: BGEMM_STREAM_MAX_N, 0 switches the kernel off).
int stream_max_n() {
    static const int v = [] {
        const char* e = std::getenv("BGEMM_STREAM_MAX_N");
        const int n = e ? std::atoi(e) : 16;
        return n < 0 ? 0 : (n > 16 ? 16 : n);
    }();
    return v;
}

// The variant for a problem: two CTAs of 8 warps per SM where the activations leave room for a ring of at least four
// K blocks per warp beside them, else one CTA of 16 warps; 0 = does not fit.
int stream_variant(int N, int kblocks) {
    const int NT = N <= 8 ? 1 : 2;
    static const int forced = [] { const char* e = std::getenv("BGEMM_STREAM_VARIANT"); return e ? std::atoi(e) : 0; }();   // tuning override
    if (forced == 88 || forced == 84 || forced == 168 || forced == 164) {
        const int W = forced / 10 >= 16 ? 16 : 8, D = forced % 10;
        if (stream_smem_bytes(N, kblocks, NT, W, D) <= (W == 8 ? 110 * 1024 : (size_t)kStreamMaxSmem)) return forced;
    }
    if (stream_smem_bytes(N, kblocks, NT, 8, 8) <= 110 * 1024) return 88;
    if (stream_smem_bytes(N, kblocks, NT, 8, 4) <= 110 * 1024) return 84;
    if (stream_smem_bytes(N, kblocks, NT, 16, 8) <= (size_t)kStreamMaxSmem) return 168;
    if (stream_smem_bytes(N, kblocks, NT, 16, 4) <= (size_t)kStreamMaxSmem) return 164;
    return 0;
}

}  // namespace

int stream_min_n() {       // smallest N served here (tuning override: BGEMM_STREAM_MIN_N)
    static const int v = [] {
        const char* e = std::getenv("BGEMM_STREAM_MIN_N");
        return e ? std::atoi(e) : 1;
    }();
    return v;
}

bool stream_supported(const GemmParams& p, long long batch) {
    if (p.N > stream_max_n() || p.N < stream_min_n() || p.out_kind == kOutActs || batch > 65535) return false;
    // accumulator set 3 holds 64 x (its quarter of) the sum: |x| <= 128 keeps it inside int32 far beyond this limit, which
    // is the one the other narrow-tile kernels need
    if (p.K > 65536) return false;
    // Batches of 9-16 activation rows: every CTA stages its problem's activations (N x K bytes) for a share of the weights
    // that is hardly larger, and the tensor-core kernels are faster (48 x [1024 x 4096 x 16]: 21 against 30 us;
    // 64 x [2048 x 2048 x 12]: 30 against 41). Up to 8 rows the streaming kernel stays level or ahead.
    if (batch > 1 && p.N > 8) return false;
    return stream_variant(p.N, p.kblocks) != 0;
}

// Activation rows one launch of the fp16-activation variant can hold in shared memory (0: K is too large even for one).
int w1a16_rows_per_launch(int kblocks) {
    for (int n = 8; n >= 1; n--)
        if (stream16_smem_bytes(n, kblocks, 16, 4) <= (size_t)kStreamMaxSmem) return n;
    return 0;
}

// One launch: `p.N` <= w1a16_rows_per_launch activation rows starting at x16.
int launch_gemm_w1a16(cudaStream_t stream, const GemmParams& p, const __half* x16, long long x_ld) {
    StreamArgs a{};
    a.x16 = x16;
    a.x_ld = x_ld;
    a.groups = p.mtiles * 4;
    a.weights_static = p.weights_static;
    if (stream16_smem_bytes(p.N, p.kblocks, 8, 8) <= 110 * 1024) return launch_stream16_variant<8, 8>(stream, p, a);
    if (stream16_smem_bytes(p.N, p.kblocks, 8, 4) <= 110 * 1024) return launch_stream16_variant<8, 4>(stream, p, a);
    if (stream16_smem_bytes(p.N, p.kblocks, 16, 8) <= (size_t)kStreamMaxSmem) return launch_stream16_variant<16, 8>(stream, p, a);
    if (stream16_smem_bytes(p.N, p.kblocks, 16, 4) <= (size_t)kStreamMaxSmem) return launch_stream16_variant<16, 4>(stream, p, a);
    return BGEMM_ERR_UNSUPPORTED;
}

int launch_gemm_stream(cudaStream_t stream, const GemmParams& p, const int8_t* acts, long long act_ld, long long batch, bool weights_static) {
    StreamArgs a{};
    a.acts = acts;
    a.act_ld = act_ld;
    a.groups = p.mtiles * 4;
    a.weights_static = weights_static ? 1 : 0;
    const int v = stream_variant(p.N, p.kblocks);
    if (p.N <= 8) {
        switch (v) {
            case 88: return launch_stream_variant<1, 8, 8>(stream, p, a, batch);
            case 84: return launch_stream_variant<1, 8, 4>(stream, p, a, batch);
            case 168: return launch_stream_variant<1, 16, 8>(stream, p, a, batch);
            case 164: return launch_stream_variant<1, 16, 4>(stream, p, a, batch);
        }
    } else {
        switch (v) {
            case 88: return launch_stream_variant<2, 8, 8>(stream, p, a, batch);
            case 84: return launch_stream_variant<2, 8, 4>(stream, p, a, batch);
            case 168: return launch_stream_variant<2, 16, 8>(stream, p, a, batch);
            case 164: return launch_stream_variant<2, 16, 4>(stream, p, a, batch);
        }
    }
    return BGEMM_ERR_UNSUPPORTED;
}

}  // namespace bgemm
