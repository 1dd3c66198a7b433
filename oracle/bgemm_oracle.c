/*
 * bgemm_oracle.c -- CPU restatement of the 1-bit GEMM path of yifu-ding/BGEMM-CUDA.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or calls this file; it is the
 * checker the GPU results are compared against, and the scalar CPU baseline a benchmark may time.
 *
 * Every function names the reference code it restates (paths relative to the reference project).
 * Parity pin: oracle_pack_rowmajor_msb is checked word for word against the reference's own
 * bin_matrix_prepacking_to_uint32 compiled from its header (see Makefile, target _ref), and the
 * integer products are checked against golden outputs of the reference's torch layers
 * (tests/golden). The device-only PTX definitions (AND / XOR / ATTN) cannot execute on a CPU, so
 * they are restated twice -- once on packed bits exactly as the PTX combines them, once on dense
 * values -- and the two are required to agree.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* ---- fp16 <-> fp32 (IEEE binary16, round to nearest even), no compiler half type needed ---------- */
float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t oracle_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (absx > 0x7f800000u ? 0x200u : 0));
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);            /* rounds to >= 65520 -> inf */
    if (absx < 0x33000001u) return (uint16_t)sign;                         /* below half the smallest subnormal */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u;
    uint32_t shift, half_lsb;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); } else { shift = 13; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    half_lsb = 1u << (shift - 1);
    if (rem > half_lsb || (rem == half_lsb && (q & 1))) q++;
    uint32_t h;
    if (e < -14) h = q;                                  /* subnormal (q may carry into exponent 1) */
    else h = ((uint32_t)(e + 15) << 10) + (q - 0x400u);  /* carry from q propagates into the exponent */
    return (uint16_t)(sign | h);
}

static inline int sign_bit16(uint16_t h) { return (h >> 15) & 1; }
static inline int popc32(uint32_t v) { return __builtin_popcount(v); }

/* Binary value of an fp16: -1 if the sign bit is set else +1 (SIGN_32_HALF_TO_UINT32 keeps only
 * bit 15 of each half, lowbit_kernel/csrc/include/ptx_mma.cuh:371-379).                              */
static inline int bin_val(uint16_t h) { return sign_bit16(h) ? -1 : 1; }
/* Ternary value = torch.sign (tests/python/bgemm_linear.py:241): 0 for +-0, NaN is not modelled.      */
static inline int ter_val(uint16_t h) { return ((h & 0x7fffu) == 0) ? 0 : (sign_bit16(h) ? -1 : 1); }

/* Sign-bit prepack, 32 halves -> one uint32, element k at bit 31-k.
 * Restates _sign_32_half_To_1_uint32 + bin_matrix_prepacking_to_uint32
 * (lowbit_kernel/csrc/utils/weight_prepacking.h:181-230); the reference ORs into an uninitialised
 * malloc (fp6_linear.cu:468), here the destination is written from zero.                              */
void oracle_pack_rowmajor_msb(const uint16_t* src, int64_t rows, int64_t K, int64_t ld, uint32_t* dst) {
    int64_t words = K / 32;
    for (int64_t r = 0; r < rows; r++)
        for (int64_t w = 0; w < words; w++) {
            uint32_t v = 0;
            for (int k = 0; k < 32; k++) v |= (uint32_t)sign_bit16(src[r * ld + w * 32 + k]) << (31 - k);
            dst[r * words + w] = v;
        }
}

/* The three device ops on PACKED words, combined exactly as the PTX does per 128-bit step:
 *   AND  : c += popc(a & b)                                  ptx_mma.cuh:180-210
 *   XOR  : c += 128 - 2 popc(a ^ b)                          ptx_mma.cuh:212-250, utils_core.cuh:274-297
 *   ATTN : c += popc(~a & ~b) - popc(~a & b)                 ptx_mma.cuh:299-336
 * wbits [M, K/32], xbits [N, K/32] in the rowmajor-MSB format; out is [N, M] (M contiguous), the
 * layout PACK_BGEMM_Kernel writes (kernel_matmul.cuh:534-546). K % 128 == 0 as the reference asserts. */
void oracle_bgemm_bits(const uint32_t* wbits, const uint32_t* xbits, int64_t M, int64_t N, int64_t K,
                       int instr, int32_t* out) {
    int64_t words = K / 32;
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            int32_t c = 0;
            for (int64_t s = 0; s < words; s += 4) {            /* one m8n8k128 step */
                int32_t t = 0, t2 = 0;
                for (int q = 0; q < 4; q++) {
                    uint32_t a = wbits[m * words + s + q], b = xbits[n * words + s + q];
                    if (instr == 0) t += popc32(a & b);
                    else if (instr == 1) t += popc32(a ^ b);
                    else { t += popc32(~a & b); t2 += popc32(~a & ~b); }
                }
                if (instr == 0) c += t;
                else if (instr == 1) c += 128 - 2 * t;
                else c += t2 - t;
            }
            out[n * M + m] = c;
        }
}

/* The same four products from DENSE fp16 values (any K). op: 0 AND, 1 XOR, 2 ATTN, 3 BWTA.
 * BWTA is the reference's torch path: ternary(input) @ ternary(weight).T with binary weights
 * (tests/python/bgemm_linear.py:270-272); here weights are binary by sign bit and activations ternary. */
void oracle_bgemm_dense(const uint16_t* w, int64_t ldw, const uint16_t* x, int64_t ldx,
                        int64_t M, int64_t N, int64_t K, int op, int32_t* out) {
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            int32_t c = 0;
            const uint16_t* wr = w + m * ldw;
            const uint16_t* xr = x + n * ldx;
            switch (op) {
            case 0: for (int64_t k = 0; k < K; k++) c += sign_bit16(wr[k]) & sign_bit16(xr[k]); break;
            case 1: for (int64_t k = 0; k < K; k++) c += bin_val(wr[k]) * bin_val(xr[k]); break;
            case 2: for (int64_t k = 0; k < K; k++) c += (1 - sign_bit16(wr[k])) * bin_val(xr[k]); break;
            default: for (int64_t k = 0; k < K; k++) c += bin_val(wr[k]) * ter_val(xr[k]); break;
            }
            out[n * M + m] = c;
        }
}

/* Output conversions.
 *   oracle_store_f16        : __int2half_rn(acc)                       kernel_matmul.cuh:540
 *   oracle_store_f16_scaled : fp16(float(acc) * float(alpha[m])), one fp32 multiply, one rounding --
 *                             the fused form of `out * sw` in Python   bgemm_linear.py:378,482
 * acc is [N, M]; alpha is fp16 [M].                                                                   */
void oracle_store_f16(const int32_t* acc, int64_t count, uint16_t* out) {
    for (int64_t i = 0; i < count; i++) out[i] = oracle_f32_to_f16((float)acc[i]);
}
void oracle_store_f16_scaled(const int32_t* acc, const uint16_t* alpha, int64_t M, int64_t N, uint16_t* out) {
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++)
            out[n * M + m] = oracle_f32_to_f16((float)acc[n * M + m] * oracle_f16_to_f32(alpha[m]));
}

/* Split-K: the reference GEMM writes fp32 partial slabs [Split_K][N*M] and a second kernel sums them
 * and rounds once (kernel_reduction.cuh:29-48). Partial sums are integers below 2^24, so the fp32 sum
 * equals the integer sum; this restatement exists to show that and is compared with the direct path.   */
void oracle_splitk_reduce_f16(const float* slabs, int64_t count, int split_k, uint16_t* out) {
    for (int64_t i = 0; i < count; i++) {
        float s = 0.f;
        for (int t = 0; t < split_k; t++) s += slabs[(int64_t)t * count + i];
        out[i] = oracle_f32_to_f16(s);
    }
}
/* Partial XOR/AND/ATTN/BWTA product over k in [k0, k1), written as float like the reference's
 * split-K GEMM does (kernel_matmul.cuh:543-545).                                                       */
void oracle_bgemm_dense_partial_f32(const uint16_t* w, int64_t ldw, const uint16_t* x, int64_t ldx,
                                    int64_t M, int64_t N, int64_t k0, int64_t k1, int op, float* out) {
    for (int64_t n = 0; n < N; n++)
        for (int64_t m = 0; m < M; m++) {
            int32_t c = 0;
            const uint16_t* wr = w + m * ldw;
            const uint16_t* xr = x + n * ldx;
            for (int64_t k = k0; k < k1; k++) {
                if (op == 0) c += sign_bit16(wr[k]) & sign_bit16(xr[k]);
                else if (op == 1) c += bin_val(wr[k]) * bin_val(xr[k]);
                else if (op == 2) c += (1 - sign_bit16(wr[k])) * bin_val(xr[k]);
                else c += bin_val(wr[k]) * ter_val(xr[k]);
            }
            out[n * M + m] = (float)c;
        }
}

/* Per-row scale of a sign-binarised layer: alpha[m] = mean(|w[m,:]|) accumulated in fp32 in index
 * order, rounded once to fp16. (The reference layers use w.norm(1,1)/w.nelement(), bgemm_linear.py:468;
 * that scalar variant is computed in Python by the layer, not here.)                                  */
void oracle_rowmeanabs_f16(const uint16_t* w, int64_t M, int64_t K, int64_t ld, uint16_t* alpha) {
    for (int64_t m = 0; m < M; m++) {
        double s = 0.0;
        for (int64_t k = 0; k < K; k++) {
            float v = oracle_f16_to_f32(w[m * ld + k]);
            s += v < 0 ? -v : v;
        }
        alpha[m] = oracle_f32_to_f16((float)(s / (double)K));
    }
}

/* Number of sign bits set per row (the "rowpop" a prepack may fold in).                               */
void oracle_rowpop(const uint16_t* w, int64_t M, int64_t K, int64_t ld, int invert, int32_t* rowpop) {
    for (int64_t m = 0; m < M; m++) {
        int32_t c = 0;
        for (int64_t k = 0; k < K; k++) c += sign_bit16(w[m * ld + k]) ^ (invert ? 1 : 0);
        rowpop[m] = c;
    }
}
