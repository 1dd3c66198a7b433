/*
 * bgemm_b200.h -- C ABI of libbgemm_b200.so: binary / ternary GEMM for NVIDIA B200 (sm_100a).
 *
 * The library replaces the 1-bit hot path of yifu-ding/BGEMM-CUDA (reference paths below are relative
 * to that project):
 *   - the C++ launcher  bin_pack_linear_kernel()        lowbit_kernel/csrc/fp6_linear.cu:275-337
 *   - the device kernel PACK_BGEMM_Kernel               lowbit_kernel/csrc/include/kernel_matmul.cuh:370-547
 *   - the split-K pass  SplitK_Reduction                lowbit_kernel/csrc/include/kernel_reduction.cuh:29-48
 *   - the binary prepack bin_matrix_prepacking_to_uint32 lowbit_kernel/csrc/utils/weight_prepacking.h:181-230
 *     and its torch wrappers (one of them an empty stub) lowbit_kernel/csrc/fp6_linear.cu:463-542
 * and adds what the reference only has as torch code: the binary-weight x ternary-activation (BWTA)
 * product (tests/python/bgemm_linear.py:246-275), a per-output-channel fp16 scale epilogue
 * (the reference multiplies in Python afterwards, bgemm_linear.py:378,482,512), arbitrary M/N/K,
 * and a batched {0,1} x {-1,+1} attention product (bgemm_linear.py:45-62 loops heads in Python).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the name ends in _host. The library never allocates,
 *     frees or synchronises; the caller owns all buffers and passes a workspace where one is needed.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Every entry point returns an int: 0 = success, < 0 = BGEMM_ERR_* (bad argument; nothing was
 *     launched or enqueued), > 0 = a cudaError_t from the CUDA runtime.
 *   - int32 results are exact: |acc| <= K for binary / ternary activations, <= 128 K for general int8 activations
 *     (op W1A8), for which N <= 32 additionally requires K <= 65536 (BGEMM_ERR_UNSUPPORTED beyond).
 *   - Binary value of an element: -1 if its sign bit is set, else +1 (so +0.0 -> +1, -0.0 -> -1), as in
 *     the reference device code (ptx_mma.cuh:341-399). Ternary value: -1, 0, +1 = torch.sign().
 *   - Result matrices are int32-exact internally; `out_kind` selects how they are stored.
 */
#ifndef BGEMM_B200_H_
#define BGEMM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------------ */
#define BGEMM_OK                 0
#define BGEMM_ERR_NULL          -1   /* a required pointer is NULL                                   */
#define BGEMM_ERR_SHAPE         -2   /* M, N, K, batch or a leading dimension is out of range        */
#define BGEMM_ERR_ALIGN         -3   /* a pointer or leading dimension breaks an alignment rule      */
#define BGEMM_ERR_ENUM          -4   /* unknown dtype / op / out_kind / layout value                 */
#define BGEMM_ERR_WORKSPACE     -5   /* workspace missing or smaller than bgemm_*_workspace_bytes()  */
#define BGEMM_ERR_UNSUPPORTED   -6   /* valid request that this build cannot serve                   */
#define BGEMM_ERR_DRIVER        -7   /* the CUDA driver entry point for tensor maps is unavailable   */
#define BGEMM_ERR_TOO_LARGE     -8   /* size beyond the fixed capacity of an entry point             */

/* ---- element types of unpacked sources --------------------------------------------------------- */
#define BGEMM_DT_F16   0
#define BGEMM_DT_BF16  1
#define BGEMM_DT_F32   2
#define BGEMM_DT_I8    3

/* ---- the operation; values 0..2 are the reference's INSTR argument (include/configs.h:70-72) ---- */
#define BGEMM_OP_AND   0   /* C[n,m] = #k where w and x are both negative  (ptx_mma.cuh:180-210)       */
#define BGEMM_OP_XOR   1   /* C[n,m] = sum_k sgn(w) sgn(x), both in {-1,+1}  (ptx_mma.cuh:212-250)     */
#define BGEMM_OP_ATTN  2   /* C[n,m] = sum_k [w >= 0] sgn(x): w-slot is a {0,1} mask (ptx_mma.cuh:252-337) */
#define BGEMM_OP_BWTA  3   /* C[n,m] = sum_k sgn(w) t(x), t = torch.sign in {-1,0,+1} (bgemm_linear.py:241,270-272) */
#define BGEMM_OP_W1A8  4   /* C[n,m] = sum_k sgn(w) x, x any int8 (prepared with BGEMM_ACT_INT8). Same arithmetic as BWTA, which
                              also returns exact results for such x; this code only tells bgemm_gemm not to expect ternary
                              activations, which keeps N = 3..8 on the tensor-core kernel (accepted by bgemm_gemm only) */

/* ---- how a weight-slot row is turned into a bit (bgemm_pack_weights mode) ----------------------- */
#define BGEMM_WBIT_NEGATIVE     0   /* bit = sign bit            (ops AND, XOR, BWTA)                   */
#define BGEMM_WBIT_NONNEGATIVE  1   /* bit = !sign bit           (op ATTN: 1 where the mask is "1")     */
#define BGEMM_WBIT_NONZERO      2   /* bit = (w != 0)            (mask plane of a ternary matrix)       */
#define BGEMM_WBIT_NEGATIVE_NZ  3   /* bit = (w < 0), -0.0 -> 0  (sign plane of a ternary matrix)       */

/* ---- how an activation-slot element is turned into an int8 (bgemm_prepare_acts mode) ------------ */
#define BGEMM_ACT_SIGN      0   /* -1 if sign bit else +1          (ops XOR, ATTN)                     */
#define BGEMM_ACT_TERNARY   1   /* -1 / 0 / +1 = torch.sign        (op BWTA)                           */
#define BGEMM_ACT_NEG01     2   /* 1 if sign bit else 0            (op AND)                            */
#define BGEMM_ACT_INT8      3   /* int8 source values as they are: binary weight x int8 activation ("W1A8", listed as to-do
                                   in the reference's README.md:29). Source dtype must be BGEMM_DT_I8; use with op BWTA
                                   (result = sum_k sign(w) * x, exact in int32).                                          */

/* ---- how the int32 result is stored ------------------------------------------------------------- */
#define BGEMM_OUT_I32         0   /* int32 accumulators, untouched                                     */
#define BGEMM_OUT_F16         1   /* fp16 = round-to-nearest-even(acc)   (kernel_matmul.cuh:540)       */
#define BGEMM_OUT_F16_SCALED  2   /* fp16 = rne(float(acc) * float(alpha[m])), alpha = per-row scale   */
#define BGEMM_OUT_F32         3   /* fp32 sums (bgemm_w1a16_gemm only)                                  */

/* ---- result matrix orientation ------------------------------------------------------------------ */
#define BGEMM_LAYOUT_NM  0   /* C is [N, M], M contiguous: the reference's linear output (kernel_matmul.cuh:534-546) */
#define BGEMM_LAYOUT_MN  1   /* C is [M, N], N contiguous: what bgemm_attn_matmul returns after its .T (bgemm_linear.py:60) */

/* ---- packed-plane geometry ------------------------------------------------------------------------
 * A weight-slot matrix [M, K] is stored as ONE bit per element in tiles of 128 rows x 256 columns.
 * Tile (mt, kb) covers rows [128 mt, 128 mt + 128) and columns [256 kb, 256 kb + 256); tiles are
 * stored kb-fastest, each tile is 4096 contiguous bytes. A row owns 8 little-endian uint32 words:
 * element k = 256 kb + 32 j + 4 c + b (j in 0..7, c in 0..7, b in 0..3) is bit (8 b + j) of word c,
 * and word c of row r sits at byte (c / 4) * 2048 + r * 16 + (c % 4) * 4 of the tile (two 2 KB halves,
 * so 32 consecutive rows read 16 bytes each as one contiguous 512-byte access). Slice j of a tile is
 * thus a 128 x 32 operand whose 4-element groups are selected by one mask 0x01010101 << j.
 * Rows >= M and columns >= K hold 0 bits.
 *
 * bgemm_plane_bytes(M, K)  = ceil(M/128) * ceil(K/256) * 4096
 * bgemm_act_ld(K)          = ceil(K/256) * 256        (bytes per prepared activation row)
 */
size_t  bgemm_plane_bytes(int64_t M, int64_t K);
int64_t bgemm_act_ld(int64_t K);

/* Reference-compatible row-major prepack: uint32 [rows, K/32], element k of a row is bit 31-(k%32) of
 * word k/32 -- bit for bit what bin_matrix_prepacking_to_uint32 (weight_prepacking.h:203-230) writes.
 * Requires K % 32 == 0. `src` is rows x K with leading dimension `ld` elements. Runs on the GPU
 * (the reference's binary_weight_prepacking_cuda, fp6_linear.cu:519-542, never launched a kernel).   */
int bgemm_pack_rowmajor_msb(void* stream, const void* src, int src_dtype, int64_t rows, int64_t K,
                            int64_t ld, uint32_t* dst);
/* The same on the CPU with HOST pointers (binary_matrix_prepacking_cpu, fp6_linear.cu:463-485).       */
int bgemm_pack_rowmajor_msb_host(const void* src_host, int src_dtype, int64_t rows, int64_t K,
                                 int64_t ld, uint32_t* dst_host);

/* Convert a reference-format row-major plane (above) into the tiled plane the GEMM consumes.          */
int bgemm_retile_rowmajor_msb(void* stream, const uint32_t* src_words, int64_t M, int64_t K,
                              int invert, void* plane);

/* Weight prepack: unpacked [M, K] (leading dimension ld elements) -> tiled bit plane.
 *   wbit_mode  BGEMM_WBIT_*
 *   plane      bgemm_plane_bytes(M, K) bytes, 16-byte aligned; fully written (padding included)
 *   rowpop     optional int32 [M]: number of 1 bits in each row
 *   alpha      optional fp16 [M]: mean(|w[m, :]|), the per-channel scale of a sign-binarised layer
 * `batch` independent matrices are packed in one call: matrix i starts at src + i*src_batch_stride
 * elements and writes plane + i*bgemm_plane_bytes(M,K) (rowpop/alpha + i*M).                          */
int bgemm_pack_weights(void* stream, const void* src, int src_dtype, int64_t M, int64_t K, int64_t ld,
                       int wbit_mode, void* plane, int32_t* rowpop, void* alpha,
                       int64_t batch, int64_t src_batch_stride);
/* CPU twin with HOST pointers (same bytes out).                                                        */
int bgemm_pack_weights_host(const void* src_host, int src_dtype, int64_t M, int64_t K, int64_t ld,
                            int wbit_mode, void* plane_host, int32_t* rowpop_host, void* alpha_host);

/* Packed-weight bundle: ONE byte buffer that holds everything a prepacked layer needs and says which layout it is in,
 * so that a saved layer can be told from one written by another layout version (the reference's prepack returns a
 * bare malloc'd word array, fp6_linear.cu:463-485, and saves nothing):
 *   bytes 0..63   header, little endian: uint32 magic "BGPK" (0x4B504742), uint32 layout version (BGEMM_LAYOUT_VERSION),
 *                 int64 M, int64 K, int32 wbit_mode, int32 reserved, int64 plane offset, int64 rowpop offset,
 *                 int64 alpha offset, int64 total bytes
 *   plane         bgemm_plane_bytes(M, K) bytes at a 256-byte aligned offset (the tiled bit plane above)
 *   rowpop        int32 [M]   number of 1 bits per row
 *   alpha         fp16 [M]    mean |w[m, :]|
 * bgemm_bundle_bytes        total size for an [M, K] matrix (0 for bad sizes)
 * bgemm_bundle_header_host  writes the 64 header bytes at `header_host`
 * bgemm_bundle_parse_host   validates 64 header bytes (magic, version, sizes, offsets against `bundle_bytes`) and
 *                           returns the fields; BGEMM_ERR_UNSUPPORTED for an unknown magic or layout version,
 *                           BGEMM_ERR_SHAPE for inconsistent sizes. Any out pointer may be NULL.
 * The parts are filled by bgemm_pack_weights{,_host} called with plane / rowpop / alpha pointing into the bundle. */
#define BGEMM_LAYOUT_VERSION 1
#define BGEMM_BUNDLE_HEADER_BYTES 64
size_t bgemm_bundle_bytes(int64_t M, int64_t K);
int bgemm_bundle_header_host(void* header_host, int64_t M, int64_t K, int wbit_mode);
int bgemm_bundle_parse_host(const void* header_host, size_t bundle_bytes, int64_t* M, int64_t* K, int* wbit_mode,
                            size_t* plane_offset, size_t* rowpop_offset, size_t* alpha_offset);

/* Activation prepare: unpacked [N, K] (leading dimension ld) -> int8 [N, bgemm_act_ld(K)] (zero padded)
 * plus colsum int32 [N] = sum_k of the int8 row. act_mode BGEMM_ACT_*. Batched like the weights:
 * matrix i reads src + i*src_batch_stride and writes dst + i*N*bgemm_act_ld(K), colsum + i*N.
 * If `transpose` is non-zero the source matrix is [K, N] (ld = its row pitch) and is transposed on the
 * fly: this is value.transpose(-1,-2).contiguous() of bgemm_attn_matmul (bgemm_linear.py:60).          */
int bgemm_prepare_acts(void* stream, const void* src, int src_dtype, int64_t N, int64_t K, int64_t ld,
                       int act_mode, int transpose, int8_t* dst, int32_t* colsum,
                       int64_t batch, int64_t src_batch_stride);

/* The GEMM on prepared operands.
 *   plane     tiled weight-slot bits of an [M, K] matrix (bgemm_pack_weights)
 *   acts      int8 [N, bgemm_act_ld(K)] and colsum int32 [N] (bgemm_prepare_acts with the mode of `op`)
 *   out       BGEMM_LAYOUT_NM: [N, M]; BGEMM_LAYOUT_MN: [M, N]; element type per out_kind
 *   alpha     fp16 [M], required for BGEMM_OUT_F16_SCALED, else may be NULL
 *   N <= 16   is served by a weight-streaming kernel (register-fed mma.sync int8; any op, any int8 activations, K <= 65536
 *             and activations that fit in shared memory beside the weight ring), for which split_k and workspace have no
 *             meaning (they are validated and ignored); results are the same bits.
 *   split_k   >= 1 forces that many K partitions, 0 lets the library choose (at most 8). Up to 8 partitions
 *             are reduced on chip (thread-block cluster + distributed shared memory) and need no workspace.
 *   workspace needed only when split_k > 8: bgemm_gemm_workspace_bytes() bytes, 256-byte aligned.
 *             Zero it once after allocating it; the library restores the part that must be zero
 *             (arrival counters in its first 64 KiB) before each call returns, so one buffer can serve
 *             calls of any shapes one after another on a stream.
 *   batch     number of independent problems (A x V heads); problem i uses plane + i*plane_bytes,
 *             acts + i*N*act_ld, colsum + i*N, out + i*M*N elements, alpha + i*M.
 * Replaces bin_pack_linear_kernel + PACK_BGEMM_Kernel + SplitK_Reduction (see file header).           */
int bgemm_gemm(void* stream, const void* plane, int64_t M, int64_t K,
               const int8_t* acts, const int32_t* colsum, int64_t N,
               int op, void* out, int out_kind, int out_layout, const void* alpha,
               int split_k, void* workspace, size_t workspace_bytes, int64_t batch);
size_t bgemm_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int split_k, int64_t batch);

/* bgemm_gemm with flags (an OR of the values below; 0 = bgemm_gemm).
 *   BGEMM_FLAG_STATIC_WEIGHTS     the promise of bgemm_gemm_static_weights (next entry point).
 *   BGEMM_FLAG_BALANCE_WORKSPACE  `workspace` is a BALANCE workspace: bgemm_gemm_balance_workspace_bytes() bytes, 256-byte
 *       aligned, zeroed once after allocation and never written by anybody but this library (its first 64 KiB are flags
 *       that every launch leaves at zero). With it the kernel for wide activation matrices (N > 512 and K >= 2560; the
 *       size query below says for which calls) splits its work into exactly equal parts per SM pair -- tiles that straddle a boundary are accumulated in two or more places and
 *       summed through the workspace -- instead of whole tiles, which matters whenever the number of 256 x 256 tiles is
 *       not a multiple of the SM pairs (28672 x 8192 x 1024: 171 -> 158 us). Results are the same bits (integer sums).
 *       One balance workspace must not serve two calls that overlap on the GPU; calls on one stream may share it.
 *       bgemm_gemm_balance_workspace_bytes() returns 0 for calls that would not use one (the flag is then ignored);
 *       a workspace that is missing or too small for a call that would is refused with BGEMM_ERR_WORKSPACE.
 *       The flag cannot be combined with split_k > 8 (whose workspace has another layout).
 * No reference counterpart.                                                                                         */
#define BGEMM_FLAG_STATIC_WEIGHTS 1
#define BGEMM_FLAG_BALANCE_WORKSPACE 2
int bgemm_gemm_ex(void* stream, const void* plane, int64_t M, int64_t K,
                  const int8_t* acts, const int32_t* colsum, int64_t N,
                  int op, void* out, int out_kind, int out_layout, const void* alpha,
                  int split_k, void* workspace, size_t workspace_bytes, int64_t batch, int flags);
size_t bgemm_gemm_balance_workspace_bytes(int64_t M, int64_t N, int64_t K, int split_k, int64_t batch);

/* bgemm_gemm with one promise added by the caller: `plane` was complete in device memory BEFORE the kernel that precedes
 * this call on `stream` was launched -- the normal case for inference, where weights are prepacked when the model is
 * loaded (synchronise once after packing). The library launches its kernels so that a kernel may start while its
 * predecessor on the stream is still finishing and waits, inside the kernel, before it touches anything the predecessor
 * may have produced; with this promise the weight-streaming kernels (N <= 16) fetch the first weights ahead of that
 * wait, which hides launch and memory latency behind the previous kernel's tail in back-to-back decode loops.
 * Activations, column sums, scales and the output carry no such promise and are touched after the wait. Without the
 * promise (plane written by the preceding kernels of the stream) use bgemm_gemm. Same arguments, same results.
 * The reference has no counterpart (one stream-0 launch per call, fp6_linear.cu:593).                              */
int bgemm_gemm_static_weights(void* stream, const void* plane, int64_t M, int64_t K,
                              const int8_t* acts, const int32_t* colsum, int64_t N,
                              int op, void* out, int out_kind, int out_layout, const void* alpha,
                              int split_k, void* workspace, size_t workspace_bytes, int64_t batch);

/* The GEMM with its result stored `n_outs` (1..8) times, once at every address of the HOST array `outs_host` (device
 * pointers; the array itself is read during the call only), inside a matrix of row pitch `out_ld` elements
 * ([N, M] layout: out_ld >= M, 0 = M; [M, N] layout: out_ld >= N, 0 = N). This is the all-gather of a row-sharded layer
 * fused into the GEMM epilogue: rank r computes rows [start_r, end_r) of a layer with M_total rows and passes, for every
 * rank q, the peer-mapped address of q's full [N, M_total] result plus start_r elements, with out_ld = M_total; every
 * 16-byte piece of the slab then leaves the SM once per destination as an ordinary global store (remote ones travel
 * over NVLink) while the tensor cores work on the next tile. No TMA and no multicast is involved. The caller makes
 * the stores visible to the other ranks' later kernels the usual way (a cross-rank barrier after the launch).
 * One problem per call (no batch). `flags`: as in bgemm_gemm_ex (1 = the promise of bgemm_gemm_static_weights).
 * The reference has no multi-GPU path; this entry point has no counterpart there.                                  */
int bgemm_gemm_multi_out(void* stream, const void* plane, int64_t M, int64_t K,
                         const int8_t* acts, const int32_t* colsum, int64_t N, int op,
                         void* const* outs_host, int n_outs, int64_t out_ld, int out_kind, int out_layout,
                         const void* alpha, int split_k, void* workspace, size_t workspace_bytes, int flags);

/* Binary weight x fp16 activation ("W1A16", listed as to-do in the reference's README.md:29; no counterpart in its code):
 *   C[n, m] = sum_k sgn(w[m, k]) * x[n, k]   (* alpha[m] when alpha != NULL),   sgn by the sign bit as everywhere else,
 * with fp32 accumulation on the tensor cores (mma.sync m16n8k16: the weight bits are expanded to fp16 -1 / +1 in
 * registers). `plane` is the ordinary tiled weight plane (BGEMM_WBIT_NEGATIVE); `x_f16` is the UNPREPARED activation
 * matrix [N, K], fp16, row pitch x_ld elements. out_kind: BGEMM_OUT_F32 (fp32) or BGEMM_OUT_F16 (fp16 = rne(sum, scaled
 * when alpha is given)); out_layout as in bgemm_gemm. It is a weight-streaming kernel built for decode shapes: eight
 * activation rows per pass over the weights (fewer for very large K), so the time grows with ceil(N / 8); sums of fp32
 * partial sums are order-dependent in their last bits (compare within 1e-3 relative, not bit for bit).
 * BGEMM_ERR_UNSUPPORTED when one activation row does not fit in shared memory beside the weight ring (K beyond ~75000).
 * `weights_static` != 0 adds the promise of bgemm_gemm_static_weights.                                                  */
int bgemm_w1a16_gemm(void* stream, const void* plane, int64_t M, int64_t K, const void* x_f16, int64_t x_ld, int64_t N,
                     void* out, int out_kind, int out_layout, const void* alpha, int weights_static);

/* The same GEMM with a fused activation producer: the result is not stored, it becomes the NEXT layer's prepared
 * activations. next_acts int8 [N, bgemm_act_ld(M)] (this GEMM's M is the next layer's K) receives
 * act(fp16 result) under next_act_mode (BGEMM_ACT_*), where the fp16 result is rne(acc) or, with alpha != NULL,
 * rne(float(acc) * float(alpha[m])) -- bit for bit what bgemm_gemm (BGEMM_OUT_F16 / _SCALED, BGEMM_LAYOUT_NM)
 * followed by bgemm_prepare_acts would produce -- and next_colsum int32 [N] its row sums. Both buffers are
 * fully written (padding zeroed) by the call. Batched like bgemm_gemm (problem i: next_acts + i*N*act_ld(M),
 * next_colsum + i*N). Replaces the per-layer elementwise chain between two binary layers of the reference
 * (sign / scale / cast of the fp16 output, tests/python/bgemm_linear.py:479-484 and :357-378).               */
int bgemm_gemm_to_acts(void* stream, const void* plane, int64_t M, int64_t K,
                       const int8_t* acts, const int32_t* colsum, int64_t N, int op, const void* alpha,
                       int next_act_mode, int8_t* next_acts, int32_t* next_colsum,
                       int split_k, void* workspace, size_t workspace_bytes, int64_t batch);

/* bgemm_gemm_to_acts with flags: BGEMM_FLAG_STATIC_WEIGHTS as in bgemm_gemm_ex, and
 *   BGEMM_FLAG_SUMS_ZEROED   the caller has set next_colsum to zero on `stream` before this call (for instance one
 *       memset over the row-sum buffers of all layers of a chain at the start of a forward pass): the library adds
 *       the row sums to it without its own memset, so that nothing but kernels stands between the GEMMs of the chain
 *       (in a CUDA graph a memset node costs about as much as a small kernel and ends the overlap of consecutive
 *       launches). Sums that do not start at zero give wrong row sums, nothing worse.                              */
#define BGEMM_FLAG_SUMS_ZEROED 4
int bgemm_gemm_to_acts_ex(void* stream, const void* plane, int64_t M, int64_t K,
                          const int8_t* acts, const int32_t* colsum, int64_t N, int op,
                          const void* alpha, int next_act_mode, int8_t* next_acts, int32_t* next_colsum,
                          int split_k, void* workspace, size_t workspace_bytes, int64_t batch, int flags);
/* The split_k the library would pick for split_k = 0.                                                 */
int bgemm_gemm_auto_split_k(int64_t M, int64_t N, int64_t K, int64_t batch);

/* Literal drop-in for bin_pack_linear_kernel(stream, Weight, B, C, M, N, K, workspace, Split_K, INSTR)
 * (fp6_linear.cu:275-337): unpacked fp16 weights [M, K] and activations [N, K] in, fp16 [N, M] out
 * (BGEMM_OUT_F16). Unlike the reference M, N, K are unrestricted, split_k may be 0 (auto) and the
 * workspace (bgemm_linear_workspace_bytes) also holds the packed operands. Same zero-once rule.
 * out_kind / out_layout / alpha as in bgemm_gemm so callers can fuse the scale.                       */
int bgemm_linear_forward(void* stream, const void* weight_f16, const void* acts_f16, void* out,
                         int64_t M, int64_t N, int64_t K, int op, int out_kind, int out_layout,
                         const void* alpha, int split_k, void* workspace, size_t workspace_bytes);
size_t bgemm_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int split_k);

/* Text for a status returned by any entry point (static storage).                                     */
const char* bgemm_status_string(int status);
/* Library version: major*10000 + minor*100 + patch.                                                   */
int bgemm_version(void);
/* Number of kernels this library has launched in this process (for launch accounting in benchmarks). */
uint64_t bgemm_launch_count(void);

/* bgemm_linear_forward for callers that cannot provide a workspace. This entry point has no counterpart in the
 * reference, whose wrapper allocates its scratch with torch::empty on every call (fp6_linear.cu:580-586).
 *
 * Who needs it: code that runs where device memory cannot be obtained at call time -- a serving loop that
 * reserves all GPU memory for its own pools at start-up and forbids allocation on the request path (an
 * allocation may take a driver-wide lock, synchronise the device or simply fail once the pools own the
 * memory), or a plug-in written in C whose host application owns the allocator and exposes no hook to it.
 * Such callers still pass their operands and the output buffer; only the library's internal scratch (packed
 * weight plane, int8 activations, column sums) is missing, and here it comes from a fixed array of
 * BGEMM_NOALLOC_SCRATCH_BYTES in device global memory that belongs to the library image. Every GPU that loads
 * the library holds that array until the process exits.
 *
 * Same arguments and results as bgemm_linear_forward, minus split_k (chosen by the library, at most 8, so the
 * reduction stays on chip) and the workspace. Limits and rules:
 *   - the problem must satisfy bgemm_linear_workspace_bytes(M, N, K, 0) <= BGEMM_NOALLOC_SCRATCH_BYTES (for
 *     example M = K = 4096 with N up to ~1400, or 28672 x 1024 x 16); larger ones return BGEMM_ERR_TOO_LARGE
 *     and launch nothing;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress with that device
 *     current) and sets kernel attributes; make that first call outside any stream capture;
 *   - the call itself performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *   - all calls on a device share the one array, which keeps the previous call's contents: nothing in it has
 *     to start at zero for this variant, but two calls whose kernels can overlap on the GPU (different
 *     streams, or different host threads without ordering) race on it -- serialise them on one stream.        */
#define BGEMM_NOALLOC_SCRATCH_BYTES (8u << 20)
int bgemm_linear_forward_noalloc(void* stream, const void* weight_f16, const void* acts_f16, void* out,
                                 int64_t M, int64_t N, int64_t K, int op, int out_kind, int out_layout,
                                 const void* alpha);

/* Every wait inside the kernels is time-bounded (about 0.2 s of SM clock). A wait that runs out makes its kernel
 * drain and exit normally and records a small positive code in a per-device status word (11-18: tile-per-CTA
 * GEMM, 21-29: persistent GEMM; the number names the barrier that was not reached); the results of that launch
 * are then undefined. This call synchronises with the device, returns the word (0 = no wait
 * ever ran out) and clears it when `reset` is non-zero. The reference has no counterpart: its kernels
 * have no inter-thread waits beyond __syncthreads (kernel_matmul.cuh:458-459,507-508).                   */
int bgemm_device_status(int reset);

/* Test hook for the wait-expiry path above (no counterpart in the reference; not for production use). The settings
 * are process-wide and apply to the GEMM launches that follow: `wait_budget_clocks` > 0 shortens every bounded wait
 * to that many SM clocks (0 = back to the default), and `skip_kblock` >= 0 makes the weight producer of every CTA
 * of the tensor-core kernels withhold the weight tile of that K block (counted from the start of the CTA's own K
 * range; -1 = none), so that the consumers' waits run out: the launch then drains, exits normally and reports a
 * code through bgemm_device_status; its results are undefined. Nothing faults or hangs.                     */
void bgemm_debug_set_wait_test(int64_t wait_budget_clocks, int skip_kblock);

/* Test and tuning hook (no counterpart in the reference): which launches the kernel on SM pairs (256 x 256 tiles,
 * tcgen05 cta_group::2) takes. 1 = every launch whose shape it can take (N >= 256, an even number of 128-row tiles,
 * K > 256, no K partitioning), however small; 0 = none; -1 = the library's own rule (the default; the BGEMM_PAIR
 * environment variable sets the same at load time). Process-wide; results never depend on it.             */
void bgemm_debug_set_pair_kernel(int mode);

#ifdef __cplusplus
}
#endif
#endif /* BGEMM_B200_H_ */
