// Declarations shared by the translation units of libbgemm_b200.so (not part of the public ABI).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/bgemm_b200.h"

namespace bgemm {

struct GemmParams {
    const uint8_t* plane;         // tiled weight-slot bits
    const int32_t* colsum;        // [batch][N]
    void* out;
    const __half* alpha;          // [batch][M] or null
    int32_t* ws_partial;          // split-K slabs [tile][split][NT][128], null when split_k == 1
    unsigned int* ws_counters;    // split-K arrival counters [tile]
    int* status;                  // device status word (0 = fine), may be null
#ifdef BGEMM_TUNING
    long long* prof;              // phase stamps, 32 slots per CTA (tuning builds only)
#endif
    int M, N, K;
    int kblocks;                  // ceil(K / 256)
    int mtiles, ntiles;
    int split_k;
    int cluster;                  // 1: the split_k CTAs of a tile form a cluster and reduce through DSMEM
    int epi;                      // 0: result = D, 1: result = colsum[n] - 2 D
    int out_kind, out_layout;
    long long plane_batch_bytes;
    // kOutActs only: the result becomes the next layer's prepared activations (int8 rows of pitch out_ld in `out`,
    // row sums accumulated into colsum_next, which the launcher has zeroed)
    int32_t* colsum_next;
    long long out_ld;
    int act_mode;
    int acts_general;             // 1: the caller declared general int8 activations (op W1A8); 0: at most ternary expected
    // Output addressing: the row pitch of the result matrix in elements ([N, M] layout: M unless the slab is written into
    // a wider matrix; [M, N] layout: N) and up to 7 further destinations that receive the same result (peer-mapped
    // buffers of other GPUs: the all-gather of a row-sharded layer fused into the epilogue). Batches need the default pitch.
    long long ldo;
    void* out_more[7];
    int n_out_more;
    int weights_static;           // 1: the caller promised that the plane was complete before the previous kernel of the stream was
                                  // launched (bgemm_gemm_static_weights): weight-streaming kernels may fetch it before the dependency wait
    // Test hooks (bgemm_debug_set_wait_test): budget of every bounded wait in SM clocks (0 = the default) and the
    // K block (CTA-relative stream position) whose weight tile the producer withholds (-1 = none).
    long long wait_budget;
    int test_skip_kblock;
};

constexpr int kOutActs = 100;     // internal out_kind of bgemm_gemm_to_acts

void count_launch();
bool programmatic_launch_enabled();   // BGEMM_PDL=0 in the environment switches it off
#ifdef BGEMM_TUNING
long long* debug_profile_buffer();
#endif
int* device_status_word();        // per-device status word, lazily created (cudaGetSymbolAddress)
void apply_test_hooks(GemmParams& p);   // copies the process-wide test settings (normally: none) into the launch parameters

int sm_count();                   // SMs of the current device (cached)
int gemm_tile_n(long long M, long long N, long long K, long long batch);
int max_resident_clusters(int NT, int split, bool deep);   // clusters of `split` CTAs of gemm_kernel the device holds at once; -1: unknown
int launch_gemm(cudaStream_t stream, GemmParams p, const int8_t* acts, long long act_ld, long long batch);

// Persistent variant (gemm_persist.cu); `tensor_map` points to the CUtensorMap of the activations.
bool persistent_supported(int NT);
bool persistent_kblocks_ok(int NT, int kblocks);   // K-block counts per tile the issuers' hand-over protocol covers
int launch_gemm_persistent(cudaStream_t stream, const void* tensor_map, const GemmParams& p, int NT, long long total_tiles, int ctas);

// Persistent kernel on CTA pairs, 256 x 256 tiles (gemm_pair.cu); `tensor_map` must have boxes of 128 activation rows
// and p.ntiles must count 256-column tiles. With p.ws_counters / p.ws_partial set (64 KiB of zeroed flags, one partial
// accumulator per CTA) it splits the work exactly.
void set_pair_mode(int mode);      // bgemm_debug_set_pair_kernel
bool pair_supported(const GemmParams& p, long long batch);
int launch_gemm_pair(cudaStream_t stream, const void* tensor_map, const GemmParams& p, long long batch);
size_t pair_balance_workspace_bytes(long long M, long long N, long long K, long long batch);   // 0: the shape would not use it

// Weight-streaming kernel for N <= 16 on mma.sync int8 (gemm_stream.cu).
bool stream_supported(const GemmParams& p, long long batch);
int w1a16_rows_per_launch(int kblocks);
int launch_gemm_w1a16(cudaStream_t stream, const GemmParams& p, const __half* x16, long long x_ld);
int stream_min_n();               // smallest N the kernel takes (1 unless BGEMM_STREAM_MIN_N says otherwise)
int launch_gemm_stream(cudaStream_t stream, const GemmParams& p, const int8_t* acts, long long act_ld, long long batch, bool weights_static);

// Weight-streaming CUDA-core kernel for N <= 8 (gemm_skinny.cu).
bool skinny_supported(const GemmParams& p, long long batch, bool ternary_acts_expected);
int launch_gemm_skinny(cudaStream_t stream, const GemmParams& p, const int8_t* acts, long long act_ld, long long batch);

int launch_pack_weights(cudaStream_t stream, const void* src, int dtype, long long M, long long K, long long ld, int wbit_mode,
                        void* plane, int32_t* rowpop, void* alpha, long long batch, long long src_batch_stride);
int launch_prepare_acts(cudaStream_t stream, const void* src, int dtype, long long N, long long K, long long ld, int act_mode,
                        int transpose, int8_t* dst, int32_t* colsum, long long batch, long long src_batch_stride);
int launch_pack_rowmajor_msb(cudaStream_t stream, const void* src, int dtype, long long rows, long long K, long long ld, uint32_t* dst);
int launch_retile(cudaStream_t stream, const uint32_t* src_words, long long M, long long K, int invert, void* plane);

// Launch with the programmatic-stream-serialization attribute (when enabled): the kernel may start while the
// previous kernel of the stream drains and must execute griddepcontrol.wait before touching global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (programmatic_launch_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace bgemm
