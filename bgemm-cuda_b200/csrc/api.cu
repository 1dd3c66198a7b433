// extern "C" surface of libbgemm_b200.so: argument validation, workspace carving, launch order.
// Declared and documented in include/bgemm_b200.h.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "internal.h"

namespace bgemm {

static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

bool programmatic_launch_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("BGEMM_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

#ifdef BGEMM_TUNING
static long long* g_prof = nullptr;
long long* debug_profile_buffer() { return g_prof; }
#endif

// Device status word: kernels record here which bounded wait ran out (0 = never). One word per device,
// addressed through cudaGetSymbolAddress with that device current.
__device__ int g_status_word = 0;
int* device_status_word() {
    static int* cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!cache[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_status_word) != cudaSuccess) return nullptr;
        cache[dev] = static_cast<int*>(ptr);
    }
    return cache[dev];
}

// Test settings of bgemm_debug_set_wait_test (process-wide; 0 / -1 = none).
static std::atomic<long long> g_test_wait_budget{0};
static std::atomic<int> g_test_skip_kblock{-1};
void apply_test_hooks(GemmParams& p) {
    p.wait_budget = g_test_wait_budget.load(std::memory_order_relaxed);
    p.test_skip_kblock = g_test_skip_kblock.load(std::memory_order_relaxed);
}

static bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
static bool valid_dtype(int d) { return d >= BGEMM_DT_F16 && d <= BGEMM_DT_I8; }
static size_t dt_size(int d) { return d == BGEMM_DT_F32 ? 4 : (d == BGEMM_DT_I8 ? 1 : 2); }

// Largest M, N, K: keeps index computations and the int32 accumulators of binary / ternary activations exact
// (|acc| <= K). General int8 activations (|acc| <= 128 K) are exact up to K = 2^24 as well on tiles of 64 columns or
// more; narrower tiles are limited to kMaxKGeneralNarrow (see bgemm_gemm).
constexpr long long kMaxDim = 1LL << 24;
constexpr long long kMaxKGeneralNarrow = 65536;
constexpr int kMaxSplitK = 64;
constexpr int kMaxClusterSplit = 8;           // portable thread-block cluster size
// Split-K beyond the cluster limit keeps one arrival counter per output tile in a FIXED-size prefix of the
// workspace, so that a workspace shared by calls of different shapes never has partial sums where a later
// call expects zeroed counters.
constexpr size_t kCounterBytes = 64 * 1024;
constexpr long long kMaxCounterTiles = kCounterBytes / 4;

static size_t counter_bytes(long long) { return kCounterBytes; }

static int resolve_split_k(long long M, long long N, long long K, long long batch, int split_k) {
    const long long kblocks = (K + 255) / 256;
    const int NT = gemm_tile_n(M, N, K, batch);
    const long long tiles = ((M + 127) / 128) * ((N + NT - 1) / NT) * batch;
    if (split_k >= 1) {
        if (split_k > kMaxClusterSplit && tiles > kMaxCounterTiles) split_k = kMaxClusterSplit;
        return (int)(split_k > kblocks ? kblocks : split_k);
    }
    // auto: fill the SMs once (one deep-pipeline CTA per SM measured best), keep at least 2 K blocks per partition
    const long long target = sm_count();
    long long s = target / (tiles > 0 ? tiles : 1);
    if (s < 1) s = 1;
    if (s > kblocks / 2) s = kblocks / 2;
    if (s < 1) s = 1;
    if (s > kMaxClusterSplit) s = kMaxClusterSplit;
    // every cluster resident at once: a launch that needs a second wave of clusters takes twice as long
    while (s > 1) {
        const int fit = max_resident_clusters(NT, (int)s, tiles * s <= sm_count());
        if (fit < 0 || tiles <= fit) break;
        s--;
    }
    return (int)s;
}

}  // namespace bgemm

using namespace bgemm;

extern "C" {

size_t bgemm_plane_bytes(int64_t M, int64_t K) {
    if (M < 1 || K < 1) return 0;
    return (size_t)((M + 127) / 128) * (size_t)((K + 255) / 256) * 4096;
}
int64_t bgemm_act_ld(int64_t K) { return K < 1 ? 0 : (K + 255) / 256 * 256; }

int bgemm_version(void) { return 200; }

// ---- packed-weight bundle (host-side bookkeeping only) ---------------------------------------------------------
namespace {
struct BundleHeader {
    uint32_t magic, version;
    int64_t M, K;
    int32_t wbit_mode, reserved;
    int64_t plane_off, rowpop_off, alpha_off, total;
};
static_assert(sizeof(BundleHeader) == BGEMM_BUNDLE_HEADER_BYTES, "bundle header is 64 bytes");
constexpr uint32_t kBundleMagic = 0x4B504742u;     // "BGPK"
bool bundle_layout(int64_t M, int64_t K, BundleHeader* h) {
    if (M < 1 || K < 1 || M > kMaxDim || K > kMaxDim) return false;
    size_t o = 256;
    h->plane_off = (int64_t)o; o += align_up(bgemm_plane_bytes(M, K), 256);
    h->rowpop_off = (int64_t)o; o += align_up((size_t)M * 4, 256);
    h->alpha_off = (int64_t)o; o += align_up((size_t)M * 2, 256);
    h->total = (int64_t)o;
    return true;
}
}  // namespace

size_t bgemm_bundle_bytes(int64_t M, int64_t K) {
    BundleHeader h{};
    return bundle_layout(M, K, &h) ? (size_t)h.total : 0;
}
int bgemm_bundle_header_host(void* header_host, int64_t M, int64_t K, int wbit_mode) {
    if (!header_host) return BGEMM_ERR_NULL;
    if (wbit_mode < BGEMM_WBIT_NEGATIVE || wbit_mode > BGEMM_WBIT_NEGATIVE_NZ) return BGEMM_ERR_ENUM;
    BundleHeader h{};
    if (!bundle_layout(M, K, &h)) return BGEMM_ERR_SHAPE;
    h.magic = kBundleMagic; h.version = BGEMM_LAYOUT_VERSION; h.M = M; h.K = K; h.wbit_mode = wbit_mode;
    std::memcpy(header_host, &h, sizeof(h));
    return BGEMM_OK;
}
int bgemm_bundle_parse_host(const void* header_host, size_t bundle_bytes, int64_t* M, int64_t* K, int* wbit_mode, size_t* plane_offset,
                            size_t* rowpop_offset, size_t* alpha_offset) {
    if (!header_host) return BGEMM_ERR_NULL;
    BundleHeader h;
    std::memcpy(&h, header_host, sizeof(h));
    if (h.magic != kBundleMagic || h.version != BGEMM_LAYOUT_VERSION) return BGEMM_ERR_UNSUPPORTED;
    BundleHeader want{};
    if (!bundle_layout(h.M, h.K, &want) || h.wbit_mode < BGEMM_WBIT_NEGATIVE || h.wbit_mode > BGEMM_WBIT_NEGATIVE_NZ) return BGEMM_ERR_SHAPE;
    if (h.plane_off != want.plane_off || h.rowpop_off != want.rowpop_off || h.alpha_off != want.alpha_off || h.total != want.total ||
        (size_t)h.total > bundle_bytes)
        return BGEMM_ERR_SHAPE;
    if (M) *M = h.M;
    if (K) *K = h.K;
    if (wbit_mode) *wbit_mode = h.wbit_mode;
    if (plane_offset) *plane_offset = (size_t)h.plane_off;
    if (rowpop_offset) *rowpop_offset = (size_t)h.rowpop_off;
    if (alpha_offset) *alpha_offset = (size_t)h.alpha_off;
    return BGEMM_OK;
}
#ifdef BGEMM_TUNING
// Tuning builds only (-DBGEMM_TUNING; not declared in the public header): device buffer that the GEMM kernels fill with
// phase stamps and wait-time counters, 32 int64 per CTA; the persistent kernel appends an event trace of its CTA 0
// (8 x 1024 int64 behind the per-CTA slots), so size it for (CTAs of the launch) * 32 + 8192 entries. NULL = off.
// One process-wide pointer: set it from one thread, for one device.
void bgemm_debug_set_profile_buffer(void* dev_buffer) { g_prof = static_cast<long long*>(dev_buffer); }
#endif
uint64_t bgemm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void bgemm_debug_set_wait_test(int64_t wait_budget_clocks, int skip_kblock) {
    g_test_wait_budget.store(wait_budget_clocks > 0 ? wait_budget_clocks : 0, std::memory_order_relaxed);
    g_test_skip_kblock.store(skip_kblock >= 0 ? skip_kblock : -1, std::memory_order_relaxed);
}

void bgemm_debug_set_pair_kernel(int mode) { set_pair_mode(mode); }

int bgemm_device_status(int reset) {
    int* w = device_status_word();
    if (!w) return BGEMM_ERR_DRIVER;
    int v = 0;
    if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return BGEMM_ERR_DRIVER;
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpy(w, &zero, sizeof(int), cudaMemcpyHostToDevice);
    }
    return v;
}

const char* bgemm_status_string(int status) {
    switch (status) {
        case BGEMM_OK: return "ok";
        case BGEMM_ERR_NULL: return "a required pointer is NULL";
        case BGEMM_ERR_SHAPE: return "M, N, K, batch or a leading dimension is out of range";
        case BGEMM_ERR_ALIGN: return "a pointer or leading dimension breaks an alignment rule";
        case BGEMM_ERR_ENUM: return "unknown dtype / op / out_kind / layout value";
        case BGEMM_ERR_WORKSPACE: return "workspace missing or too small";
        case BGEMM_ERR_UNSUPPORTED: return "request not supported by this build";
        case BGEMM_ERR_DRIVER: return "CUDA driver entry point for tensor maps unavailable or rejected the map";
        case BGEMM_ERR_TOO_LARGE: return "size beyond the fixed capacity of this entry point";
        default: return status > 0 ? cudaGetErrorString((cudaError_t)status) : "unknown status";
    }
}

int bgemm_pack_rowmajor_msb(void* stream, const void* src, int src_dtype, int64_t rows, int64_t K, int64_t ld, uint32_t* dst) {
    if (!src || !dst) return BGEMM_ERR_NULL;
    if (!valid_dtype(src_dtype)) return BGEMM_ERR_ENUM;
    if (rows < 1 || K < 32 || K % 32 != 0 || ld < K || rows > kMaxDim || K > kMaxDim) return BGEMM_ERR_SHAPE;
    return launch_pack_rowmajor_msb((cudaStream_t)stream, src, src_dtype, rows, K, ld, dst);
}

int bgemm_retile_rowmajor_msb(void* stream, const uint32_t* src_words, int64_t M, int64_t K, int invert, void* plane) {
    if (!src_words || !plane) return BGEMM_ERR_NULL;
    if (M < 1 || K < 32 || K % 32 != 0 || M > kMaxDim || K > kMaxDim) return BGEMM_ERR_SHAPE;
    if (!aligned(plane, 16)) return BGEMM_ERR_ALIGN;
    return launch_retile((cudaStream_t)stream, src_words, M, K, invert ? 1 : 0, plane);
}

int bgemm_pack_weights(void* stream, const void* src, int src_dtype, int64_t M, int64_t K, int64_t ld, int wbit_mode, void* plane,
                       int32_t* rowpop, void* alpha, int64_t batch, int64_t src_batch_stride) {
    if (!src || !plane) return BGEMM_ERR_NULL;
    if (!valid_dtype(src_dtype) || wbit_mode < BGEMM_WBIT_NEGATIVE || wbit_mode > BGEMM_WBIT_NEGATIVE_NZ) return BGEMM_ERR_ENUM;
    if (M < 1 || K < 1 || ld < K || batch < 1 || batch > 65535 || M > kMaxDim || K > kMaxDim) return BGEMM_ERR_SHAPE;
    if (batch > 1 && src_batch_stride < 0) return BGEMM_ERR_SHAPE;
    if (!aligned(plane, 16) || !aligned(src, dt_size(src_dtype))) return BGEMM_ERR_ALIGN;
    return launch_pack_weights((cudaStream_t)stream, src, src_dtype, M, K, ld, wbit_mode, plane, rowpop, alpha, batch, src_batch_stride);
}

int bgemm_prepare_acts(void* stream, const void* src, int src_dtype, int64_t N, int64_t K, int64_t ld, int act_mode, int transpose,
                       int8_t* dst, int32_t* colsum, int64_t batch, int64_t src_batch_stride) {
    if (!src || !dst || !colsum) return BGEMM_ERR_NULL;
    if (!valid_dtype(src_dtype) || act_mode < 0 || act_mode > BGEMM_ACT_INT8) return BGEMM_ERR_ENUM;
    if (act_mode == BGEMM_ACT_INT8 && src_dtype != BGEMM_DT_I8) return BGEMM_ERR_UNSUPPORTED;
    if (N < 1 || K < 1 || batch < 1 || batch > 65535 || N > kMaxDim || K > kMaxDim) return BGEMM_ERR_SHAPE;
    if (ld < (transpose ? N : K)) return BGEMM_ERR_SHAPE;
    if (!aligned(dst, 16) || !aligned(src, dt_size(src_dtype))) return BGEMM_ERR_ALIGN;
    return launch_prepare_acts((cudaStream_t)stream, src, src_dtype, N, K, ld, act_mode, transpose ? 1 : 0, dst, colsum, batch,
                               src_batch_stride);
}

int bgemm_gemm_auto_split_k(int64_t M, int64_t N, int64_t K, int64_t batch) {
    if (M < 1 || N < 1 || K < 1 || batch < 1) return 1;
    return resolve_split_k(M, N, K, batch, 0);
}

size_t bgemm_gemm_workspace_bytes(int64_t M, int64_t N, int64_t K, int split_k, int64_t batch) {
    if (M < 1 || N < 1 || K < 1 || batch < 1) return 0;
    const int s = resolve_split_k(M, N, K, batch, split_k);
    if (s <= kMaxClusterSplit) return 0;          // cluster / DSMEM reduction needs no global memory
    const int NT = gemm_tile_n(M, N, K, batch);
    const long long tiles = ((M + 127) / 128) * ((N + NT - 1) / NT) * batch;
    return counter_bytes(tiles) + (size_t)tiles * (size_t)s * (size_t)NT * 128 * 4;
}

// Optional workspace of bgemm_gemm and its variants (see the header): with it the CTA-pair kernel cuts its work into
// exactly equal ranges per SM pair. Layout: [64 KiB of flags, zero between launches][one partial accumulator per CTA].
size_t bgemm_gemm_balance_workspace_bytes(int64_t M, int64_t N, int64_t K, int split_k, int64_t batch) {
    if (M < 1 || N < 1 || K < 1 || batch < 1) return 0;
    if (resolve_split_k(M, N, K, batch, split_k) != 1) return 0;
    return pair_balance_workspace_bytes(M, N, K, batch);
}

static int gemm_entry(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N, int op,
                      void* out, int out_kind, int out_layout, const void* alpha, int split_k, void* workspace, size_t workspace_bytes,
                      int64_t batch, int flags, void* const* more_outs = nullptr, int n_more = 0, int64_t out_ld = 0) {
    const int weights_static = (flags & BGEMM_FLAG_STATIC_WEIGHTS) ? 1 : 0;
    if (flags & ~(BGEMM_FLAG_STATIC_WEIGHTS | BGEMM_FLAG_BALANCE_WORKSPACE)) return BGEMM_ERR_ENUM;
    if (!plane || !acts || !colsum || !out) return BGEMM_ERR_NULL;
    if (n_more < 0 || n_more > 7 || (n_more > 0 && !more_outs)) return BGEMM_ERR_SHAPE;
    for (int i = 0; i < n_more; i++)
        if (!more_outs[i]) return BGEMM_ERR_NULL;
    if (op < BGEMM_OP_AND || op > BGEMM_OP_W1A8 || out_kind < BGEMM_OUT_I32 || out_kind > BGEMM_OUT_F16_SCALED ||
        out_layout < BGEMM_LAYOUT_NM || out_layout > BGEMM_LAYOUT_MN)
        return BGEMM_ERR_ENUM;
    if (out_kind == BGEMM_OUT_F16_SCALED && !alpha) return BGEMM_ERR_NULL;
    if (M < 1 || N < 1 || K < 1 || batch < 1 || batch > 65535 || M > kMaxDim || N > kMaxDim || K > kMaxDim || split_k < 0 ||
        split_k > kMaxSplitK)
        return BGEMM_ERR_SHAPE;
    if (!aligned(plane, 16) || !aligned(acts, 16) || !aligned(colsum, 4) || !aligned(out, out_kind == BGEMM_OUT_I32 ? 4 : 2))
        return BGEMM_ERR_ALIGN;
    for (int i = 0; i < n_more; i++)
        if (!aligned(more_outs[i], out_kind == BGEMM_OUT_I32 ? 4 : 2)) return BGEMM_ERR_ALIGN;
    const int64_t ld_default = out_layout == BGEMM_LAYOUT_NM ? M : N;
    if (out_ld == 0) out_ld = ld_default;
    if (out_ld < ld_default || out_ld > (int64_t)1 << 40 || (out_ld != ld_default && batch != 1)) return BGEMM_ERR_SHAPE;
    // Tiles of 16 and 32 columns keep bit j of a weight byte at value 2^j and shift the sums down afterwards: with
    // general int8 activations accumulator 7 holds up to 128 * 128 * K, which leaves int32 beyond K = 65536.
    if (op == BGEMM_OP_W1A8 && N <= 32 && K > kMaxKGeneralNarrow) return BGEMM_ERR_UNSUPPORTED;
    const int s = resolve_split_k(M, N, K, batch, split_k);
    const long long mtiles = (M + 127) / 128;
    if (mtiles * s > 65535) return BGEMM_ERR_SHAPE;

    GemmParams p{};
    p.plane = static_cast<const uint8_t*>(plane);
    p.colsum = colsum;
    p.out = out;
    p.alpha = static_cast<const __half*>(alpha);
    p.status = device_status_word();
    apply_test_hooks(p);
#ifdef BGEMM_TUNING
    p.prof = debug_profile_buffer();
#endif
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.kblocks = (int)((K + 255) / 256);
    p.mtiles = (int)mtiles;
    p.split_k = s;
    p.epi = (op == BGEMM_OP_XOR || op == BGEMM_OP_BWTA || op == BGEMM_OP_W1A8) ? 1 : 0;
    p.acts_general = op == BGEMM_OP_W1A8 ? 1 : 0;
    p.weights_static = weights_static;
    p.ldo = out_ld;
    p.n_out_more = n_more;
    for (int i = 0; i < n_more; i++) p.out_more[i] = more_outs[i];
    p.out_kind = out_kind;
    p.out_layout = out_layout;
    p.plane_batch_bytes = (long long)bgemm_plane_bytes(M, K);
    p.cluster = (s > 1 && s <= kMaxClusterSplit) ? 1 : 0;
    if (s > kMaxClusterSplit) {
        const size_t need = bgemm_gemm_workspace_bytes(M, N, K, s, batch);
        if (!workspace || workspace_bytes < need) return BGEMM_ERR_WORKSPACE;
        if (!aligned(workspace, 256)) return BGEMM_ERR_ALIGN;
        const int NT = gemm_tile_n(M, N, K, batch);
        const long long tiles = mtiles * ((N + NT - 1) / NT) * batch;
        p.ws_counters = static_cast<unsigned int*>(workspace);
        p.ws_partial = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + counter_bytes(tiles));
    } else if (s == 1 && (flags & BGEMM_FLAG_BALANCE_WORKSPACE)) {
        // the caller declared `workspace` to be a balance workspace (zeroed once, used for nothing else): room for the
        // pair kernel's exact work split, if this shape takes that kernel
        const size_t want = pair_balance_workspace_bytes(M, N, K, batch);
        if (want) {
            if (!workspace || workspace_bytes < want) return BGEMM_ERR_WORKSPACE;
            if (!aligned(workspace, 256)) return BGEMM_ERR_ALIGN;
            p.ws_counters = static_cast<unsigned int*>(workspace);
            p.ws_partial = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + 65536);
        }
    }
    return launch_gemm((cudaStream_t)stream, p, acts, bgemm_act_ld(K), batch);
}

int bgemm_gemm(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N, int op,
               void* out, int out_kind, int out_layout, const void* alpha, int split_k, void* workspace, size_t workspace_bytes,
               int64_t batch) {
    return gemm_entry(stream, plane, M, K, acts, colsum, N, op, out, out_kind, out_layout, alpha, split_k, workspace, workspace_bytes, batch, 0);
}

int bgemm_gemm_static_weights(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N,
                              int op, void* out, int out_kind, int out_layout, const void* alpha, int split_k, void* workspace,
                              size_t workspace_bytes, int64_t batch) {
    return gemm_entry(stream, plane, M, K, acts, colsum, N, op, out, out_kind, out_layout, alpha, split_k, workspace, workspace_bytes, batch,
                      BGEMM_FLAG_STATIC_WEIGHTS);
}

int bgemm_gemm_ex(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N, int op, void* out,
                  int out_kind, int out_layout, const void* alpha, int split_k, void* workspace, size_t workspace_bytes, int64_t batch, int flags) {
    return gemm_entry(stream, plane, M, K, acts, colsum, N, op, out, out_kind, out_layout, alpha, split_k, workspace, workspace_bytes, batch, flags);
}

int bgemm_gemm_multi_out(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N, int op,
                         void* const* outs_host, int n_outs, int64_t out_ld, int out_kind, int out_layout, const void* alpha, int split_k,
                         void* workspace, size_t workspace_bytes, int flags) {
    if (!outs_host || n_outs < 1 || n_outs > 8) return outs_host ? BGEMM_ERR_SHAPE : BGEMM_ERR_NULL;
    return gemm_entry(stream, plane, M, K, acts, colsum, N, op, outs_host[0], out_kind, out_layout, alpha, split_k, workspace, workspace_bytes, 1,
                      flags, outs_host + 1, n_outs - 1, out_ld);
}

int bgemm_w1a16_gemm(void* stream, const void* plane, int64_t M, int64_t K, const void* x_f16, int64_t x_ld, int64_t N, void* out, int out_kind,
                     int out_layout, const void* alpha, int weights_static) {
    if (!plane || !x_f16 || !out) return BGEMM_ERR_NULL;
    if ((out_kind != BGEMM_OUT_F32 && out_kind != BGEMM_OUT_F16) || out_layout < BGEMM_LAYOUT_NM || out_layout > BGEMM_LAYOUT_MN) return BGEMM_ERR_ENUM;
    if (M < 1 || N < 1 || K < 1 || M > kMaxDim || N > kMaxDim || K > kMaxDim || x_ld < K) return BGEMM_ERR_SHAPE;
    if (!aligned(plane, 16) || !aligned(x_f16, 2) || !aligned(out, out_kind == BGEMM_OUT_F32 ? 4 : 2)) return BGEMM_ERR_ALIGN;
    const int kblocks = (int)((K + 255) / 256);
    const int rows = w1a16_rows_per_launch(kblocks);
    if (rows < 1) return BGEMM_ERR_UNSUPPORTED;
    const size_t esz = out_kind == BGEMM_OUT_F32 ? 4 : 2;
    for (int64_t n0 = 0; n0 < N; n0 += rows) {
        GemmParams p{};
        p.plane = static_cast<const uint8_t*>(plane);
        // rows n0.. of an [N, M] result start n0 * M elements in; columns n0.. of an [M, N] result start n0 elements in
        p.out = static_cast<char*>(out) + esz * (size_t)(out_layout == BGEMM_LAYOUT_NM ? n0 * M : n0);
        p.alpha = static_cast<const __half*>(alpha);
        p.status = device_status_word();
        apply_test_hooks(p);
        p.M = (int)M; p.N = (int)(N - n0 < rows ? N - n0 : rows); p.K = (int)K;
        p.kblocks = kblocks;
        p.mtiles = (int)((M + 127) / 128);
        p.split_k = 1;
        p.out_kind = out_kind;
        p.out_layout = out_layout;
        p.ldo = out_layout == BGEMM_LAYOUT_NM ? M : N;
        p.plane_batch_bytes = (long long)bgemm_plane_bytes(M, K);
        p.weights_static = weights_static ? 1 : 0;
        const int rc = launch_gemm_w1a16((cudaStream_t)stream, p, static_cast<const __half*>(x_f16) + (size_t)n0 * x_ld, x_ld);
        if (rc) return rc;
    }
    return BGEMM_OK;
}

int bgemm_gemm_to_acts(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N, int op,
                       const void* alpha, int next_act_mode, int8_t* next_acts, int32_t* next_colsum, int split_k, void* workspace,
                       size_t workspace_bytes, int64_t batch) {
    return bgemm_gemm_to_acts_ex(stream, plane, M, K, acts, colsum, N, op, alpha, next_act_mode, next_acts, next_colsum, split_k, workspace,
                                 workspace_bytes, batch, 0);
}

int bgemm_gemm_to_acts_ex(void* stream, const void* plane, int64_t M, int64_t K, const int8_t* acts, const int32_t* colsum, int64_t N, int op,
                          const void* alpha, int next_act_mode, int8_t* next_acts, int32_t* next_colsum, int split_k, void* workspace,
                          size_t workspace_bytes, int64_t batch, int flags) {
    if (flags & ~(BGEMM_FLAG_STATIC_WEIGHTS | BGEMM_FLAG_SUMS_ZEROED)) return BGEMM_ERR_ENUM;
    if (!plane || !acts || !colsum || !next_acts || !next_colsum) return BGEMM_ERR_NULL;
    if (op < BGEMM_OP_AND || op > BGEMM_OP_BWTA || next_act_mode < BGEMM_ACT_SIGN || next_act_mode > BGEMM_ACT_NEG01) return BGEMM_ERR_ENUM;
    if (M < 1 || N < 1 || K < 1 || batch < 1 || batch > 65535 || M > kMaxDim || N > kMaxDim || K > kMaxDim || split_k < 0 ||
        split_k > kMaxSplitK)
        return BGEMM_ERR_SHAPE;
    if (!aligned(plane, 16) || !aligned(acts, 16) || !aligned(colsum, 4) || !aligned(next_acts, 16) || !aligned(next_colsum, 4))
        return BGEMM_ERR_ALIGN;
    const int s = resolve_split_k(M, N, K, batch, split_k);
    const long long mtiles = (M + 127) / 128;
    if (mtiles * s > 65535) return BGEMM_ERR_SHAPE;
    const long long ld = bgemm_act_ld(M);
    cudaStream_t st = (cudaStream_t)stream;
    // every check comes before the first memset or launch: a negative status means nothing was enqueued
    if (s > kMaxClusterSplit) {
        const size_t need = bgemm_gemm_workspace_bytes(M, N, K, s, batch);
        if (!workspace || workspace_bytes < need) return BGEMM_ERR_WORKSPACE;
        if (!aligned(workspace, 256)) return BGEMM_ERR_ALIGN;
    }
    // the kernel adds row sums with atomics and writes whole 8-column chunks: sums and the padding beyond them start at zero
    cudaError_t e = cudaSuccess;
    if (!(flags & BGEMM_FLAG_SUMS_ZEROED)) e = cudaMemsetAsync(next_colsum, 0, (size_t)N * (size_t)batch * sizeof(int32_t), st);
    const long long written = (M + 7) / 8 * 8;
    if (e == cudaSuccess && written < ld)
        e = cudaMemset2DAsync(next_acts + written, (size_t)ld, 0, (size_t)(ld - written), (size_t)N * (size_t)batch, st);
    if (e != cudaSuccess) return (int)e;

    GemmParams p{};
    p.plane = static_cast<const uint8_t*>(plane);
    p.colsum = colsum;
    p.out = next_acts;
    p.alpha = static_cast<const __half*>(alpha);
    p.status = device_status_word();
    apply_test_hooks(p);
#ifdef BGEMM_TUNING
    p.prof = debug_profile_buffer();
#endif
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.kblocks = (int)((K + 255) / 256);
    p.mtiles = (int)mtiles;
    p.split_k = s;
    p.epi = (op == BGEMM_OP_XOR || op == BGEMM_OP_BWTA) ? 1 : 0;
    p.out_kind = kOutActs;
    p.out_layout = BGEMM_LAYOUT_NM;
    p.ldo = M;
    p.plane_batch_bytes = (long long)bgemm_plane_bytes(M, K);
    p.cluster = (s > 1 && s <= kMaxClusterSplit) ? 1 : 0;
    p.colsum_next = next_colsum;
    p.out_ld = ld;
    p.act_mode = next_act_mode;
    p.weights_static = (flags & BGEMM_FLAG_STATIC_WEIGHTS) ? 1 : 0;
    if (s > kMaxClusterSplit) {
        const int NT = gemm_tile_n(M, N, K, batch);
        const long long tiles = mtiles * ((N + NT - 1) / NT) * batch;
        p.ws_counters = static_cast<unsigned int*>(workspace);
        p.ws_partial = reinterpret_cast<int32_t*>(static_cast<char*>(workspace) + counter_bytes(tiles));
    }
    return launch_gemm(st, p, acts, bgemm_act_ld(K), batch);
}

// Workspace of the unpacked-operand entry point: [gemm workspace][plane][acts int8][colsum].
static void linear_ws_layout(int64_t M, int64_t N, int64_t K, int s, size_t* off_plane, size_t* off_acts, size_t* off_colsum,
                             size_t* total) {
    // The counter prefix is reserved even when this call needs no counters, so that operands are never
    // parked where a later call on the same buffer expects zeroed counters.
    size_t o = align_up(bgemm_gemm_workspace_bytes(M, N, K, s, 1), 256);
    if (o < kCounterBytes) o = kCounterBytes;
    *off_plane = o; o += align_up(bgemm_plane_bytes(M, K), 256);
    *off_acts = o;  o += align_up((size_t)N * (size_t)bgemm_act_ld(K), 256);
    *off_colsum = o; o += align_up((size_t)N * 4, 256);
    *total = o;
}

size_t bgemm_linear_workspace_bytes(int64_t M, int64_t N, int64_t K, int split_k) {
    if (M < 1 || N < 1 || K < 1) return 0;
    const int s = resolve_split_k(M, N, K, 1, split_k);
    size_t a, b, c, total;
    linear_ws_layout(M, N, K, s, &a, &b, &c, &total);
    return total;
}

int bgemm_linear_forward(void* stream, const void* weight_f16, const void* acts_f16, void* out, int64_t M, int64_t N, int64_t K, int op,
                         int out_kind, int out_layout, const void* alpha, int split_k, void* workspace, size_t workspace_bytes) {
    if (!weight_f16 || !acts_f16 || !out || !workspace) return weight_f16 && acts_f16 && out ? BGEMM_ERR_WORKSPACE : BGEMM_ERR_NULL;
    if (op < BGEMM_OP_AND || op > BGEMM_OP_BWTA || out_kind < BGEMM_OUT_I32 || out_kind > BGEMM_OUT_F16_SCALED ||
        out_layout < BGEMM_LAYOUT_NM || out_layout > BGEMM_LAYOUT_MN)
        return BGEMM_ERR_ENUM;
    if (out_kind == BGEMM_OUT_F16_SCALED && !alpha) return BGEMM_ERR_NULL;
    if (M < 1 || N < 1 || K < 1 || M > kMaxDim || N > kMaxDim || K > kMaxDim || split_k < 0 || split_k > kMaxSplitK) return BGEMM_ERR_SHAPE;
    // everything the three calls below would refuse is refused here, before the first launch
    if (!aligned(workspace, 256) || !aligned(weight_f16, 2) || !aligned(acts_f16, 2) || !aligned(out, out_kind == BGEMM_OUT_I32 ? 4 : 2))
        return BGEMM_ERR_ALIGN;
    const int s = resolve_split_k(M, N, K, 1, split_k);
    if (((M + 127) / 128) * s > 65535) return BGEMM_ERR_SHAPE;
    size_t off_plane, off_acts, off_colsum, total;
    linear_ws_layout(M, N, K, s, &off_plane, &off_acts, &off_colsum, &total);
    if (workspace_bytes < total) return BGEMM_ERR_WORKSPACE;
    char* ws = static_cast<char*>(workspace);
    const int wbit = op == BGEMM_OP_ATTN ? BGEMM_WBIT_NONNEGATIVE : BGEMM_WBIT_NEGATIVE;
    const int amode = op == BGEMM_OP_AND ? BGEMM_ACT_NEG01 : (op == BGEMM_OP_BWTA ? BGEMM_ACT_TERNARY : BGEMM_ACT_SIGN);
    int rc = bgemm_pack_weights(stream, weight_f16, BGEMM_DT_F16, M, K, K, wbit, ws + off_plane, nullptr, nullptr, 1, 0);
    if (rc) return rc;
    rc = bgemm_prepare_acts(stream, acts_f16, BGEMM_DT_F16, N, K, K, amode, 0, reinterpret_cast<int8_t*>(ws + off_acts),
                            reinterpret_cast<int32_t*>(ws + off_colsum), 1, 0);
    if (rc) return rc;
    return bgemm_gemm(stream, ws + off_plane, M, K, reinterpret_cast<const int8_t*>(ws + off_acts),
                      reinterpret_cast<const int32_t*>(ws + off_colsum), N, op, out, out_kind, out_layout, alpha, s, ws,
                      bgemm_gemm_workspace_bytes(M, N, K, s, 1), 1);
}

}  // extern "C"
