// bgemm_linear_forward_noalloc: the unpacked-operand linear forward for callers that have no way to hand the
// library a scratch buffer. Its scratch (packed weight plane, int8 activations, column sums) lives in a
// fixed-size array in device global memory that is part of the library image.
#include "internal.h"

namespace {

constexpr size_t kScratchBytes = BGEMM_NOALLOC_SCRATCH_BYTES;

// Every GPU that loads the library carries this array until the process exits.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

// In host code `g_noalloc_scratch` is only a handle for the runtime, never an address a kernel may be given.
// The device address is looked up once per device, with that device current, and cached.
unsigned char* scratch_of_current_device(int* status) {
    static unsigned char* cache[64] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { *status = (int)e; return nullptr; }
    if (dev < 0 || dev >= 64) { *status = BGEMM_ERR_UNSUPPORTED; return nullptr; }
    // Host threads may race on a cache slot: harmless, every thread computes and stores the same address.
    if (!cache[dev]) {
        unsigned char* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) { *status = e != cudaSuccess ? (int)e : BGEMM_ERR_DRIVER; return nullptr; }
        cache[dev] = ptr;
    }
    *status = BGEMM_OK;
    return cache[dev];
}

}  // namespace

extern "C" int bgemm_linear_forward_noalloc(void* stream, const void* weight_f16, const void* acts_f16, void* out, int64_t M, int64_t N,
                                            int64_t K, int op, int out_kind, int out_layout, const void* alpha) {
    if (!weight_f16 || !acts_f16 || !out) return BGEMM_ERR_NULL;
    if (M < 1 || N < 1 || K < 1) return BGEMM_ERR_SHAPE;
    // K partitions are left to the library, which never picks more than 8: those reduce on chip, so no part of the
    // scratch has to start at zero and nothing of a previous call can leak into this one (plane, activations and
    // column sums are rewritten in full, padding included, before the GEMM reads them).
    const size_t need = bgemm_linear_workspace_bytes(M, N, K, 0);
    if (need == 0 || need > kScratchBytes) return BGEMM_ERR_TOO_LARGE;
    int status = BGEMM_OK;
    unsigned char* scratch = scratch_of_current_device(&status);
    if (!scratch) return status;
    return bgemm_linear_forward(stream, weight_f16, acts_f16, out, M, N, K, op, out_kind, out_layout, alpha, 0, scratch, kScratchBytes);
}
