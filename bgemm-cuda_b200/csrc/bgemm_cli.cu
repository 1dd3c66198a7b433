// Native benchmark / parity command line for libbgemm_b200.so.
//
//   bgemm_cli M K N SplitK [op]          one shape: weight rows, weight columns, batch size, K partitions (0 = auto),
//                                        op 1 = XOR (default), 0 = AND, 2 = ATTN, 3 = BWTA
//   bgemm_cli --sweep llama|opt [N]      the layer shapes of the llama-1 / OPT families at batch size N (default 128)
//
// Same arguments and the same report as the reference's CLI (lowbit_kernel/csrc/benchmark.cu:19-26 argv,
// :181-218 cuBLAS fp16 GEMM on the same mapped values as the yardstick, :344-350 and tests/cpp/kernel_test.h:48-66
// "Time/ms, Performance/TFLOPs, TotalAbsError/TotalAbsSum" lines); the sweeps are the shape lists of
// lowbit_kernel/run.sh:8-29. Reported for this library: the GEMM on prepared operands (weights packed once,
// activations prepared per call) and the drop-in call that packs both operands every time.
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/bgemm_b200.h"

#define CLI_CUDA(x)                                                                              \
    do {                                                                                         \
        cudaError_t e__ = (x);                                                                   \
        if (e__ != cudaSuccess) {                                                                \
            std::fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e__), __LINE__); \
            return 2;                                                                            \
        }                                                                                        \
    } while (0)
#define CLI_BGEMM(x)                                                                            \
    do {                                                                                        \
        int s__ = (x);                                                                          \
        if (s__ != 0) {                                                                         \
            std::fprintf(stderr, "bgemm error %d (%s) at line %d\n", s__, bgemm_status_string(s__), __LINE__); \
            return 3;                                                                           \
        }                                                                                       \
    } while (0)

namespace {

constexpr int kWarmup = 10, kIters = 100;

// The value a 16-bit float contributes to the product under `op`, as fp16 (what cuBLAS multiplies).
__global__ void map_operand(const __half* src, __half* dst, size_t n, int op, int is_weight) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned short bits = __half_as_ushort(src[i]);
        const int neg = bits >> 15, zero = (bits & 0x7fff) == 0;
        float v;
        if (op == BGEMM_OP_AND) v = (float)neg;
        else if (op == BGEMM_OP_ATTN) v = is_weight ? (float)(1 - neg) : (float)(1 - 2 * neg);
        else if (op == BGEMM_OP_BWTA) v = is_weight ? (float)(1 - 2 * neg) : (zero ? 0.f : (float)(1 - 2 * neg));
        else v = (float)(1 - 2 * neg);
        dst[i] = __float2half(v);
    }
}

double total_error(const std::vector<__half>& ref, const std::vector<__half>& got) {
    long double err = 0, sum = 0;
    for (size_t i = 0; i < ref.size(); i++) {
        err += std::fabs(__half2float(ref[i]) - __half2float(got[i]));
        sum += std::fabs(__half2float(ref[i]));
    }
    return sum > 0 ? (double)(err / sum) : (double)err;
}

void report(const char* name, float ms, double tflops, double error) {
    std::printf("%-22s \t -> \t\t Time/ms: %5.3f \t Performance/TFLOPs: %4.2f \t TotalAbsError/TotalAbsSum: %.8lf\n", name, ms, tflops, error);
}

int run_shape(long long M, long long K, long long N, int split_k, int op) {
    std::srand(1234);
    std::vector<__half> w_h((size_t)M * K), x_h((size_t)N * K);
    for (auto& v : w_h) v = __float2half((std::rand() % 100 - 50) / 17.0f);
    for (auto& v : x_h) {
        const int r = std::rand() % 100;
        v = __float2half(op == BGEMM_OP_BWTA ? (r < 30 ? 0.f : (r - 65) / 17.0f) : (r - 50) / 17.0f);
    }
    __half *w_d, *x_d, *wm_d, *xm_d, *ref_d, *out_d, *out2_d;
    CLI_CUDA(cudaMalloc(&w_d, w_h.size() * 2));
    CLI_CUDA(cudaMalloc(&x_d, x_h.size() * 2));
    CLI_CUDA(cudaMalloc(&wm_d, w_h.size() * 2));
    CLI_CUDA(cudaMalloc(&xm_d, x_h.size() * 2));
    CLI_CUDA(cudaMalloc(&ref_d, (size_t)M * N * 2));
    CLI_CUDA(cudaMalloc(&out_d, (size_t)M * N * 2));
    CLI_CUDA(cudaMalloc(&out2_d, (size_t)M * N * 2));
    CLI_CUDA(cudaMemcpy(w_d, w_h.data(), w_h.size() * 2, cudaMemcpyHostToDevice));
    CLI_CUDA(cudaMemcpy(x_d, x_h.data(), x_h.size() * 2, cudaMemcpyHostToDevice));
    map_operand<<<1024, 256>>>(w_d, wm_d, w_h.size(), op, 1);
    map_operand<<<1024, 256>>>(x_d, xm_d, x_h.size(), op, 0);
    CLI_CUDA(cudaGetLastError());

    cudaEvent_t e0, e1;
    CLI_CUDA(cudaEventCreate(&e0));
    CLI_CUDA(cudaEventCreate(&e1));
    const double flops = 2.0 * (double)M * (double)N * (double)K;

    // ---- cuBLAS: C[N, M] row-major = X[N, K] W[M, K]^T, i.e. column-major C^T[M, N] = W^T-as-col-major ... ----
    std::printf("Launching CuBlas...\n");
    cublasHandle_t handle;
    if (cublasCreate(&handle) != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasCreate failed\n"); return 4; }
    const float one = 1.f, zero = 0.f;
    auto cublas_once = [&]() {
        return cublasGemmEx(handle, CUBLAS_OP_T, CUBLAS_OP_N, (int)M, (int)N, (int)K, &one, wm_d, CUDA_R_16F, (int)K, xm_d, CUDA_R_16F, (int)K,
                            &zero, ref_d, CUDA_R_16F, (int)M, CUDA_R_32F, CUBLAS_GEMM_DEFAULT);
    };
    for (int i = 0; i < kWarmup; i++)
        if (cublas_once() != CUBLAS_STATUS_SUCCESS) { std::fprintf(stderr, "cublasGemmEx failed\n"); return 4; }
    CLI_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < kIters; i++) cublas_once();
    CLI_CUDA(cudaEventRecord(e1));
    CLI_CUDA(cudaEventSynchronize(e1));
    float ms_cublas = 0;
    CLI_CUDA(cudaEventElapsedTime(&ms_cublas, e0, e1));
    ms_cublas /= kIters;
    std::vector<__half> ref_h((size_t)M * N), got_h((size_t)M * N), got2_h((size_t)M * N);
    CLI_CUDA(cudaMemcpy(ref_h.data(), ref_d, ref_h.size() * 2, cudaMemcpyDeviceToHost));

    // ---- this library on prepared operands ----
    std::printf("Launching BGEMM...\n");
    const int wbit = op == BGEMM_OP_ATTN ? BGEMM_WBIT_NONNEGATIVE : BGEMM_WBIT_NEGATIVE;
    const int act_mode = op == BGEMM_OP_AND ? BGEMM_ACT_NEG01 : (op == BGEMM_OP_BWTA ? BGEMM_ACT_TERNARY : BGEMM_ACT_SIGN);
    void* plane;
    int8_t* acts;
    int32_t* colsum;
    CLI_CUDA(cudaMalloc(&plane, bgemm_plane_bytes(M, K)));
    CLI_CUDA(cudaMalloc(&acts, (size_t)N * (size_t)bgemm_act_ld(K)));
    CLI_CUDA(cudaMalloc(&colsum, (size_t)N * 4));
    const size_t ws_bytes = bgemm_linear_workspace_bytes(M, N, K, split_k) + bgemm_gemm_workspace_bytes(M, N, K, split_k, 1) + 256;
    void* ws;
    CLI_CUDA(cudaMalloc(&ws, ws_bytes));
    CLI_CUDA(cudaMemset(ws, 0, ws_bytes));
    // wide activation matrices: a balance workspace of its own (zeroed once, written by the library only) lets the
    // kernel split its work into exactly equal parts per SM pair
    const size_t bal_bytes = bgemm_gemm_workspace_bytes(M, N, K, split_k, 1) ? 0 : bgemm_gemm_balance_workspace_bytes(M, N, K, split_k, 1);
    void* bal = nullptr;
    if (bal_bytes) {
        CLI_CUDA(cudaMalloc(&bal, bal_bytes));
        CLI_CUDA(cudaMemset(bal, 0, bal_bytes));
    }
    CLI_CUDA(cudaEventRecord(e0));
    CLI_BGEMM(bgemm_pack_weights(nullptr, w_d, BGEMM_DT_F16, M, K, K, wbit, plane, nullptr, nullptr, 1, 0));
    CLI_CUDA(cudaEventRecord(e1));
    CLI_CUDA(cudaEventSynchronize(e1));
    float ms_pack = 0;
    CLI_CUDA(cudaEventElapsedTime(&ms_pack, e0, e1));
    auto prepared_once = [&]() -> int {
        int s = bgemm_prepare_acts(nullptr, x_d, BGEMM_DT_F16, N, K, K, act_mode, 0, acts, colsum, 1, 0);
        if (s) return s;
        if (bal_bytes)
            return bgemm_gemm_ex(nullptr, plane, M, K, acts, colsum, N, op, out_d, BGEMM_OUT_F16, BGEMM_LAYOUT_NM, nullptr, split_k, bal, bal_bytes, 1,
                                 BGEMM_FLAG_BALANCE_WORKSPACE);
        return bgemm_gemm(nullptr, plane, M, K, acts, colsum, N, op, out_d, BGEMM_OUT_F16, BGEMM_LAYOUT_NM, nullptr, split_k, ws, ws_bytes, 1);
    };
    for (int i = 0; i < kWarmup; i++) CLI_BGEMM(prepared_once());
    CLI_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < kIters; i++) prepared_once();
    CLI_CUDA(cudaEventRecord(e1));
    CLI_CUDA(cudaEventSynchronize(e1));
    float ms_prepared = 0;
    CLI_CUDA(cudaEventElapsedTime(&ms_prepared, e0, e1));
    ms_prepared /= kIters;
    CLI_CUDA(cudaMemcpy(got_h.data(), out_d, got_h.size() * 2, cudaMemcpyDeviceToHost));

    // ---- the drop-in call (packs weights and activations every time, like bin_pack_linear_kernel's callers) ----
    auto dropin_once = [&]() { return bgemm_linear_forward(nullptr, w_d, x_d, out2_d, M, N, K, op, BGEMM_OUT_F16, BGEMM_LAYOUT_NM, nullptr, split_k, ws, ws_bytes); };
    for (int i = 0; i < kWarmup; i++) CLI_BGEMM(dropin_once());
    CLI_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < kIters; i++) dropin_once();
    CLI_CUDA(cudaEventRecord(e1));
    CLI_CUDA(cudaEventSynchronize(e1));
    float ms_dropin = 0;
    CLI_CUDA(cudaEventElapsedTime(&ms_dropin, e0, e1));
    ms_dropin /= kIters;
    CLI_CUDA(cudaMemcpy(got2_h.data(), out2_d, got2_h.size() * 2, cudaMemcpyDeviceToHost));
    const int dev_status = bgemm_device_status(1);

    std::printf("Verifying correctness of the computations...\n");
    const double err1 = total_error(ref_h, got_h), err2 = total_error(ref_h, got2_h);
    std::printf("M: %lld N: %lld K: %lld SplitK: %d (resolved %d) Iter: %d  op: %d  weight prepack once: %.3f ms  device status: %d\n", M, N, K,
                split_k, split_k ? split_k : bgemm_gemm_auto_split_k(M, N, K, 1), kIters, op, ms_pack, dev_status);
    std::printf("******************************************Performance*******************************************\n");
    report("cuBLAS fp16", ms_cublas, flops / (ms_cublas * 1e-3) / 1e12, 0.0);
    report("BGEMM (prepacked W)", ms_prepared, flops / (ms_prepared * 1e-3) / 1e12, err1);
    report("BGEMM (drop-in)", ms_dropin, flops / (ms_dropin * 1e-3) / 1e12, err2);

    cublasDestroy(handle);
    cudaFree(w_d); cudaFree(x_d); cudaFree(wm_d); cudaFree(xm_d); cudaFree(ref_d); cudaFree(out_d); cudaFree(out2_d);
    cudaFree(plane); cudaFree(acts); cudaFree(colsum); cudaFree(ws); cudaFree(bal);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return (err1 == 0.0 && err2 == 0.0 && dev_status == 0) ? 0 : 1;
}

struct Shape { long long M, K; };
// layer shapes listed in lowbit_kernel/run.sh (weight rows, weight columns)
const Shape kLlama[] = {{12288, 4096}, {4096, 4096}, {11008, 4096}, {4096, 11008}, {15360, 5120}, {5120, 5120}, {13824, 5120}, {5120, 13824},
                        {19968, 6656}, {6656, 6656}, {17920, 6656}, {6656, 17920}, {24576, 8192}, {8192, 8192}, {22016, 8192}, {8192, 22016}};
const Shape kOpt[] = {{21504, 7168}, {7168, 7168}, {28672, 7168}, {7168, 28672}, {27648, 9216}, {9216, 9216}, {36864, 9216}, {9216, 36864},
                      {36864, 12288}, {12288, 12288}, {49152, 12288}, {12288, 49152}};

}  // namespace

int main(int argc, char** argv) {
    if (argc >= 3 && std::strcmp(argv[1], "--sweep") == 0) {
        const bool llama = std::strcmp(argv[2], "llama") == 0;
        if (!llama && std::strcmp(argv[2], "opt") != 0) { std::printf("unknown sweep %s (llama | opt)\n", argv[2]); return -1; }
        const long long N = argc >= 4 ? std::atoll(argv[3]) : 128;
        const Shape* shapes = llama ? kLlama : kOpt;
        const int count = llama ? (int)(sizeof(kLlama) / sizeof(Shape)) : (int)(sizeof(kOpt) / sizeof(Shape));
        int worst = 0;
        for (int i = 0; i < count; i++) {
            std::printf("Processing Shape %d...\nBS=%lld\n", i, N);
            const int rc = run_shape(shapes[i].M, shapes[i].K, N, 0, BGEMM_OP_XOR);
            if (rc > worst) worst = rc;
        }
        return worst;
    }
    if (argc != 5 && argc != 6) {
        std::printf("Wrong Inputs! Correct input format: %s #Row_Weight #Column_Weight BatchSize SplitK [op]\n"
                    "                         or: %s --sweep llama|opt [BatchSize]\n", argv[0], argv[0]);
        return -1;
    }
    const long long M = std::atoll(argv[1]), K = std::atoll(argv[2]), N = std::atoll(argv[3]);
    const int split_k = std::atoi(argv[4]);
    const int op = argc == 6 ? std::atoi(argv[5]) : BGEMM_OP_XOR;
    if (M < 1 || K < 1 || N < 1 || split_k < 0 || op < BGEMM_OP_AND || op > BGEMM_OP_BWTA) { std::printf("bad arguments\n"); return -1; }
    return run_shape(M, K, N, split_k, op);
}
