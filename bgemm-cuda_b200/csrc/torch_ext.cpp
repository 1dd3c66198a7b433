// Python module `lowbit_kernel`: the reference's extension surface (lowbit_kernel/csrc/pybind.cpp:7-13)
// as a thin torch wrapper over the C ABI of libbgemm_b200.so. Tensors in, tensors out; every
// computation is one or more calls declared in include/bgemm_b200.h on torch's current stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <algorithm>

#include "../../include/bgemm_b200.h"

namespace {

void check(int status, const char* where) {
    TORCH_CHECK(status == 0, where, ": status ", status, ": ", bgemm_status_string(status));
}

int dtype_code(const torch::Tensor& t) {
    switch (t.scalar_type()) {
        case at::kHalf: return BGEMM_DT_F16;
        case at::kBFloat16: return BGEMM_DT_BF16;
        case at::kFloat: return BGEMM_DT_F32;
        case at::kChar: return BGEMM_DT_I8;
        default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type(), ": use float16, bfloat16, float32 or int8");
    }
}

void* stream_of(const torch::Tensor& t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// Scratch for one call, taken from torch's caching allocator on the current stream: stream-ordered like every other
// temporary of the call (the reference's wrapper does the same, fp6_linear.cu:580-586), so calls on different streams
// or threads never share operands. Only launches with more than 8 K partitions keep arrival counters in the first
// 64 KiB, which must start at zero: `zero_counters` clears just that prefix.
torch::Tensor workspace(const torch::Device& dev, size_t bytes, bool zero_counters) {
    auto ws = torch::empty({(int64_t)std::max<size_t>(bytes, 256)}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
    if (zero_counters) ws.narrow(0, 0, std::min<int64_t>(ws.numel(), 64 * 1024)).zero_();
    return ws;
}

int act_mode_of(int op) { return op == BGEMM_OP_AND ? BGEMM_ACT_NEG01 : (op == BGEMM_OP_BWTA ? BGEMM_ACT_TERNARY : BGEMM_ACT_SIGN); }

// reference: bgemm_linear_forward_cuda(in_feats[N,K] half, weights[M,K] half, splitK=1, INSTR=1) -> [N,M] half
// (lowbit_kernel/csrc/fp6_linear.cu:561-616). Differences: any M, N, K; runs on the current stream; splitK <= 1
// lets the library pick the K partitioning (results do not depend on it); non-contiguous inputs are made
// contiguous instead of being read as if they were.
torch::Tensor bgemm_linear_forward_cuda(torch::Tensor in_feats, torch::Tensor weights, int64_t splitK, int64_t INSTR) {
    TORCH_CHECK(in_feats.is_cuda() && weights.is_cuda(), "bgemm_linear_forward_cuda: CUDA tensors required (no CPU path)");
    TORCH_CHECK(in_feats.dim() == 2 && weights.dim() == 2, "bgemm_linear_forward_cuda: 2-D tensors required");
    TORCH_CHECK(in_feats.size(1) == weights.size(1), "bgemm_linear_forward_cuda: K mismatch");
    TORCH_CHECK(INSTR >= 0 && INSTR <= 3, "bgemm_linear_forward_cuda: INSTR must be 0 (and), 1 (xor), 2 (attn) or 3 (bwta)");
    c10::cuda::CUDAGuard guard(in_feats.device());
    auto x = in_feats.to(at::kHalf).contiguous();
    auto w = weights.to(at::kHalf).contiguous();
    const int64_t N = x.size(0), K = x.size(1), M = w.size(0);
    auto out = torch::empty({N, M}, x.options());
    const int sk = splitK <= 1 ? 0 : (int)splitK;
    const size_t need = bgemm_linear_workspace_bytes(M, N, K, sk);
    auto ws = workspace(x.device(), need, bgemm_gemm_workspace_bytes(M, N, K, sk, 1) > 0);
    check(bgemm_linear_forward(stream_of(x), w.data_ptr(), x.data_ptr(), out.data_ptr(), M, N, K, (int)INSTR, BGEMM_OUT_F16,
                               BGEMM_LAYOUT_NM, nullptr, sk, ws.data_ptr(), (size_t)ws.numel()),
          "bgemm_linear_forward");
    return out;
}

// The reference's GPU prepack entry (fp6_linear.cu:519-542) returned an uninitialised tensor; this one
// packs. Returns the tiled 1-bit plane as a uint8 tensor. wbit_mode: 0 bit = sign bit, 1 bit = !sign bit
// (ATTN mask slot), 2 bit = (w != 0), 3 bit = (w < 0) with -0.0 -> 0 (planes of a ternary matrix).
torch::Tensor binary_weight_prepacking_cuda(torch::Tensor w, int64_t wbit_mode) {
    TORCH_CHECK(w.is_cuda() && (w.dim() == 2 || w.dim() == 3), "binary_weight_prepacking_cuda: 2-D or 3-D CUDA tensor required");
    c10::cuda::CUDAGuard guard(w.device());
    if (w.stride(-1) != 1) w = w.contiguous();
    const bool batched = w.dim() == 3;
    const int64_t B = batched ? w.size(0) : 1, M = w.size(-2), K = w.size(-1);
    auto plane = torch::empty({(int64_t)(B * bgemm_plane_bytes(M, K))}, torch::TensorOptions().dtype(torch::kUInt8).device(w.device()));
    check(bgemm_pack_weights(stream_of(w), w.data_ptr(), dtype_code(w), M, K, w.stride(-2), (int)wbit_mode, plane.data_ptr(), nullptr,
                             nullptr, B, batched ? w.stride(0) : 0),
          "bgemm_pack_weights");
    return plane;
}

// Same plus the per-row scale alpha[m] = mean |w[m,:]| (fp16) and the per-row bit count.
std::vector<torch::Tensor> binary_weight_prepacking_scaled_cuda(torch::Tensor w) {
    TORCH_CHECK(w.is_cuda() && w.dim() == 2, "binary_weight_prepacking_scaled_cuda: 2-D CUDA tensor required");
    c10::cuda::CUDAGuard guard(w.device());
    if (w.stride(-1) != 1) w = w.contiguous();
    const int64_t M = w.size(0), K = w.size(1);
    auto plane = torch::empty({(int64_t)bgemm_plane_bytes(M, K)}, torch::TensorOptions().dtype(torch::kUInt8).device(w.device()));
    auto alpha = torch::empty({M}, torch::TensorOptions().dtype(at::kHalf).device(w.device()));
    auto rowpop = torch::empty({M}, torch::TensorOptions().dtype(at::kInt).device(w.device()));
    check(bgemm_pack_weights(stream_of(w), w.data_ptr(), dtype_code(w), M, K, w.stride(0), 0, plane.data_ptr(), rowpop.data_ptr<int>(),
                             alpha.data_ptr(), 1, 0),
          "bgemm_pack_weights");
    return {plane, alpha, rowpop};
}

// ---- packed-weight bundle: header (magic, layout version, M, K, bit mode, offsets) + plane + rowpop + alpha in ONE
// uint8 tensor, so that a saved layer carries its own description (see bgemm_bundle_* in the C header).
struct BundleViews {
    int64_t M, K;
    int wbit_mode;
    torch::Tensor plane, rowpop, alpha;
};

// Validates the header (64 bytes are copied to the host when the bundle lives on a GPU) and returns views of the parts.
BundleViews open_bundle(const torch::Tensor& bundle) {
    TORCH_CHECK(bundle.scalar_type() == at::kByte && bundle.dim() == 1 && bundle.is_contiguous() && bundle.numel() >= BGEMM_BUNDLE_HEADER_BYTES,
                "packed-weight bundle: a contiguous 1-D uint8 tensor is required");
    auto head = bundle.narrow(0, 0, BGEMM_BUNDLE_HEADER_BYTES).cpu();
    BundleViews v;
    size_t po = 0, ro = 0, ao = 0;
    const int rc = bgemm_bundle_parse_host(head.data_ptr(), (size_t)bundle.numel(), &v.M, &v.K, &v.wbit_mode, &po, &ro, &ao);
    TORCH_CHECK(rc == 0, "packed-weight bundle: ", rc == BGEMM_ERR_UNSUPPORTED ? "unknown magic or layout version (this library reads version " : "inconsistent header (",
                BGEMM_LAYOUT_VERSION, ")");
    v.plane = bundle.narrow(0, (int64_t)po, (int64_t)bgemm_plane_bytes(v.M, v.K));
    v.rowpop = bundle.narrow(0, (int64_t)ro, v.M * 4).view(at::kInt);
    v.alpha = bundle.narrow(0, (int64_t)ao, v.M * 2).view(at::kHalf);
    return v;
}

torch::Tensor new_bundle(const torch::Device& dev, int64_t M, int64_t K, int wbit_mode) {
    const size_t bytes = bgemm_bundle_bytes(M, K);
    TORCH_CHECK(bytes > 0, "packed-weight bundle: bad shape");
    auto head = torch::zeros({BGEMM_BUNDLE_HEADER_BYTES}, torch::TensorOptions().dtype(torch::kUInt8));
    check(bgemm_bundle_header_host(head.data_ptr(), M, K, wbit_mode), "bgemm_bundle_header_host");
    auto bundle = torch::zeros({(int64_t)bytes}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
    bundle.narrow(0, 0, BGEMM_BUNDLE_HEADER_BYTES).copy_(head);
    return bundle;
}

// `weight_prepacking_cpu` keeps the reference's export name (pybind.cpp:10); its FP6 meaning is out of scope, so it is
// the binary prepack on the CPU: [OC, IC] CPU tensor -> packed-weight bundle (uint8, CPU): header, tiled bit plane,
// per-row bit counts, per-row mean-abs scales. `unpack_bundle` gives the parts.
torch::Tensor weight_prepacking_cpu(torch::Tensor w) {
    TORCH_CHECK(!w.is_cuda() && w.dim() == 2, "weight_prepacking_cpu: 2-D CPU tensor required");
    w = w.contiguous();
    const int64_t M = w.size(0), K = w.size(1);
    auto bundle = new_bundle(w.device(), M, K, BGEMM_WBIT_NEGATIVE);
    auto v = open_bundle(bundle);
    check(bgemm_pack_weights_host(w.data_ptr(), dtype_code(w), M, K, K, BGEMM_WBIT_NEGATIVE, v.plane.data_ptr(), v.rowpop.data_ptr<int>(),
                                  v.alpha.data_ptr()),
          "bgemm_pack_weights_host");
    return bundle;
}

// The same on the GPU (one prepack launch).
torch::Tensor binary_weight_prepacking_bundle_cuda(torch::Tensor w, int64_t wbit_mode) {
    TORCH_CHECK(w.is_cuda() && w.dim() == 2, "binary_weight_prepacking_bundle_cuda: 2-D CUDA tensor required");
    c10::cuda::CUDAGuard guard(w.device());
    if (w.stride(-1) != 1) w = w.contiguous();
    const int64_t M = w.size(0), K = w.size(1);
    auto bundle = new_bundle(w.device(), M, K, (int)wbit_mode);
    auto v = open_bundle(bundle);
    check(bgemm_pack_weights(stream_of(w), w.data_ptr(), dtype_code(w), M, K, w.stride(0), (int)wbit_mode, v.plane.data_ptr(),
                             v.rowpop.data_ptr<int>(), v.alpha.data_ptr(), 1, 0),
          "bgemm_pack_weights");
    return bundle;
}

// (plane uint8, alpha fp16 [M], rowpop int32 [M], M, K, wbit_mode): views into the bundle, header validated first.
py::tuple unpack_bundle(torch::Tensor bundle) {
    auto v = open_bundle(bundle);
    return py::make_tuple(v.plane, v.alpha, v.rowpop, v.M, v.K, v.wbit_mode);
}

// The reference's row-major format (binary_matrix_prepacking_cpu, fp6_linear.cu:463-485): int32 [rows, K/32],
// element k at bit 31 - k % 32. Works on CPU and CUDA tensors.
torch::Tensor binary_matrix_prepacking(torch::Tensor w) {
    TORCH_CHECK(w.dim() == 2 && w.size(1) % 32 == 0, "binary_matrix_prepacking: [rows, K] with K % 32 == 0 required");
    w = w.contiguous();
    const int64_t rows = w.size(0), K = w.size(1);
    auto out = torch::empty({rows, K / 32}, torch::TensorOptions().dtype(at::kInt).device(w.device()));
    if (w.is_cuda()) {
        c10::cuda::CUDAGuard guard(w.device());
        check(bgemm_pack_rowmajor_msb(stream_of(w), w.data_ptr(), dtype_code(w), rows, K, K, reinterpret_cast<uint32_t*>(out.data_ptr<int>())),
              "bgemm_pack_rowmajor_msb");
    } else {
        check(bgemm_pack_rowmajor_msb_host(w.data_ptr(), dtype_code(w), rows, K, K, reinterpret_cast<uint32_t*>(out.data_ptr<int>())),
              "bgemm_pack_rowmajor_msb_host");
    }
    return out;
}

// Activation prepare: [N, K] (or [B, N, K]; with transpose the matrices are [K, N]) -> (int8 rows, colsum).
std::vector<torch::Tensor> prepare_acts(torch::Tensor x, int64_t act_mode, bool transpose) {
    TORCH_CHECK(x.is_cuda() && (x.dim() == 2 || x.dim() == 3), "prepare_acts: 2-D or 3-D CUDA tensor required");
    c10::cuda::CUDAGuard guard(x.device());
    if (x.stride(-1) != 1) x = x.contiguous();
    const bool batched = x.dim() == 3;
    const int64_t B = batched ? x.size(0) : 1;
    const int64_t N = transpose ? x.size(-1) : x.size(-2), K = transpose ? x.size(-2) : x.size(-1);
    std::vector<int64_t> ashape = batched ? std::vector<int64_t>{B, N, bgemm_act_ld(K)} : std::vector<int64_t>{N, bgemm_act_ld(K)};
    std::vector<int64_t> cshape = batched ? std::vector<int64_t>{B, N} : std::vector<int64_t>{N};
    auto acts = torch::empty(ashape, torch::TensorOptions().dtype(at::kChar).device(x.device()));
    auto colsum = torch::empty(cshape, torch::TensorOptions().dtype(at::kInt).device(x.device()));
    check(bgemm_prepare_acts(stream_of(x), x.data_ptr(), dtype_code(x), N, K, x.stride(-2), (int)act_mode, transpose ? 1 : 0,
                             acts.data_ptr<int8_t>(), colsum.data_ptr<int>(), B, batched ? x.stride(0) : 0),
          "bgemm_prepare_acts");
    return {acts, colsum};
}

// GEMM on prepared operands (see bgemm_gemm). out_kind: 0 int32, 1 fp16, 2 fp16 scaled by alpha[m].
// static_weights: the caller promises that `plane` was complete before the previous kernel of the current stream was launched
// (see bgemm_gemm_static_weights).
torch::Tensor gemm_prepared(torch::Tensor plane, int64_t M, int64_t K, torch::Tensor acts, torch::Tensor colsum, int64_t op,
                            int64_t out_kind, int64_t out_layout, c10::optional<torch::Tensor> alpha, int64_t splitK, bool static_weights) {
    TORCH_CHECK(plane.is_cuda() && acts.is_cuda() && colsum.is_cuda(), "gemm_prepared: CUDA tensors required");
    TORCH_CHECK(acts.is_contiguous() && colsum.is_contiguous() && plane.is_contiguous(), "gemm_prepared: contiguous tensors required");
    TORCH_CHECK(acts.scalar_type() == at::kChar && colsum.scalar_type() == at::kInt, "gemm_prepared: acts int8 / colsum int32 required");
    TORCH_CHECK(acts.size(-1) == bgemm_act_ld(K), "gemm_prepared: activation row pitch must be bgemm_act_ld(K)");
    c10::cuda::CUDAGuard guard(acts.device());
    const bool batched = acts.dim() == 3;
    const int64_t B = batched ? acts.size(0) : 1, N = acts.size(-2);
    TORCH_CHECK((size_t)plane.numel() >= (size_t)B * bgemm_plane_bytes(M, K), "gemm_prepared: plane too small for M, K");
    std::vector<int64_t> shape = out_layout == BGEMM_LAYOUT_NM ? std::vector<int64_t>{N, M} : std::vector<int64_t>{M, N};
    if (batched) shape.insert(shape.begin(), B);
    auto out = torch::empty(shape, torch::TensorOptions().dtype(out_kind == BGEMM_OUT_I32 ? at::kInt : at::kHalf).device(acts.device()));
    const void* alpha_ptr = nullptr;
    torch::Tensor a;
    if (alpha.has_value()) {
        a = alpha->to(at::kHalf).contiguous();
        TORCH_CHECK(a.is_cuda() && a.numel() == B * M, "gemm_prepared: alpha must hold M values per batch on the GPU");
        alpha_ptr = a.data_ptr();
    }
    const size_t need = bgemm_gemm_workspace_bytes(M, N, K, (int)splitK, B);
    torch::Tensor ws;
    if (need) ws = workspace(acts.device(), need, true);
    check((static_weights ? bgemm_gemm_static_weights : bgemm_gemm)(stream_of(acts), plane.data_ptr(), M, K, acts.data_ptr<int8_t>(),
                                                                     colsum.data_ptr<int>(), N, (int)op, out.data_ptr(), (int)out_kind, (int)out_layout,
                                                                     alpha_ptr, (int)splitK, need ? ws.data_ptr() : nullptr,
                                                                     need ? (size_t)ws.numel() : 0, B),
          "bgemm_gemm");
    return out;
}

// GEMM on prepared operands whose result becomes the next layer's prepared activations (see bgemm_gemm_to_acts):
// returns (int8 [N, act_ld(M)], colsum int32 [N]) = prepare_acts(fp16 result, next_act_mode) without the round trip.
// `sums` (optional): an int32 tensor of the row sums' shape that the caller has ZEROED on the current stream; it receives the
// row sums and is returned as the second result, and the library skips its own memset (see BGEMM_FLAG_SUMS_ZEROED).
std::vector<torch::Tensor> gemm_prepared_to_acts(torch::Tensor plane, int64_t M, int64_t K, torch::Tensor acts, torch::Tensor colsum,
                                                 int64_t op, int64_t next_act_mode, c10::optional<torch::Tensor> alpha, int64_t splitK,
                                                 c10::optional<torch::Tensor> sums) {
    TORCH_CHECK(plane.is_cuda() && acts.is_cuda() && colsum.is_cuda(), "gemm_prepared_to_acts: CUDA tensors required");
    TORCH_CHECK(acts.is_contiguous() && colsum.is_contiguous() && plane.is_contiguous(), "gemm_prepared_to_acts: contiguous tensors required");
    TORCH_CHECK(acts.scalar_type() == at::kChar && colsum.scalar_type() == at::kInt, "gemm_prepared_to_acts: acts int8 / colsum int32 required");
    TORCH_CHECK(acts.size(-1) == bgemm_act_ld(K), "gemm_prepared_to_acts: activation row pitch must be bgemm_act_ld(K)");
    c10::cuda::CUDAGuard guard(acts.device());
    const bool batched = acts.dim() == 3;
    const int64_t B = batched ? acts.size(0) : 1, N = acts.size(-2);
    TORCH_CHECK((size_t)plane.numel() >= (size_t)B * bgemm_plane_bytes(M, K), "gemm_prepared_to_acts: plane too small for M, K");
    std::vector<int64_t> ashape = batched ? std::vector<int64_t>{B, N, bgemm_act_ld(M)} : std::vector<int64_t>{N, bgemm_act_ld(M)};
    std::vector<int64_t> cshape = batched ? std::vector<int64_t>{B, N} : std::vector<int64_t>{N};
    auto next_acts = torch::empty(ashape, torch::TensorOptions().dtype(at::kChar).device(acts.device()));
    torch::Tensor next_colsum;
    if (sums.has_value()) {
        next_colsum = *sums;
        TORCH_CHECK(next_colsum.is_cuda() && next_colsum.device() == acts.device() && next_colsum.scalar_type() == at::kInt &&
                        next_colsum.is_contiguous() && next_colsum.numel() == B * N,
                    "gemm_prepared_to_acts: sums must be a contiguous int32 CUDA tensor with one value per activation row");
    } else {
        next_colsum = torch::empty(cshape, torch::TensorOptions().dtype(at::kInt).device(acts.device()));
    }
    const void* alpha_ptr = nullptr;
    torch::Tensor a;
    if (alpha.has_value()) {
        a = alpha->to(at::kHalf).contiguous();
        TORCH_CHECK(a.is_cuda() && a.numel() == B * M, "gemm_prepared_to_acts: alpha must hold M values per batch on the GPU");
        alpha_ptr = a.data_ptr();
    }
    const size_t need = bgemm_gemm_workspace_bytes(M, N, K, (int)splitK, B);
    torch::Tensor ws;
    if (need) ws = workspace(acts.device(), need, true);
    check(bgemm_gemm_to_acts_ex(stream_of(acts), plane.data_ptr(), M, K, acts.data_ptr<int8_t>(), colsum.data_ptr<int>(), N, (int)op, alpha_ptr,
                                (int)next_act_mode, next_acts.data_ptr<int8_t>(), next_colsum.data_ptr<int>(), (int)splitK,
                                need ? ws.data_ptr() : nullptr, need ? (size_t)ws.numel() : 0, B, sums.has_value() ? BGEMM_FLAG_SUMS_ZEROED : 0),
          "bgemm_gemm_to_acts");
    return {next_acts, sums.has_value() ? next_colsum.view(cshape) : next_colsum};
}

// x [N, K] unpacked x prepacked weights -> [N, M]. INSTR as in the reference; out_kind 1 = fp16, 0 = int32,
// 2 = fp16 scaled by alpha (required then).
torch::Tensor bgemm_linear_forward_packed(torch::Tensor x, torch::Tensor plane, int64_t M, int64_t K, c10::optional<torch::Tensor> alpha,
                                          int64_t splitK, int64_t INSTR, int64_t out_kind, bool static_weights) {
    TORCH_CHECK(x.dim() == 2 && x.size(1) == K, "bgemm_linear_forward_packed: x must be [N, K]");
    auto prep = prepare_acts(x, act_mode_of((int)INSTR), false);
    return gemm_prepared(plane, M, K, prep[0], prep[1], INSTR, out_kind, BGEMM_LAYOUT_NM, alpha, splitK, static_weights);
}

// Binary weight x ternary activation with the per-channel scale fused: fp16 [N, M] = sign(x) . sign(w)^T * alpha.
torch::Tensor bwta_linear_forward_cuda(torch::Tensor x, torch::Tensor plane, int64_t M, int64_t K, torch::Tensor alpha, int64_t splitK) {
    return bgemm_linear_forward_packed(x, plane, M, K, alpha, splitK, BGEMM_OP_BWTA, BGEMM_OUT_F16_SCALED, false);
}

// Batched {0,1} x {-1,+1} attention product: attn [B, Sq, Sk] ("1" = sign bit clear, as the reference
// encodes it), value [B, Sk, d] -> [B, Sq, d]; int32 when exact is true, else fp16 like the reference op.
torch::Tensor bgemm_attn_matmul_batched(torch::Tensor attn, torch::Tensor value, bool exact) {
    TORCH_CHECK(attn.is_cuda() && value.is_cuda() && attn.dim() == 3 && value.dim() == 3, "bgemm_attn_matmul_batched: 3-D CUDA tensors required");
    TORCH_CHECK(attn.size(0) == value.size(0) && attn.size(2) == value.size(1), "bgemm_attn_matmul_batched: shape mismatch");
    const int64_t Sq = attn.size(1), Sk = attn.size(2);
    auto plane = binary_weight_prepacking_cuda(attn, BGEMM_WBIT_NONNEGATIVE);
    auto prep = prepare_acts(value, BGEMM_ACT_SIGN, true);
    return gemm_prepared(plane, Sq, Sk, prep[0], prep[1], BGEMM_OP_ATTN, exact ? BGEMM_OUT_I32 : BGEMM_OUT_F16, BGEMM_LAYOUT_MN, c10::nullopt, 0, false);
}

// Binary weight x fp16 activation ("W1A16"): x fp16 [N, K] (as it is, no activation pass) x prepacked plane -> [N, M],
// fp32 accumulation; fp32 result when out_f32, else fp16. alpha (optional): per-output-channel scale.
torch::Tensor w1a16_linear_forward(torch::Tensor x, torch::Tensor plane, int64_t M, int64_t K, c10::optional<torch::Tensor> alpha, bool out_f32,
                                   bool static_weights) {
    TORCH_CHECK(x.is_cuda() && plane.is_cuda() && x.dim() == 2 && x.size(1) == K, "w1a16_linear_forward: x must be a CUDA tensor [N, K]");
    TORCH_CHECK((size_t)plane.numel() >= bgemm_plane_bytes(M, K), "w1a16_linear_forward: plane too small for M, K");
    c10::cuda::CUDAGuard guard(x.device());
    auto xh = x.to(at::kHalf);
    if (xh.stride(1) != 1) xh = xh.contiguous();
    const int64_t N = xh.size(0);
    auto out = torch::empty({N, M}, torch::TensorOptions().dtype(out_f32 ? at::kFloat : at::kHalf).device(x.device()));
    const void* alpha_ptr = nullptr;
    torch::Tensor a;
    if (alpha.has_value()) {
        a = alpha->to(at::kHalf).contiguous();
        TORCH_CHECK(a.is_cuda() && a.numel() == M, "w1a16_linear_forward: alpha must hold M values on the GPU");
        alpha_ptr = a.data_ptr();
    }
    check(bgemm_w1a16_gemm(stream_of(x), plane.data_ptr(), M, K, xh.data_ptr(), xh.stride(0), N, out.data_ptr(), out_f32 ? BGEMM_OUT_F32 : BGEMM_OUT_F16,
                           BGEMM_LAYOUT_NM, alpha_ptr, static_weights ? 1 : 0),
          "bgemm_w1a16_gemm");
    return out;
}

torch::Tensor fp6_not_provided(py::args, py::kwargs) {
    throw py::type_error("the FP6 entry points of the reference (linear_forward_cuda, weight_dequant_cpu) are not part of this library");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("bgemm_linear_forward_cuda", &bgemm_linear_forward_cuda, "Computes BGEMM.", py::arg("in_feats"), py::arg("weights"),
          py::arg("splitK") = 1, py::arg("INSTR") = 1);
    m.def("weight_prepacking_cpu", &weight_prepacking_cpu, "Binary weight prepacking on the CPU: packed-weight bundle (header, plane, rowpop, alpha).");
    m.def("binary_weight_prepacking_bundle_cuda", &binary_weight_prepacking_bundle_cuda, "Binary weight prepacking on the GPU: packed-weight bundle.",
          py::arg("w"), py::arg("wbit_mode") = 0);
    m.def("unpack_bundle", &unpack_bundle, "Validate a packed-weight bundle's header and return (plane, alpha, rowpop, M, K, wbit_mode) views.");
    m.attr("LAYOUT_VERSION") = (int)BGEMM_LAYOUT_VERSION;
    m.def("binary_weight_prepacking_cuda", &binary_weight_prepacking_cuda, "Binary weight prepacking on the GPU.", py::arg("w"),
          py::arg("wbit_mode") = 0);
    m.def("binary_weight_prepacking_scaled_cuda", &binary_weight_prepacking_scaled_cuda, "Prepack + per-row mean-abs scale + bit count.");
    m.def("binary_matrix_prepacking", &binary_matrix_prepacking, "Row-major MSB-first prepack (the reference's packed format).");
    m.def("prepare_acts", &prepare_acts, "Activations -> int8 rows + column sums.", py::arg("x"), py::arg("act_mode"),
          py::arg("transpose") = false);
    m.def("gemm_prepared", &gemm_prepared, "GEMM on prepared operands.", py::arg("plane"), py::arg("M"), py::arg("K"), py::arg("acts"),
          py::arg("colsum"), py::arg("op"), py::arg("out_kind") = 0, py::arg("out_layout") = 0, py::arg("alpha") = py::none(),
          py::arg("splitK") = 0, py::arg("static_weights") = false);
    m.def("gemm_prepared_to_acts", &gemm_prepared_to_acts, "GEMM whose result becomes the next layer's prepared activations.", py::arg("plane"),
          py::arg("M"), py::arg("K"), py::arg("acts"), py::arg("colsum"), py::arg("op"), py::arg("next_act_mode"), py::arg("alpha") = py::none(),
          py::arg("splitK") = 0, py::arg("sums") = py::none());
    m.def("bgemm_linear_forward_packed", &bgemm_linear_forward_packed, "x x prepacked weights.", py::arg("x"), py::arg("plane"), py::arg("M"),
          py::arg("K"), py::arg("alpha") = py::none(), py::arg("splitK") = 0, py::arg("INSTR") = 1, py::arg("out_kind") = 1,
          py::arg("static_weights") = false);
    m.def("bwta_linear_forward_cuda", &bwta_linear_forward_cuda, "Binary weight x ternary activation, scaled.", py::arg("x"), py::arg("plane"),
          py::arg("M"), py::arg("K"), py::arg("alpha"), py::arg("splitK") = 0);
    m.def("bgemm_attn_matmul_batched", &bgemm_attn_matmul_batched, "Batched {0,1} x {-1,+1} matmul.", py::arg("attn"), py::arg("value"),
          py::arg("exact") = false);
    m.def("w1a16_linear_forward", &w1a16_linear_forward, "Binary weight x fp16 activation, fp32 accumulation.", py::arg("x"), py::arg("plane"),
          py::arg("M"), py::arg("K"), py::arg("alpha") = py::none(), py::arg("out_f32") = false, py::arg("static_weights") = false);
    m.def("linear_forward_cuda", &fp6_not_provided, "FP6 GEMM of the reference: not provided.");
    m.def("weight_dequant_cpu", &fp6_not_provided, "FP6 dequant of the reference: not provided.");
    m.def("plane_bytes", [](int64_t M, int64_t K) { return (int64_t)bgemm_plane_bytes(M, K); });
    m.def("act_ld", [](int64_t K) { return bgemm_act_ld(K); });
    m.def("launch_count", []() { return (uint64_t)bgemm_launch_count(); });
}
