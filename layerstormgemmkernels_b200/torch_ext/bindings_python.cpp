// PyTorch extension module `sm120_gemm_kernels` for B200: the reference's Python operator
// surface (csrc/bindings_python.cu:752-859 of kkontosis/LayerStoRmGemmKernels - same
// function names, argument names, defaults, checks and return values) as a thin wrapper over
// the C ABI of liblsg_b200.so.  torch supplies tensors, the caching allocator and the
// current stream; every operator runs the sm_100a kernels of the library.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <tuple>

#include "lsg.h"

namespace {

void* current_stream() { return static_cast<void*>(at::cuda::getCurrentCUDAStream().stream()); }

// status -> the exception the reference would have raised
void check(int rc) {
    if (rc == LSG_OK) return;
    const std::string msg = lsg_last_error();
    if (rc == LSG_ERR_INVALID) throw std::invalid_argument(msg);
    throw std::runtime_error(msg);
}

int parse_output_dtype(const std::string& s, at::ScalarType* t) {
    if (s == "bf16" || s == "bfloat16") { *t = at::kBFloat16; return LSG_DTYPE_BF16; }
    if (s == "fp16" || s == "float16") { *t = at::kHalf; return LSG_DTYPE_F16; }
    TORCH_CHECK(false, "Unknown output dtype: ", s, ". Expected 'bf16' or 'fp16'.");
    return LSG_DTYPE_BF16;
}

}  // namespace

std::tuple<torch::Tensor, torch::Tensor> dynamic_fp8_quant(torch::Tensor input, bool m_major_scales) {
    TORCH_CHECK(input.is_cuda(), "dynamic_fp8_quant: input must be on CUDA");
    TORCH_CHECK(input.is_contiguous(), "dynamic_fp8_quant: input must be contiguous");
    TORCH_CHECK(input.dim() == 2, "dynamic_fp8_quant: input must be 2D [M, K]");
    TORCH_CHECK(input.scalar_type() == at::kBFloat16, "dynamic_fp8_quant: input must be BF16");
    const int M = input.size(0), K = input.size(1), nb = (K + 127) / 128;
    auto output = torch::empty({M, K}, input.options().dtype(at::kFloat8_e4m3fn));
    auto scales = m_major_scales ? torch::empty({nb, M}, input.options().dtype(at::kFloat))
                                 : torch::empty({M, nb}, input.options().dtype(at::kFloat));
    lsg_dynamic_fp8_quant_params p;
    p.num_tokens = M; p.hidden_size = K; p.input = input.data_ptr(); p.output = output.data_ptr();
    p.scales = scales.data_ptr(); p.m_major_scales = m_major_scales ? 1 : 0;
    check(lsg_dynamic_fp8_quant(&p, current_stream()));
    return {output, scales};
}

static std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> nvfp4_grouped_quant(
    const char* op, bool swiglu, torch::Tensor x, c10::optional<torch::Tensor> up,
    torch::Tensor expert_offsets, c10::optional<torch::Tensor> input_scales) {
    TORCH_CHECK(x.is_cuda() && x.dtype() == torch::kBFloat16, op, ": input must be BF16 on CUDA");
    TORCH_CHECK(x.dim() == 2 && x.is_contiguous(), op, ": input must be contiguous [T, K]");
    if (swiglu) {
        TORCH_CHECK(up->is_cuda() && up->dtype() == torch::kBFloat16, op, ": up must be BF16 on CUDA");
        TORCH_CHECK(up->dim() == 2 && up->is_contiguous(), op, ": up must be contiguous [T, K]");
        TORCH_CHECK(up->size(0) == x.size(0) && up->size(1) == x.size(1), op,
                    ": gate and up must have the same shape");
    }
    TORCH_CHECK(expert_offsets.dim() == 1 && expert_offsets.scalar_type() == at::kInt, op,
                ": expert_offsets must be 1D int32");
    const int T = x.size(0), K = x.size(1), E = expert_offsets.size(0) - 1;
    TORCH_CHECK(K % 64 == 0, op, ": K must be divisible by 64 "
                "(K/16 groups must align to the 4-group Sm1xx atom)");
    auto offs_cpu = expert_offsets.to(torch::kCPU).contiguous();
    const int32_t* offs = offs_cpu.data_ptr<int32_t>();
    TORCH_CHECK(offs[E] == T, op, ": expert_offsets must end at total_tokens");
    auto sf_cpu = torch::empty({E + 1}, torch::TensorOptions().dtype(at::kInt));
    int32_t* sf = sf_cpu.data_ptr<int32_t>();
    int padded_total = 0;
    for (int e = 0; e <= E; ++e) {
        sf[e] = padded_total;
        if (e < E) padded_total += ((offs[e + 1] - offs[e] + 127) / 128) * 128;
    }
    auto packed = torch::empty({T, K / 2}, x.options().dtype(torch::kUInt8));
    auto scales = torch::zeros({static_cast<int64_t>(padded_total) * (K / 16)}, x.options().dtype(torch::kUInt8));
    auto offs_dev = expert_offsets.is_cuda() ? expert_offsets.contiguous() : expert_offsets.to(x.device()).contiguous();
    auto sf_dev = sf_cpu.to(x.device());
    lsg_nvfp4_grouped_quant_params p = {};
    p.input = x.data_ptr();
    p.up = swiglu ? up->data_ptr() : nullptr;
    p.output_packed = packed.data_ptr();
    p.output_scales = scales.data_ptr();
    p.expert_offsets = offs_dev.data_ptr<int32_t>();
    p.sf_offsets = sf_dev.data_ptr<int32_t>();
    p.total_tokens = T; p.num_experts = E; p.K = K;
    if (input_scales.has_value()) {
        auto& is = input_scales.value();
        TORCH_CHECK(is.is_cuda() && is.scalar_type() == at::kFloat && is.numel() == E, op,
                    ": input_scales must be [num_experts] float32 on CUDA");
        p.input_scales = is.data_ptr<float>();
    }
    check(swiglu ? lsg_silu_mul_to_nvfp4_grouped(&p, current_stream())
                 : lsg_bf16_to_nvfp4_grouped(&p, current_stream()));
    return {packed, scales, sf_dev};
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> bf16_to_nvfp4_grouped(
    torch::Tensor input, torch::Tensor expert_offsets, c10::optional<torch::Tensor> input_scales) {
    return nvfp4_grouped_quant("bf16_to_nvfp4_grouped", false, input, c10::nullopt, expert_offsets, input_scales);
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> silu_mul_to_nvfp4_grouped(
    torch::Tensor gate, torch::Tensor up, torch::Tensor expert_offsets,
    c10::optional<torch::Tensor> input_scales) {
    return nvfp4_grouped_quant("silu_mul_to_nvfp4_grouped", true, gate, up, expert_offsets, input_scales);
}

torch::Tensor nvfp4_gemm_preprocess(torch::Tensor weight_scales, int64_t N, int64_t K) {
    TORCH_CHECK(weight_scales.is_cuda(), "weight_scales must be on CUDA");
    TORCH_CHECK(weight_scales.dim() == 2 && weight_scales.is_contiguous(),
                "weight_scales must be contiguous [N, K/16]");
    TORCH_CHECK(weight_scales.size(0) == N && weight_scales.size(1) == K / 16, "weight_scales shape mismatch");
    auto src = weight_scales.to(torch::kFloat32).contiguous();
    auto out = torch::zeros({static_cast<int64_t>(lsg_nvfp4_sf_buffer_bytes((int)N, (int)K))},
                            torch::TensorOptions().dtype(torch::kUInt8).device(weight_scales.device()));
    check(lsg_nvfp4_reformat_scales(src.data_ptr<float>(), out.data_ptr(), (int)N, (int)K, current_stream()));
    return out;
}

torch::Tensor nvfp4_grouped_gemm(torch::Tensor A_base, torch::Tensor B_base, torch::Tensor D_base,
                                 torch::Tensor scale_A_base, torch::Tensor scale_B_base,
                                 torch::Tensor alphas, torch::Tensor expert_offsets,
                                 torch::Tensor sf_offsets, torch::Tensor problem_sizes, int64_t N,
                                 int64_t K, const std::string& output_dtype) {
    TORCH_CHECK(A_base.is_cuda(), "nvfp4_grouped_gemm: A_base must be on CUDA");
    at::ScalarType st;
    const int code = parse_output_dtype(output_dtype, &st);
    const int E = expert_offsets.size(0) - 1;
    const int T = A_base.size(0);
    const size_t ws_bytes = lsg_nvfp4_grouped_gemm_workspace_bytes(T, E, (int)N, (int)K);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, A_base.options().dtype(at::kByte));
    lsg_nvfp4_grouped_gemm_params p = {};
    p.num_experts = E; p.N = (int)N; p.K = (int)K;
    p.A_base = A_base.data_ptr(); p.B_base = B_base.data_ptr(); p.D_base = D_base.data_ptr();
    p.scale_A_base = scale_A_base.data_ptr(); p.scale_B_base = scale_B_base.data_ptr();
    p.alphas = alphas.data_ptr<float>();
    p.expert_offsets = expert_offsets.data_ptr<int32_t>();
    p.sf_offsets = sf_offsets.data_ptr<int32_t>();
    p.problem_sizes = problem_sizes.data_ptr<int32_t>();
    p.output_dtype = code;
    check(lsg_nvfp4_grouped_gemm(&p, T, ws.data_ptr(), ws_bytes, current_stream()));
    return D_base;
}

torch::Tensor gguf_grouped_gemm(torch::Tensor A_base, torch::Tensor expert_offsets, torch::Tensor b_ptrs,
                                int64_t type_i, int64_t strategy_i, int64_t N, int64_t K, int64_t force_i) {
    TORCH_CHECK(A_base.is_cuda() && A_base.dtype() == torch::kBFloat16,
                "gguf_grouped_gemm: A_base must be BF16 on CUDA");
    TORCH_CHECK(A_base.dim() == 2 && A_base.is_contiguous(), "gguf_grouped_gemm: A_base must be contiguous [T, K]");
    TORCH_CHECK(expert_offsets.is_cuda() && expert_offsets.dtype() == torch::kInt32,
                "gguf_grouped_gemm: expert_offsets must be int32 on CUDA");
    TORCH_CHECK(b_ptrs.is_cuda() && b_ptrs.dtype() == torch::kInt64,
                "gguf_grouped_gemm: b_ptrs must be int64 (device pointers) on CUDA");
    const int T = static_cast<int>(A_base.size(0));
    const int E = static_cast<int>(b_ptrs.numel());
    TORCH_CHECK(expert_offsets.numel() == E + 1, "gguf_grouped_gemm: expert_offsets must be [num_experts+1]");
    auto D = torch::empty({T, N}, A_base.options());
    lsg_gguf_grouped_gemm_params p = {};
    p.type = (int)type_i; p.strategy = (int)strategy_i; p.num_experts = E; p.N = (int)N; p.K = (int)K;
    p.A_base = A_base.data_ptr(); p.D_base = D.data_ptr();
    p.expert_offsets = expert_offsets.data_ptr<int32_t>();
    p.B_ptrs = reinterpret_cast<const void* const*>(b_ptrs.data_ptr());
    p.out_dtype = LSG_DTYPE_BF16;
    const bool tensor_cores = strategy_i == LSG_GGUF_STRATEGY_INT && force_i != LSG_GGUF_FORCE_HOSTLOOP && E > 0 &&
                              (force_i == LSG_GGUF_FORCE_MMQ || (force_i == LSG_GGUF_FORCE_AUTO && T / E > 8));
    const size_t ws_bytes = tensor_cores ? lsg_gguf_grouped_gemm_workspace_bytes_ex(T, (int)K, E, (int)N)
                                         : lsg_gguf_grouped_gemm_workspace_bytes(T, (int)K, E);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, A_base.options().dtype(at::kByte));
    check(lsg_gguf_grouped_gemm(&p, T, ws.data_ptr(), ws_bytes, (int)force_i, current_stream()));
    return D;
}

torch::Tensor gguf_mmvq(torch::Tensor A, torch::Tensor B_packed, int64_t type_i, int64_t N, int64_t K) {
    TORCH_CHECK(A.is_cuda() && A.dtype() == torch::kBFloat16, "gguf_mmvq: A must be BF16 on CUDA");
    TORCH_CHECK(A.dim() == 2 && A.is_contiguous(), "gguf_mmvq: A must be contiguous [M, K]");
    TORCH_CHECK(A.size(1) == K, "gguf_mmvq: A.size(1) != K");
    TORCH_CHECK(B_packed.is_cuda() && B_packed.dtype() == torch::kUInt8 && B_packed.is_contiguous(),
                "gguf_mmvq: B_packed must be contiguous uint8 on CUDA");
    const int M = static_cast<int>(A.size(0));
    auto C = torch::empty({M, N}, A.options());
    lsg_gguf_mmvq_params p = {};
    p.M = M; p.N = (int)N; p.K = (int)K; p.A = A.data_ptr(); p.B = B_packed.data_ptr(); p.C = C.data_ptr();
    p.type = (int)type_i; p.out_dtype = LSG_DTYPE_BF16;
    const size_t ws_bytes = lsg_gguf_mmvq_workspace_bytes(M, (int)K);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, A.options().dtype(at::kByte));
    check(lsg_gguf_mmvq(&p, ws.data_ptr(), ws_bytes, current_stream()));
    return C;
}

// Legacy Q4_K GEMMs (csrc/bindings_python.cu:647-721): x_bf16 @ dequant(W_q4k).T -> BF16.  Both
// names run the tensor-core kernel with in-kernel decoding and unquantized activations.
static torch::Tensor q4k_gemm(const char* op, torch::Tensor x_bf16, torch::Tensor weight_q4k_packed) {
    TORCH_CHECK(x_bf16.is_cuda() && x_bf16.dtype() == torch::kBFloat16, "x_bf16 must be BF16 on CUDA");
    TORCH_CHECK(x_bf16.dim() == 2 && x_bf16.is_contiguous(), "x_bf16 must be contiguous [M, K]");
    TORCH_CHECK(weight_q4k_packed.is_cuda() && weight_q4k_packed.dtype() == torch::kUInt8,
                "weight_q4k_packed must be uint8 on CUDA");
    TORCH_CHECK(weight_q4k_packed.dim() == 2 && weight_q4k_packed.is_contiguous(),
                "weight_q4k_packed must be contiguous [N, K*9/16]");
    const int M = static_cast<int>(x_bf16.size(0));
    const int K = static_cast<int>(x_bf16.size(1));
    const int N = static_cast<int>(weight_q4k_packed.size(0));
    TORCH_CHECK(K % 256 == 0, "K must be divisible by 256, got K=" + std::to_string(K));
    const int expected_row_bytes = (K / 256) * 144;
    TORCH_CHECK(weight_q4k_packed.size(1) == expected_row_bytes,
                "weight row bytes mismatch: expected " + std::to_string(expected_row_bytes) + ", got " +
                    std::to_string((int)weight_q4k_packed.size(1)));
    auto output = torch::empty({M, N}, x_bf16.options());
    lsg_gguf_mmvq_params p = {};
    p.M = M; p.N = N; p.K = K; p.A = x_bf16.data_ptr(); p.B = weight_q4k_packed.data_ptr(); p.C = output.data_ptr();
    p.type = LSG_GGUF_Q4_K; p.out_dtype = LSG_DTYPE_BF16;
    const size_t ws_bytes = lsg_gguf_gemm_bf16_workspace_bytes(M, N, K);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, x_bf16.options().dtype(at::kByte));
    (void)op;
    check(lsg_gguf_gemm_bf16(&p, ws.data_ptr(), ws_bytes, current_stream()));
    return output;
}
torch::Tensor q4k_dequant_gemm(torch::Tensor x, torch::Tensor w) { return q4k_gemm("q4k_dequant_gemm", x, w); }
torch::Tensor q4k_cutlass_gemm(torch::Tensor x, torch::Tensor w) { return q4k_gemm("q4k_cutlass_gemm", x, w); }

int64_t query_sf_a(int64_t M, int64_t, int64_t K) { return (int64_t)lsg_nvfp4_sf_buffer_bytes((int)M, (int)K); }
int64_t query_sf_b(int64_t, int64_t N, int64_t K) { return (int64_t)lsg_nvfp4_sf_buffer_bytes((int)N, (int)K); }
int64_t query_nvfp4_grouped_gemm_ws(int64_t, int64_t, int64_t, const std::string&) {
    // the operator sizes and allocates its own scratch per call (it depends on the row count)
    return 0;
}

// Single-problem NVFP4 (csrc/bindings_python.cu:64-110 and 147-244).
torch::Tensor nvfp4_gemm(torch::Tensor A, torch::Tensor B, torch::Tensor scale_A, torch::Tensor scale_B, int64_t M,
                         int64_t N, int64_t K, double alpha, const std::string& output_dtype) {
    TORCH_CHECK(A.is_cuda() && B.is_cuda(), "nvfp4_gemm: A and B must be on CUDA");
    TORCH_CHECK(scale_A.is_cuda() && scale_B.is_cuda(), "nvfp4_gemm: scales must be on CUDA");
    TORCH_CHECK(A.is_contiguous() && B.is_contiguous(), "nvfp4_gemm: A and B must be contiguous");
    at::ScalarType st;
    const int code = parse_output_dtype(output_dtype, &st);
    auto D = torch::empty({M, N}, A.options().dtype(st));
    const size_t ws_bytes = lsg_nvfp4_gemm_workspace_bytes((int)M, (int)N, (int)K);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, A.options().dtype(at::kByte));
    lsg_nvfp4_gemm_params p = {};
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.A = A.data_ptr(); p.B = B.data_ptr(); p.D = D.data_ptr();
    p.scale_A = scale_A.data_ptr(); p.scale_B = scale_B.data_ptr();
    p.alpha = static_cast<float>(alpha); p.output_dtype = code;
    check(lsg_nvfp4_gemm(&p, ws.data_ptr(), ws_bytes, current_stream()));
    return D;
}

torch::Tensor nvfp4_gemm_preprocess(torch::Tensor weight_scales, int64_t N, int64_t K);

torch::Tensor nvfp4_gemm_from_bf16(torch::Tensor x_bf16, torch::Tensor weight_packed_uint8, torch::Tensor weight_scales,
                                   double weight_scale_global) {
    TORCH_CHECK(x_bf16.is_cuda() && x_bf16.dtype() == torch::kBFloat16, "x_bf16 must be BF16 on CUDA");
    TORCH_CHECK(x_bf16.dim() == 2 && x_bf16.is_contiguous(), "x_bf16 must be contiguous [M, K]");
    TORCH_CHECK(weight_packed_uint8.is_cuda() && weight_packed_uint8.dtype() == torch::kUInt8,
                "weight_packed_uint8 must be uint8 on CUDA");
    TORCH_CHECK(weight_packed_uint8.dim() == 2 && weight_packed_uint8.is_contiguous(),
                "weight_packed_uint8 must be contiguous [N, K/2]");
    TORCH_CHECK(weight_scales.is_cuda(), "weight_scales must be on CUDA");
    const int M = (int)x_bf16.size(0), K = (int)x_bf16.size(1), N = (int)weight_packed_uint8.size(0);
    TORCH_CHECK(weight_packed_uint8.size(1) == K / 2, "weight shape mismatch: expected [N, K/2]");
    TORCH_CHECK(K % 32 == 0, "K must be divisible by 32, got K=" + std::to_string(K));
    TORCH_CHECK(N % 32 == 0, "N must be divisible by 32, got N=" + std::to_string(N));
    const bool pre = weight_scales.dtype() == torch::kUInt8 && weight_scales.dim() == 1;
    torch::Tensor sfb = pre ? weight_scales : nvfp4_gemm_preprocess(weight_scales, N, K);
    auto bytes = x_bf16.options().dtype(at::kByte);
    auto codes = torch::empty({M, K / 2}, bytes);
    auto sfa = torch::zeros({static_cast<int64_t>(lsg_nvfp4_sf_buffer_bytes(M, K))}, bytes);
    check(lsg_bf16_to_nvfp4(x_bf16.data_ptr(), codes.data_ptr(), sfa.data_ptr(), M, K, current_stream()));
    return nvfp4_gemm(codes, weight_packed_uint8, sfa, sfb, M, N, K, weight_scale_global, "bf16");
}

// FP8 family (csrc/bindings_python.cu:444-545).
std::tuple<torch::Tensor, torch::Tensor> weight_fp8_quant(torch::Tensor weight) {
    TORCH_CHECK(weight.is_cuda() && weight.dtype() == torch::kBFloat16, "weight_fp8_quant: weight must be BF16 on CUDA");
    TORCH_CHECK(weight.dim() == 2 && weight.is_contiguous(), "weight_fp8_quant: weight must be contiguous [N, K]");
    const int N = (int)weight.size(0), K = (int)weight.size(1);
    auto output = torch::empty({N, K}, weight.options().dtype(at::kFloat8_e4m3fn));
    auto scales = torch::empty({(N + 127) / 128, (K + 127) / 128}, weight.options().dtype(at::kFloat));
    check(lsg_weight_fp8_quant(weight.data_ptr(), output.data_ptr(), scales.data_ptr<float>(), N, K, current_stream()));
    return {output, scales};
}

torch::Tensor fp8_gemm(torch::Tensor A, torch::Tensor B, torch::Tensor scale_A, torch::Tensor scale_B, int64_t M,
                       int64_t N, int64_t K, const std::string& output_dtype) {
    TORCH_CHECK(A.is_cuda() && B.is_cuda(), "fp8_gemm: A and B must be on CUDA");
    TORCH_CHECK(A.is_contiguous() && B.is_contiguous(), "fp8_gemm: must be contiguous");
    at::ScalarType st;
    const int code = parse_output_dtype(output_dtype, &st);
    auto D = torch::empty({M, N}, A.options().dtype(st));
    const size_t ws_bytes = lsg_fp8_gemm_workspace_bytes((int)M, (int)N, (int)K);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, A.options().dtype(at::kByte));
    lsg_fp8_gemm_params p = {};
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.A = A.data_ptr(); p.B = B.data_ptr(); p.D = D.data_ptr();
    p.scale_A = scale_A.data_ptr(); p.scale_B = scale_B.data_ptr(); p.output_dtype = code;
    check(lsg_fp8_gemm(&p, ws.data_ptr(), ws_bytes, current_stream()));
    return D;
}

torch::Tensor fp8_grouped_gemm(torch::Tensor A_base, torch::Tensor B_base, torch::Tensor D_base,
                               torch::Tensor scale_A_base, torch::Tensor scale_B_base, torch::Tensor expert_offsets,
                               torch::Tensor problem_sizes, int64_t N, int64_t K, const std::string& output_dtype) {
    TORCH_CHECK(A_base.is_cuda(), "fp8_grouped_gemm: A_base must be on CUDA");
    at::ScalarType st;
    const int code = parse_output_dtype(output_dtype, &st);
    const int E = (int)expert_offsets.size(0) - 1;
    const int T = (int)A_base.size(0);
    const size_t ws_bytes = lsg_fp8_grouped_gemm_workspace_bytes(T, E, (int)N, (int)K);
    auto ws = torch::empty({static_cast<int64_t>(ws_bytes > 0 ? ws_bytes : 1)}, A_base.options().dtype(at::kByte));
    lsg_fp8_grouped_gemm_params p = {};
    p.num_experts = E; p.N = (int)N; p.K = (int)K;
    p.A_base = A_base.data_ptr(); p.B_base = B_base.data_ptr(); p.D_base = D_base.data_ptr();
    p.scale_A_base = scale_A_base.data_ptr(); p.scale_B_base = scale_B_base.data_ptr();
    p.expert_offsets = expert_offsets.data_ptr<int32_t>();
    p.problem_sizes = problem_sizes.data_ptr<int32_t>();
    p.output_dtype = code;
    check(lsg_fp8_grouped_gemm(&p, T, ws.data_ptr(), ws_bytes, current_stream()));
    return D_base;
}

int64_t query_zero(int64_t, int64_t, int64_t, const std::string&) { return 0; }

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "B200 (sm_100a) build of the sm120_gemm_kernels operator surface";
    m.def("dynamic_fp8_quant", &dynamic_fp8_quant, py::arg("input"), py::arg("m_major_scales") = false);
    m.def("bf16_to_nvfp4_grouped", &bf16_to_nvfp4_grouped, py::arg("input"), py::arg("expert_offsets"),
          py::arg("input_scales") = py::none());
    m.def("silu_mul_to_nvfp4_grouped", &silu_mul_to_nvfp4_grouped, py::arg("gate"), py::arg("up"),
          py::arg("expert_offsets"), py::arg("input_scales") = py::none());
    m.def("weight_fp8_quant", &weight_fp8_quant, py::arg("weight"));
    m.def("nvfp4_gemm", &nvfp4_gemm, py::arg("A"), py::arg("B"), py::arg("scale_A"), py::arg("scale_B"),
          py::arg("M"), py::arg("N"), py::arg("K"), py::arg("alpha"), py::arg("output_dtype"));
    m.def("nvfp4_gemm_preprocess", &nvfp4_gemm_preprocess, py::arg("weight_scales"), py::arg("N"), py::arg("K"));
    m.def("nvfp4_gemm_from_bf16", &nvfp4_gemm_from_bf16, py::arg("x_bf16"), py::arg("weight_packed_uint8"),
          py::arg("weight_scales"), py::arg("weight_scale_global"));
    m.def("nvfp4_grouped_gemm", &nvfp4_grouped_gemm, py::arg("A_base"), py::arg("B_base"), py::arg("D_base"),
          py::arg("scale_A_base"), py::arg("scale_B_base"), py::arg("alphas"), py::arg("expert_offsets"),
          py::arg("sf_offsets"), py::arg("problem_sizes"), py::arg("N"), py::arg("K"), py::arg("output_dtype"));
    m.def("fp8_gemm", &fp8_gemm, py::arg("A"), py::arg("B"), py::arg("scale_A"), py::arg("scale_B"), py::arg("M"),
          py::arg("N"), py::arg("K"), py::arg("output_dtype"));
    m.def("fp8_grouped_gemm", &fp8_grouped_gemm, py::arg("A_base"), py::arg("B_base"), py::arg("D_base"),
          py::arg("scale_A_base"), py::arg("scale_B_base"), py::arg("expert_offsets"), py::arg("problem_sizes"),
          py::arg("N"), py::arg("K"), py::arg("output_dtype"));
    m.def("gguf_grouped_gemm", &gguf_grouped_gemm, py::arg("A_base"), py::arg("expert_offsets"), py::arg("b_ptrs"),
          py::arg("type"), py::arg("strategy"), py::arg("N"), py::arg("K"), py::arg("force") = 0);
    m.def("gguf_mmvq", &gguf_mmvq, py::arg("A"), py::arg("B_packed"), py::arg("type"), py::arg("N"), py::arg("K"));
    m.def("q4k_dequant_gemm", &q4k_dequant_gemm, py::arg("x_bf16"), py::arg("weight_q4k_packed"));
    m.def("q4k_cutlass_gemm", &q4k_cutlass_gemm, py::arg("x_bf16"), py::arg("weight_q4k_packed"));
    m.def("query_nvfp4_gemm_workspace_size", &query_zero, py::arg("M"), py::arg("N"), py::arg("K"), py::arg("output_dtype"));
    m.def("query_fp8_gemm_workspace_size", &query_zero, py::arg("M"), py::arg("N"), py::arg("K"), py::arg("output_dtype"));
    m.def("query_nvfp4_grouped_gemm_workspace_size", &query_nvfp4_grouped_gemm_ws, py::arg("max_experts"),
          py::arg("N"), py::arg("K"), py::arg("output_dtype"));
    m.def("query_fp8_grouped_gemm_workspace_size", &query_zero, py::arg("max_experts"), py::arg("N"), py::arg("K"),
          py::arg("output_dtype"));
    m.def("query_sf_buffer_size_a", &query_sf_a, py::arg("M"), py::arg("N"), py::arg("K"));
    m.def("query_sf_buffer_size_b", &query_sf_b, py::arg("M"), py::arg("N"), py::arg("K"));
}
