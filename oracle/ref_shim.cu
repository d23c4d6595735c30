// C wrappers around the reference's own CUDA launchers, compiled together with the
// reference's source files WHERE THEY LIE (see oracle/Makefile, target `ref`) into
// oracle/_ref/libref_gguf.so.  Test infrastructure only: the tests use it, when it has
// been built, to compare this library's kernels with the reference's kernels on the same
// GPU and inputs.  Nothing from the reference is copied into this repository; this file
// only includes its public headers at build time.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <exception>

#include "sm120/gemm/gguf/gguf_mmvq.h"
#include "sm120/gemm/gguf/gguf_dequant_gemm.h"
#include "smxx/quant/dynamic_fp8_quant.h"
#include "smxx/quant/bf16_to_nvfp4_grouped.h"
#include "smxx/quant/silu_mul_to_nvfp4_grouped.h"
#include "smxx/quant/bf16_to_nvfp4.h"
#include "smxx/quant/reformat_scales.h"
#include "smxx/quant/nvfp4_dequant_bf16.h"

namespace lc = layerstorm::compute;

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int ref_quantize_q8_1(const void* x, void* out, int M, int K, void* stream) {
    try {
        lc::gguf_quantize_q8_1_cuda(static_cast<const __nv_bfloat16*>(x), out, M, K,
                                    static_cast<cudaStream_t>(stream));
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_gguf_mmvq(int M, int N, int K, const void* A, const void* B, void* C, int type,
                          void* workspace, void* stream) {
    lc::GgufMmvqParams p;
    p.M = M; p.N = N; p.K = K;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.B = B;
    p.C = static_cast<__nv_bfloat16*>(C);
    p.type = static_cast<lc::GgufType>(type);
    try {
        lc::launch_gguf_mmvq(p, workspace, static_cast<cudaStream_t>(stream));
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_gguf_dequant_gemm(int M, int N, int K, const void* A, const void* B, void* C,
                                  int type, void* stream) {
    lc::GgufDequantGemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.B = B;
    p.C = static_cast<__nv_bfloat16*>(C);
    p.type = static_cast<lc::GgufType>(type);
    try {
        lc::launch_gguf_dequant_gemm(p, static_cast<cudaStream_t>(stream));
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_dynamic_fp8_quant(const void* in, void* out, void* scales, int M, int K,
                                  int m_major, void* stream) {
    lc::DynamicFp8QuantParams p;
    p.num_tokens = M; p.hidden_size = K; p.input = in; p.output = out; p.scales = scales;
    p.m_major_scales = m_major != 0;
    try {
        lc::launch_dynamic_fp8_quant(p, stream);
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_bf16_to_nvfp4_grouped(const void* in, void* packed, void* scales,
                                      const void* expert_offsets, const void* sf_offsets,
                                      int total_tokens, int num_experts, int K,
                                      const void* input_scales, void* stream) {
    lc::Bf16ToNvfp4GroupedParams p{};
    p.input = in; p.output_packed = packed; p.output_scales = scales;
    p.expert_offsets = expert_offsets; p.sf_offsets = sf_offsets;
    p.total_tokens = total_tokens; p.num_experts = num_experts; p.K = K;
    p.input_scales = input_scales;
    try {
        lc::launch_bf16_to_nvfp4_grouped(p, stream);
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_silu_mul_to_nvfp4_grouped(const void* gate, const void* up, void* packed,
                                          void* scales, const void* expert_offsets,
                                          const void* sf_offsets, int total_tokens,
                                          int num_experts, int K, const void* input_scales,
                                          void* stream) {
    lc::SiluMulToNvfp4GroupedParams p{};
    p.gate = gate; p.up = up; p.output_packed = packed; p.output_scales = scales;
    p.expert_offsets = expert_offsets; p.sf_offsets = sf_offsets;
    p.total_tokens = total_tokens; p.num_experts = num_experts; p.K = K;
    p.input_scales = input_scales;
    try {
        lc::launch_silu_mul_to_nvfp4_grouped(p, stream);
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_bf16_to_nvfp4(const void* in, void* packed, void* scales, int M, int N, int K, void* stream) {
    lc::Bf16ToNvfp4Params p{};
    p.input = static_cast<const __nv_bfloat16*>(in);
    p.output_packed = static_cast<uint8_t*>(packed);
    p.output_scales = static_cast<uint8_t*>(scales);
    p.M = M; p.N = N; p.K = K;
    try {
        lc::launch_bf16_to_nvfp4(p, static_cast<cudaStream_t>(stream));
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_reformat_scales(const float* src, void* dst, int rows, int groups_per_row, int M, int N, int K,
                                int is_scale_a, void* stream) {
    lc::ReformatScalesParams p{};
    p.src_scales = src;
    p.dst_scales = static_cast<uint8_t*>(dst);
    p.rows = rows; p.groups_per_row = groups_per_row; p.M = M; p.N = N; p.K = K;
    p.is_scale_a = is_scale_a != 0;
    try {
        lc::launch_reformat_scales(p, static_cast<cudaStream_t>(stream));
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_nvfp4_dequant_bf16(const void* packed, const void* scales, float weight_scale_2, void* out, int N,
                                   int K, void* stream) {
    lc::Nvfp4DequantBf16Params p{};
    p.N = N; p.K = K; p.input = packed; p.scales = scales; p.weight_scale_2 = weight_scale_2; p.output = out;
    try {
        lc::launch_nvfp4_dequant_bf16(p, stream);
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}
