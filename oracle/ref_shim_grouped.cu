// C wrappers around the reference's grouped (MoE) GGUF launchers and its two routing-metadata
// kernels, built into oracle/_ref/libref_grouped.so together with the reference's sources
// WHERE THEY LIE (oracle/Makefile, target `ref`).  Test infrastructure only.  The routing
// kernels are file-local in the reference, so its source file is included into this
// translation unit at build time (nothing is copied into this repository).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <exception>

#include "sm120/gemm/gguf/gguf_grouped_int.cu"   // the reference's file, compiled here
#include "sm120/gemm/gguf/gguf_grouped_gemm.h"
#include "sm120/gemm/gguf/mmq_mma/mmq_mma.h"
#include "smxx/quant/weight_fp8_quant.h"

namespace lc = layerstorm::compute;

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int ref_build_mmq_tile_map(const void* offs, int E, int tile_m, int t_max, void* tile_expert,
                                   void* tile_mstart, void* stream) {
    lc::build_mmq_tile_map<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int32_t*>(offs), E, tile_m, t_max, static_cast<int*>(tile_expert),
        static_cast<int*>(tile_mstart));
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_build_active_expert_list(const void* offs, int E, int cap, void* active, void* stream) {
    lc::build_active_expert_list<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int32_t*>(offs), E, cap, static_cast<int*>(active));
    return static_cast<int>(cudaGetLastError());
}

REF_API size_t ref_gguf_grouped_gemm_workspace_bytes(int total_tokens, int K, int E) {
    return lc::gguf_grouped_gemm_workspace_bytes(total_tokens, K, E);
}

// force: 0 auto, 1 mmvq, 2 mmq, 3 host loop (the codes of the reference's Python binding)
REF_API int ref_gguf_grouped_gemm(int type, int strategy, int E, int N, int K, const void* A, void* D,
                                  const void* offs, const void* b_ptrs, int total_tokens, void* ws,
                                  size_t ws_bytes, int force, void* stream) {
    lc::GgufGroupedGemmKernelParams p;
    p.type = static_cast<lc::GgufType>(type);
    p.strategy = static_cast<lc::GgufGroupedStrategy>(strategy);
    p.num_experts = E; p.N = N; p.K = K;
    p.A_base = static_cast<const __nv_bfloat16*>(A);
    p.D_base = static_cast<__nv_bfloat16*>(D);
    p.expert_offsets = static_cast<const int32_t*>(offs);
    p.B_ptrs = static_cast<const void**>(const_cast<void*>(b_ptrs));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    try {
        if (force == 3) lc::launch_gguf_grouped_gemm_hostloop(p, ws, ws_bytes, s);
        else if (force == 0) lc::launch_gguf_grouped_gemm(p, total_tokens, ws, ws_bytes, s);
        else lc::launch_gguf_grouped_gemm_int_forced(p, total_tokens, ws, ws_bytes,
                                                     static_cast<lc::GgufGroupedIntForce>(force), s);
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_gguf_mmq_mma(int M, int N, int K, const void* A, const void* B, void* C, int type, void* ws,
                             void* stream) {
    lc::GgufMmvqParams p;
    p.M = M; p.N = N; p.K = K;
    p.A = static_cast<const __nv_bfloat16*>(A);
    p.B = B;
    p.C = static_cast<__nv_bfloat16*>(C);
    p.type = static_cast<lc::GgufType>(type);
    try {
        lc::launch_gguf_mmq_mma(p, ws, static_cast<cudaStream_t>(stream));
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}

REF_API int ref_weight_fp8_quant(const void* in, void* out, void* scales, int N, int K, void* stream) {
    lc::WeightFp8QuantParams p;
    p.N = N; p.K = K; p.input = in; p.output = out; p.scales = scales;
    try {
        lc::launch_weight_fp8_quant(p, stream);
    } catch (const std::exception&) { return -1; }
    return static_cast<int>(cudaGetLastError());
}
