// Host-side entry points shared between translation units.
#pragma once
#include <cuda_runtime.h>
#include "../../include/lsg.h"

namespace lsg {

int quantize_q8_1(const void* x_bf16, void* q8_1_out, int M, int K, cudaStream_t stream,
                  bool pdl);
int check_gemm_params(const char* op, const lsg_gguf_mmvq_params* p);
int mmvq_q8_1(int type, int M, int N, int K, const void* W, const void* xq, void* C, int ldc,
              int out_f32, cudaStream_t stream, bool pdl, const void* A_bf16 = nullptr);
bool fused_quant_ok(int M, int K, const void* A);
int dequant_gemm(int type, int M, int N, int K, const void* A, const void* W, void* C, int ldc,
                 int out_f32, cudaStream_t stream);

}  // namespace lsg
