// Host-side entry points shared between translation units.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/lsg.h"

namespace lsg {

int quantize_q8_1(const void* x_bf16, void* q8_1_out, int M, int K, cudaStream_t stream,
                  bool pdl);
// Row r of the output = row map[r] / top_k of x (gather folded in); bf16(silu(g) * u) quantized on the way.
int quantize_q8_1_gather(const void* x_bf16, const int32_t* map, int top_k, void* q8_1_out, int rows, int K,
                          cudaStream_t stream, bool pdl);
int quantize_q8_1_silu_mul(const void* g_bf16, const void* u_bf16, void* q8_1_out, int rows, int K, cudaStream_t stream,
                           bool pdl);
// Up to eight tensors quantized by one launch (same bytes as quantize_q8_1 on each).
int quantize_q8_1_batch(int n, const void* const* x_bf16, void* const* q8_1_out, const int* M, const int* K,
                        cudaStream_t stream, bool pdl);
int check_gemm_params(const char* op, const lsg_gguf_mmvq_params* p);
int mmvq_q8_1(int type, int M, int N, int K, const void* W, const void* xq, void* C, int ldc,
              int out_f32, cudaStream_t stream, bool pdl, const void* A_bf16 = nullptr, int dep_mode = 0);
bool fused_quant_ok(int M, int K, const void* A);
int dequant_gemm(int type, int M, int N, int K, const void* A, const void* W, void* C, int ldc,
                 int out_f32, cudaStream_t stream);

int build_active_expert_list(const int32_t* offs, int E, int cap, int* active, cudaStream_t s);
// `rows` bounds every offset read from the device: offsets that run past the caller's row
// count (an expert-parallel receive buffer that overflowed) can then never index past it.
// The default leaves the offsets as they are, which is the reference's behaviour.
// balanced: tiles of an expert share its rows evenly (balanced_tile_rows) instead of full
// tiles plus a remainder; only for consumers that derive the tile height the same way.
int build_mmq_tile_map(const int32_t* offs, int E, int tile_m, int T_max, int* tile_expert,
                       int* tile_mstart, cudaStream_t s, int rows = 0x7fffffff, bool balanced = false);
int build_segment_list(const int32_t* offs, const void* const* B_ptrs, int E, int max_rows,
                       int max_segments, int* seg, cudaStream_t s, int rows = 0x7fffffff);

size_t mmq_scratch_bytes(long long rows, int K, int E, int N);
// Several output matrices for one GEMM (this GPU's and its peers'): every tile is stored
// into each at column offset col_off, row stride ldc (GEMM fused with the all-gather of a
// column-split weight).
struct MmqOutputs {
    void* const* C_ptrs;   // device array of n_out device pointers
    int n_out;
    int ldc;
    int col_off;
    void* mc_ptr;          // optional: NVLink multicast address of the same [M, ldc] output on every rank
                           // (one multimem store reaches all of them instead of n_out peer stores)
};
int mmq_dense(int type, int M, int N, int K, const void* A, const void* W, void* C, int out_f32, void* ws,
              size_t ws_bytes, cudaStream_t s, const MmqOutputs* outs = nullptr);
int mmq_grouped(int type, int T, int E, int N, int K, const void* A, const void* const* B_ptrs,
                const int32_t* expert_offsets, void* D, int out_f32, const int* tile_expert,
                const int* tile_mstart, int t_max, void* scratch, size_t scratch_bytes, cudaStream_t s);

int tc_gemm_f16(const void* A16, long long a_rows, const void* B16, long long b_rows, int K, int N,
                void* C, int out_dtype, const float* alphas, int M, const int* tile_expert,
                const int* tile_mstart, int t_max, const int32_t* expert_offsets, cudaStream_t s,
                float alpha_host = 1.0f);

// NVFP4 GEMM on tcgen05.mma.kind::mxf4nvf4.block_scale (nvfp4_mma.cu).
bool nvfp4_mma_usable(const void* A, const void* B, const void* sfa, const void* sfb, int K);
int nvfp4_mma(const void* A, long long a_rows, const void* B, long long b_rows, const void* sfa, const void* sfb,
              long long sfb_expert_bytes, int K, int N, void* D, int out_dtype, const float* alphas, float alpha_host,
              int M, const int* tile_expert, const int* tile_mstart, int t_max, const int32_t* expert_offsets,
              const int32_t* sf_offsets, cudaStream_t s);

// Tensor-core GEMM with in-kernel weight decoding (tc_fused.cu).
bool tc_fused_available(int type);
bool tc_fused_forced();   // weight path 2: every call takes the fused kernel
size_t tc_fused_dense_scratch_bytes(int M, int N, int K);
int grouped_gemm_matvec(const lsg_gguf_grouped_gemm_params* p, int T, void* ws, size_t ws_bytes, cudaStream_t s,
                        bool xq_ready, bool seg_ready);
int tc_fused_grouped_tile_m(long long T, int E);
size_t tc_fused_grouped_scratch_bytes(long long T, int E, int N, int K);
int tc_fused_dense(int type, int M, int N, int K, const void* A_bf16, const void* W, void* C, int ldc,
                   int out_dtype, void* ws, size_t ws_bytes, cudaStream_t s, const MmqOutputs* outs = nullptr);
int tc_fused_grouped(int type, int T, int E, int N, int K, const void* A_bf16, const void* const* B_ptrs,
                     const int32_t* expert_offsets, void* D, int out_dtype, const int* tile_expert,
                     const int* tile_mstart, int t_max, int tile_m, void* scratch, size_t scratch_bytes,
                     cudaStream_t s);

size_t tc_fused_bf16_scratch_bytes(int M, int N, int K);
int tc_fused_dense_bf16(int type, int M, int N, int K, const void* A_bf16, const void* W, void* C, int ldc,
                        int out_dtype, void* ws, size_t ws_bytes, cudaStream_t s);
size_t tc_fused_moe_ffn_scratch_bytes(long long T, int H, int I);
int tc_fused_moe_ffn(int type, int T, int E, int H, int I, const void* A_bf16, const void* const* gate_ptrs,
                     const void* const* up_ptrs, const void* const* down_ptrs, const int32_t* expert_offsets,
                     void* D, int out_dtype, const int* tile_expert, const int* tile_mstart, int t_max, int tile_m,
                     void* scratch, size_t scratch_bytes, cudaStream_t s, const int32_t* perm = nullptr, int top_k = 1);

}  // namespace lsg
