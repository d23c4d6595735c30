// NVFP4 grouped GEMM (MoE projection with 4-bit block-scaled operands):
//   D[rows of e, :] = alpha_e * (A_e (x) SFA) . (B_e (x) SFB)^T
// A: e2m1 codes [T, K/2] (low nibble = even k), B: [E, N, K/2], one ue4m3 scale per 16
// values in the 128-row x 4-group interleaved layout, per-expert alpha, bf16/fp16 output.
//
// Replaces launch_nvfp4_grouped_gemm / query_nvfp4_grouped_gemm_workspace_size
// (csrc/sm120/gemm/nvfp4/nvfp4_grouped_gemm.cu:373-423; params grouped_gemm.h:34-57),
// whose arithmetic is a CUTLASS block-scaled kernel for sm_120 that does not exist on this
// part, and reformat_scales (csrc/smxx/quant/reformat_scales.cu:41-61).
//
// e2m1 x ue4m3 has at most five significant bits, so every scaled operand value is exact
// in fp16.  Both operands are expanded to fp16 once per call and multiplied by the fp16
// tcgen05 kernel of tc_gemm.cu with fp32 accumulation: the products are exactly those of
// the block-scaled definition, only the accumulation order differs.  (The native
// kind::mxf4nvf4 instruction would read the packed operands directly at four times the
// rate; this version is the correct baseline for it.)
#include "common.cuh"
#include "host.h"

#include <cuda_fp8.h>

namespace lsg {

namespace {

__device__ __forceinline__ int sf_offset_sm1xx(int row, int g, int groups_padded4) {
    const int tiles_g = groups_padded4 >> 2;
    const int atom = (row >> 7) * tiles_g + (g >> 2);
    const int r = row & 127;
    return atom * 512 + (r & 31) * 16 + (r >> 5) * 4 + (g & 3);
}

__device__ __forceinline__ float ue4m3_to_float(uint32_t bits) {
    __nv_fp8_e4m3 f8;
    f8.__x = static_cast<__nv_fp8_storage_t>(bits & 0xFFu);
    return static_cast<float>(f8);
}

__device__ __forceinline__ float e2m1_value(uint32_t code) {
    // 0 .5 1 1.5 2 3 4 6 and their negatives
    const uint32_t m = code & 7u;
    const float mag = (m < 4u) ? 0.5f * static_cast<float>(m) : ((m == 4u) ? 2.0f : (m == 5u) ? 3.0f : (m == 6u) ? 4.0f : 6.0f);
    return (code & 8u) ? -mag : mag;
}

// One thread per 16-value group.  is_b == 0: rows are activation rows routed by
// expert_offsets / sf_offsets; is_b == 1: row = e * N + n of the stacked weights.
__global__ void __launch_bounds__(256)
nvfp4_to_f16_kernel(const uint8_t* __restrict__ packed, const void* const* __restrict__ ptrs,
                    const uint8_t* __restrict__ scales, const void* const* __restrict__ scale_ptrs,
                    const int32_t* __restrict__ expert_offsets, const int32_t* __restrict__ sf_offsets,
                    __half* __restrict__ out, long long rows, int K, int N, int E, int is_b) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int gpr = K >> 4;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * gpr) return;
    const long long row = idx / gpr;
    const int g = static_cast<int>(idx - row * gpr);
    const int gp4 = (gpr + 3) & ~3;
    const uint8_t* src;
    const uint8_t* sc;
    int local;
    if (expert_offsets == nullptr) {
        // single problem: rows and scales as they are
        local = static_cast<int>(row);
        src = packed + static_cast<size_t>(row) * (K >> 1);
        sc = scales;
    } else if (is_b) {
        const int e = static_cast<int>(row / N);
        local = static_cast<int>(row - static_cast<long long>(e) * N);
        if (expert_offsets[e + 1] - expert_offsets[e] <= 0) return;  // expert without rows: never read
        src = ptrs ? static_cast<const uint8_t*>(ptrs[e]) + static_cast<size_t>(local) * (K >> 1)
                   : packed + static_cast<size_t>(row) * (K >> 1);
        sc = scale_ptrs ? static_cast<const uint8_t*>(scale_ptrs[e])
                        : scales + static_cast<size_t>(e) * N * gpr;
    } else {
        int lo = 0, hi = E;
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (expert_offsets[mid + 1] <= row) lo = mid + 1;
            else hi = mid;
        }
        if (lo >= E) return;
        local = static_cast<int>(row) - expert_offsets[lo];
        src = packed + static_cast<size_t>(row) * (K >> 1);
        sc = scales + static_cast<size_t>(sf_offsets[lo]) * gpr;
    }
    const float s = ue4m3_to_float(sc[sf_offset_sm1xx(local, g, gp4)]);
    const uint2 codes = *reinterpret_cast<const uint2*>(src + g * 8);
    uint32_t p[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t w = (i < 4) ? codes.x : codes.y;
        const uint32_t byte = (w >> (8 * (i & 3))) & 0xFFu;
        const __half2 hv = __floats2half2_rn(e2m1_value(byte & 0xFu) * s, e2m1_value(byte >> 4) * s);
        p[i] = *reinterpret_cast<const uint32_t*>(&hv);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + row * K + g * 16);
    dst[0] = make_uint4(p[0], p[1], p[2], p[3]);
    dst[1] = make_uint4(p[4], p[5], p[6], p[7]);
}

__global__ void __launch_bounds__(256)
reformat_scales_kernel(const float* __restrict__ src, uint8_t* __restrict__ dst, int rows, int gpr) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * gpr) return;
    const int row = idx / gpr, g = idx - row * gpr;
    const float v = fminf(fmaxf(src[idx], 0.0f), 480.0f);
    dst[sf_offset_sm1xx(row, g, (gpr + 3) & ~3)] =
        static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}

size_t a256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" size_t lsg_nvfp4_sf_buffer_bytes(int rows, int K) {
    if (rows <= 0 || K <= 0) return 0;
    const size_t pr = (static_cast<size_t>(rows) + 127) / 128 * 128;
    const size_t pg = (static_cast<size_t>(K / 16) + 3) / 4 * 4;
    return pr * pg;
}

extern "C" int lsg_nvfp4_reformat_scales(const float* src, void* dst, int rows, int K, void* stream) {
    if (rows <= 0 || K <= 0) return LSG_OK;
    if (!src || !dst) return fail(LSG_ERR_INVALID, "nvfp4_reformat_scales: null pointer");
    const int gpr = K / 16;
    const int total = rows * gpr;
    reformat_scales_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, static_cast<uint8_t*>(dst), rows, gpr);
    LSG_CUDA_TRY(cudaGetLastError());
    return LSG_OK;
}

// expanded != 0: room for the fp16 expansion of both operands (the route taken for weight
// pointer arrays, K not a multiple of 64, or operands that are not 16-byte aligned);
// otherwise only the tile map of the block-scaled tensor-core route.
extern "C" size_t lsg_nvfp4_grouped_gemm_workspace_bytes_ex(int total_tokens, int num_experts, int N, int K,
                                                            int expanded) {
    if (total_tokens <= 0 || num_experts <= 0 || N <= 0 || K <= 0) return 0;
    const int t_max = (total_tokens + 127) / 128 + num_experts;
    const size_t map_bytes = a256(2ull * t_max * 4);
    if (!expanded && K % 64 == 0) return map_bytes;
    return map_bytes + a256(static_cast<size_t>(total_tokens) * K * 2) +
           a256(static_cast<size_t>(num_experts) * N * K * 2);
}

extern "C" size_t lsg_nvfp4_grouped_gemm_workspace_bytes(int total_tokens, int num_experts, int N, int K) {
    return lsg_nvfp4_grouped_gemm_workspace_bytes_ex(total_tokens, num_experts, N, K, 0);
}

extern "C" int lsg_nvfp4_grouped_gemm(const lsg_nvfp4_grouped_gemm_params* p, int total_tokens,
                                      void* workspace, size_t workspace_bytes, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "nvfp4_grouped_gemm: null params");
    if (p->num_experts <= 0 || total_tokens <= 0) return LSG_OK;
    if (p->N % 32 != 0 || p->K % 32 != 0)
        return fail(LSG_ERR_INVALID, "nvfp4_grouped_gemm: N and K must be multiples of 32 (N=%d, K=%d)",
                    p->N, p->K);
    if (p->output_dtype != LSG_DTYPE_BF16 && p->output_dtype != LSG_DTYPE_F16 &&
        p->output_dtype != LSG_DTYPE_F32)
        return fail(LSG_ERR_UNSUPPORTED, "nvfp4_grouped_gemm: output dtype must be bf16, fp16 or f32");
    if (!p->A_base || (!p->B_base && !p->B_ptrs) || !p->D_base || !p->scale_A_base ||
        (!p->scale_B_base && !p->scale_B_ptrs) || !p->alphas || !p->expert_offsets || !p->sf_offsets)
        return fail(LSG_ERR_INVALID, "nvfp4_grouped_gemm: null pointer in params");
    // Block-scaled tensor-core route: packed operands straight from the caller's buffers.
    const bool native = !p->B_ptrs && !p->scale_B_ptrs &&
                        nvfp4_mma_usable(p->A_base, p->B_base, p->scale_A_base, p->scale_B_base, p->K);
    const size_t need = lsg_nvfp4_grouped_gemm_workspace_bytes_ex(total_tokens, p->num_experts, p->N, p->K, native ? 0 : 1);
    if (!workspace || workspace_bytes < need)
        return fail(LSG_ERR_WORKSPACE,
                    "nvfp4_grouped_gemm: workspace too small (have %zu, need %zu%s)",
                    workspace ? workspace_bytes : size_t(0), need,
                    native ? "" : "; this call takes the expanded route: size it with lsg_nvfp4_grouped_gemm_workspace_bytes_ex(..., 1)");
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(LSG_ERR_ALIGNMENT, "nvfp4_grouped_gemm: workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int T = total_tokens, E = p->num_experts, N = p->N, K = p->K;
    const int t_max = (T + 127) / 128 + E;
    uint8_t* base = static_cast<uint8_t*>(workspace);
    int* tile_expert = reinterpret_cast<int*>(base);
    int* tile_mstart = tile_expert + t_max;
    if (native) {
        int rc = build_mmq_tile_map(p->expert_offsets, E, 128, t_max, tile_expert, tile_mstart, s, T);
        if (rc != LSG_OK) return rc;
        return nvfp4_mma(p->A_base, T, p->B_base, static_cast<long long>(E) * N, p->scale_A_base, p->scale_B_base,
                         static_cast<long long>(lsg_nvfp4_sf_buffer_bytes(N, K)), K, N, p->D_base, p->output_dtype,
                         p->alphas, 1.0f, T, tile_expert, tile_mstart, t_max, p->expert_offsets, p->sf_offsets, s);
    }
    __half* a16 = reinterpret_cast<__half*>(base + a256(2ull * t_max * 4));
    __half* b16 = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(a16) + a256(static_cast<size_t>(T) * K * 2));
    const int32_t* offs = p->expert_offsets;
    int rc = build_mmq_tile_map(offs, E, 128, t_max, tile_expert, tile_mstart, s);
    if (rc != LSG_OK) return rc;
    const int gpr = K / 16;
    {
        const long long total = static_cast<long long>(T) * gpr;
        LSG_CUDA_TRY(launch_kernel(nvfp4_to_f16_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256),
                                   0, s, true, static_cast<const uint8_t*>(p->A_base),
                                   static_cast<const void* const*>(nullptr),
                                   static_cast<const uint8_t*>(p->scale_A_base),
                                   static_cast<const void* const*>(nullptr), offs, p->sf_offsets, a16,
                                   static_cast<long long>(T), K, N, E, 0));
    }
    {
        const long long rows = static_cast<long long>(E) * N;
        const long long total = rows * gpr;
        LSG_CUDA_TRY(launch_kernel(nvfp4_to_f16_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256),
                                   0, s, true, static_cast<const uint8_t*>(p->B_base), p->B_ptrs,
                                   static_cast<const uint8_t*>(p->scale_B_base), p->scale_B_ptrs, offs,
                                   p->sf_offsets, b16, rows, K, N, E, 1));
    }
    return tc_gemm_f16(a16, T, b16, static_cast<long long>(E) * N, K, N, p->D_base, p->output_dtype,
                       p->alphas, T, tile_expert, tile_mstart, t_max, offs, s);
}

// ---------------------------------------------------------------------------
// Single problem: D[M,N] = alpha * (A (x) SFA) . (B (x) SFB)^T.
// Replaces launch_nvfp4_gemm / query_nvfp4_gemm_workspace_size
// (csrc/sm120/gemm/nvfp4/nvfp4_gemm.cu:189-200, params gemm.h) on the same exact fp16
// expansion as the grouped operator.
// ---------------------------------------------------------------------------
extern "C" size_t lsg_nvfp4_gemm_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return a256(static_cast<size_t>(M) * K * 2) + a256(static_cast<size_t>(N) * K * 2);
}
// (The single-problem query keeps the size of the expanded route: whether a call can take the
// block-scaled route also depends on pointer alignment, which a size query does not see;
// the block-scaled route itself needs no workspace.)

extern "C" int lsg_nvfp4_gemm(const lsg_nvfp4_gemm_params* p, void* workspace, size_t workspace_bytes,
                              void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "nvfp4_gemm: null params");
    if (p->M < 0 || p->N < 0 || p->K < 0) return fail(LSG_ERR_INVALID, "nvfp4_gemm: negative shape");
    if (p->M == 0 || p->N == 0) return LSG_OK;
    if (p->K % 32 != 0 || p->K == 0)
        return fail(LSG_ERR_INVALID, "nvfp4_gemm: K must be a positive multiple of 32 (K=%d)", p->K);
    if (p->output_dtype != LSG_DTYPE_BF16 && p->output_dtype != LSG_DTYPE_F16 && p->output_dtype != LSG_DTYPE_F32)
        return fail(LSG_ERR_UNSUPPORTED, "nvfp4_gemm: output dtype must be bf16, fp16 or f32");
    if (!p->A || !p->B || !p->D || !p->scale_A || !p->scale_B)
        return fail(LSG_ERR_INVALID, "nvfp4_gemm: null pointer in params");
    if (nvfp4_mma_usable(p->A, p->B, p->scale_A, p->scale_B, p->K))
        return nvfp4_mma(p->A, p->M, p->B, p->N, p->scale_A, p->scale_B, 0, p->K, p->N, p->D, p->output_dtype, nullptr,
                         p->alpha, p->M, nullptr, nullptr, 0, nullptr, nullptr, static_cast<cudaStream_t>(stream));
    const size_t need = lsg_nvfp4_gemm_workspace_bytes(p->M, p->N, p->K);
    if (!workspace || workspace_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "nvfp4_gemm: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(LSG_ERR_ALIGNMENT, "nvfp4_gemm: workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int M = p->M, N = p->N, K = p->K, gpr = K / 16;
    uint8_t* base = static_cast<uint8_t*>(workspace);
    __half* a16 = reinterpret_cast<__half*>(base);
    __half* b16 = reinterpret_cast<__half*>(base + a256(static_cast<size_t>(M) * K * 2));
    const void* const* no_ptrs = nullptr;
    const int32_t* no_offs = nullptr;
    {
        const long long total = static_cast<long long>(M) * gpr;
        LSG_CUDA_TRY(launch_kernel(nvfp4_to_f16_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256),
                                   0, s, true, static_cast<const uint8_t*>(p->A), no_ptrs,
                                   static_cast<const uint8_t*>(p->scale_A), no_ptrs, no_offs, no_offs, a16,
                                   static_cast<long long>(M), K, N, 1, 0));
    }
    {
        const long long total = static_cast<long long>(N) * gpr;
        LSG_CUDA_TRY(launch_kernel(nvfp4_to_f16_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256),
                                   0, s, true, static_cast<const uint8_t*>(p->B), no_ptrs,
                                   static_cast<const uint8_t*>(p->scale_B), no_ptrs, no_offs, no_offs, b16,
                                   static_cast<long long>(N), K, N, 1, 1));
    }
    return tc_gemm_f16(a16, M, b16, N, K, N, p->D, p->output_dtype, nullptr, M, nullptr, nullptr, 0, nullptr, s,
                       p->alpha);
}
