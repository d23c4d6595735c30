// FP8 (e4m3) block-scaled GEMM family and the weight quantizer that feeds it.
//
//   D[m,n] = sum over 128-wide K blocks kb of
//            scale_A[m,kb] * scale_B[n/128,kb] * sum_{k in kb} A8[m,k] * B8[n,k]
// with A8, B8 e4m3 bytes, scale_A fp32 [M, ceil(K/128)] M-major (scale_A[m + kb*M]) and
// scale_B fp32 [ceil(K/128), ceil(N/128)] K-major (scale_B[kb + (n/128)*KB]): the operand
// contract of launch_fp8_gemm (csrc/sm120/gemm/fp8/fp8_gemm.h:18-44), whose arithmetic is a
// CUTLASS sm_120 blockwise kernel (fp8_gemm.cu:42-129) that does not exist on this part, and of
// launch_fp8_grouped_gemm (fp8_grouped_gemm.cu:52-151: a host loop over experts with a
// device-to-host copy of the offsets; here the experts are routed on the device by the tile
// map, no synchronisation).
//
// Both operands are brought to fp16 with their block scale applied (one rounding of 2^-11
// per operand, as on the GGUF tensor-core path) and multiplied by the fp16 tcgen05 kernel of
// tc_gemm.cu with fp32 accumulation.  A native kind::f8f6f4 pipeline with the scales applied
// on a per-128-K accumulator drain would halve the operand traffic; this version is the
// correct baseline for it.
//
// weight_fp8_quant replaces launch_weight_fp8_quant (csrc/smxx/quant/weight_fp8_quant.cu:51-138):
// one scale per 128 x 128 tile (tile amax / 448, 1 for an all-zero tile), values
// clamp(x * (1/scale), +-448) rounded to e4m3, scales stored K-major.  Bit-exact.
#include "common.cuh"
#include "host.h"

#include <cuda_fp8.h>

namespace lsg {

namespace {

size_t a256(size_t v) { return (v + 255) & ~size_t(255); }

__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
    const __half_raw hr = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b & 0xFFu), __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// One thread per 8 values of a row.  mode 0: activation rows (scale M-major inside the
// row's expert, or over all M rows when expert_offsets is null); mode 1: weight rows of E
// stacked [N, K] matrices (scale K-major per 128 x 128 tile, per expert).
__global__ void __launch_bounds__(256)
fp8_to_f16_kernel(const uint8_t* __restrict__ src, const void* const* __restrict__ ptrs,
                  const float* __restrict__ scales, const void* const* __restrict__ scale_ptrs,
                  const int32_t* __restrict__ expert_offsets, __half* __restrict__ out, long long rows, int K,
                  int N, int E, int M_total, int mode) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int vpr = (K + 7) >> 3;  // 8-value pieces per row (K is a multiple of 16)
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= rows * vpr) return;
    const long long row = idx / vpr;
    const int k0 = static_cast<int>(idx - row * vpr) * 8;
    const int kb = k0 >> 7;
    const int KB = (K + 127) >> 7;
    const uint8_t* in;
    float s;
    if (mode == 0) {
        in = src + static_cast<size_t>(row) * K + k0;
        if (expert_offsets) {
            int lo = 0, hi = E;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (expert_offsets[mid + 1] <= row) lo = mid + 1;
                else hi = mid;
            }
            if (lo >= E) return;
            const int off = expert_offsets[lo], Me = expert_offsets[lo + 1] - off;
            s = scales[static_cast<size_t>(off) * KB + (row - off) + static_cast<size_t>(kb) * Me];
        } else {
            s = scales[row + static_cast<size_t>(kb) * M_total];
        }
    } else {
        const int e = static_cast<int>(row / N);
        const int n = static_cast<int>(row - static_cast<long long>(e) * N);
        if (expert_offsets && expert_offsets[e + 1] - expert_offsets[e] <= 0) return;  // never read
        const uint8_t* base = ptrs ? static_cast<const uint8_t*>(ptrs[e]) : src + static_cast<size_t>(e) * N * K;
        if (base == nullptr) return;
        in = base + static_cast<size_t>(n) * K + k0;
        const int NB = (N + 127) >> 7;
        const float* sb = scale_ptrs ? static_cast<const float*>(scale_ptrs[e])
                                     : scales + static_cast<size_t>(e) * KB * NB;
        s = sb[kb + static_cast<size_t>(n >> 7) * KB];
    }
    const uint2 raw = *reinterpret_cast<const uint2*>(in);
    const uint32_t w[2] = {raw.x, raw.y};
    uint32_t p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t two = (w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu;
        const __half2 hv = __floats2half2_rn(e4m3_to_float(two & 0xFFu) * s, e4m3_to_float(two >> 8) * s);
        p[i] = *reinterpret_cast<const uint32_t*>(&hv);
    }
    *reinterpret_cast<uint4*>(out + row * K + k0) = make_uint4(p[0], p[1], p[2], p[3]);
}

// One CTA per 128 x 128 tile of the weight.
__global__ void __launch_bounds__(256)
weight_fp8_quant_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ out, float* __restrict__ scales,
                        int N, int K, int KB) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int n0 = blockIdx.x * 128, k0 = blockIdx.y * 128;
    const int tn = min(128, N - n0), tk = min(128, K - k0);
    const int count = tn * tk;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < count; i += 256) {
        const int ln = i / tk, lk = i - ln * tk;
        amax = fmaxf(amax, fabsf(__bfloat162float(in[static_cast<size_t>(n0 + ln) * K + k0 + lk])));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __shared__ float wmax[8];
    __shared__ float s_scale;
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = 0.0f;
        for (int w = 0; w < 8; ++w) m = fmaxf(m, wmax[w]);
        const float sc = m > 0.0f ? m / 448.0f : 1.0f;
        s_scale = sc;
        scales[blockIdx.y + static_cast<size_t>(blockIdx.x) * KB] = sc;   // K-major
    }
    __syncthreads();
    const float inv = 1.0f / s_scale;
    for (int i = threadIdx.x; i < count; i += 256) {
        const int ln = i / tk, lk = i - ln * tk;
        const size_t at = static_cast<size_t>(n0 + ln) * K + k0 + lk;
        float v = __bfloat162float(in[at]) * inv;
        v = fminf(fmaxf(v, -448.0f), 448.0f);
        out[at] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
    }
}

// Small-batch path (M <= 4): one warp per output column n, lanes stride over 16-byte pieces
// of the weight row, activations (M x K bytes) come from L1/L2, products and the per-128-K
// scaling in fp32.  Exact up to fp32 summation order.  The role of the reference's
// fp8_blockscaled_gemv_kernel (csrc/sm120/gemm/fp8/fp8_blockscaled_gemv.cu:54-145), which
// covers M = 1.
__device__ __forceinline__ void e4m3x4_to_float(uint32_t w, float (&f)[4]) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w & 0xFFFFu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

template <int MR>
__global__ void __launch_bounds__(256)
fp8_gemv_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B, const float* __restrict__ sA,
                const float* __restrict__ sB, void* __restrict__ D, int M, int N, int K, int out_dtype) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const int KB = (K + 127) >> 7;
    const uint8_t* brow = B + static_cast<size_t>(n) * K;
    const float* sbrow = sB + static_cast<size_t>(n >> 7) * KB;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.0f;
    const int pieces = K >> 4;
    for (int c = lane; c < pieces; c += 32) {
        const uint4 bw = __ldg(reinterpret_cast<const uint4*>(brow) + c);
        const uint32_t b4[4] = {bw.x, bw.y, bw.z, bw.w};
        float bf[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float t[4];
            e4m3x4_to_float(b4[i], t);
            bf[4 * i] = t[0]; bf[4 * i + 1] = t[1]; bf[4 * i + 2] = t[2]; bf[4 * i + 3] = t[3];
        }
        const int kb = c >> 3;
        const float sb = sbrow[kb];
#pragma unroll
        for (int m = 0; m < MR; ++m) {
            if (m < M) {
                const uint4 aw = __ldg(reinterpret_cast<const uint4*>(A + static_cast<size_t>(m) * K) + c);
                const uint32_t a4[4] = {aw.x, aw.y, aw.z, aw.w};
                float dot = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float t[4];
                    e4m3x4_to_float(a4[i], t);
                    dot = fmaf(t[0], bf[4 * i], dot);
                    dot = fmaf(t[1], bf[4 * i + 1], dot);
                    dot = fmaf(t[2], bf[4 * i + 2], dot);
                    dot = fmaf(t[3], bf[4 * i + 3], dot);
                }
                acc[m] = fmaf(dot, sA[m + static_cast<size_t>(kb) * M] * sb, acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
    }
    if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MR; ++m) {
            if (m < M) {
                const size_t o = static_cast<size_t>(m) * N + n;
                if (out_dtype == LSG_DTYPE_F32) static_cast<float*>(D)[o] = acc[m];
                else if (out_dtype == LSG_DTYPE_F16) static_cast<__half*>(D)[o] = __float2half_rn(acc[m]);
                else static_cast<__nv_bfloat16*>(D)[o] = __float2bfloat16_rn(acc[m]);
            }
        }
    }
}

int expand(const uint8_t* src, const void* const* ptrs, const float* scales, const void* const* scale_ptrs,
           const int32_t* offs, __half* out, long long rows, int K, int N, int E, int M_total, int mode,
           cudaStream_t s) {
    const long long total = rows * ((K + 7) / 8);
    if (total == 0) return LSG_OK;
    LSG_CUDA_TRY(launch_kernel(fp8_to_f16_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, s, true,
                               src, ptrs, scales, scale_ptrs, offs, out, rows, K, N, E, M_total, mode));
    return LSG_OK;
}

int check_out_dtype(const char* op, int dt) {
    if (dt != LSG_DTYPE_BF16 && dt != LSG_DTYPE_F16 && dt != LSG_DTYPE_F32)
        return fail(LSG_ERR_UNSUPPORTED, "%s: output dtype must be bf16, fp16 or f32", op);
    return LSG_OK;
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_weight_fp8_quant(const void* weight_bf16, void* output_e4m3, float* scales, int N, int K,
                                    void* stream) {
    if (N < 0 || K < 0) return fail(LSG_ERR_INVALID, "weight_fp8_quant: negative shape");
    if (N == 0 || K == 0) return LSG_OK;
    if (!weight_bf16 || !output_e4m3 || !scales) return fail(LSG_ERR_INVALID, "weight_fp8_quant: null pointer");
    if (weight_bf16 == output_e4m3) return fail(LSG_ERR_INVALID, "weight_fp8_quant: not in-place safe");
    const int KB = (K + 127) / 128, NB = (N + 127) / 128;
    if (KB > 65535) return fail(LSG_ERR_UNSUPPORTED, "weight_fp8_quant: K too large");
    LSG_CUDA_TRY(launch_kernel(weight_fp8_quant_kernel, dim3(NB, KB), dim3(256), 0, static_cast<cudaStream_t>(stream),
                               true, static_cast<const __nv_bfloat16*>(weight_bf16),
                               static_cast<uint8_t*>(output_e4m3), scales, N, K, KB));
    return LSG_OK;
}

extern "C" size_t lsg_fp8_gemm_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return a256(static_cast<size_t>(M) * K * 2) + a256(static_cast<size_t>(N) * K * 2);
}

extern "C" int lsg_fp8_gemm(const lsg_fp8_gemm_params* p, void* workspace, size_t workspace_bytes, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "fp8_gemm: null params");
    if (p->M < 0 || p->N < 0 || p->K < 0) return fail(LSG_ERR_INVALID, "fp8_gemm: negative shape");
    if (p->M == 0 || p->N == 0) return LSG_OK;
    if (p->K == 0 || p->K % 16 != 0)
        return fail(LSG_ERR_INVALID, "fp8_gemm: K must be a positive multiple of 16 (K=%d)", p->K);
    int rc = check_out_dtype("fp8_gemm", p->output_dtype);
    if (rc != LSG_OK) return rc;
    if (!p->A || !p->B || !p->D || !p->scale_A || !p->scale_B) return fail(LSG_ERR_INVALID, "fp8_gemm: null pointer");
    if ((reinterpret_cast<uintptr_t>(p->A) | reinterpret_cast<uintptr_t>(p->B)) & 7)
        return fail(LSG_ERR_ALIGNMENT, "fp8_gemm: operands must be 8-byte aligned");
    if (p->M <= 4 && ((reinterpret_cast<uintptr_t>(p->A) | reinterpret_cast<uintptr_t>(p->B)) & 15) == 0) {
        // decode-sized batch: stream the weights once, no operand expansion, no workspace
        const dim3 grid((p->N + 7) / 8);
        const uint8_t* A8 = static_cast<const uint8_t*>(p->A);
        const uint8_t* B8 = static_cast<const uint8_t*>(p->B);
        const float* sa = static_cast<const float*>(p->scale_A);
        const float* sb = static_cast<const float*>(p->scale_B);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (p->M == 1)
            LSG_CUDA_TRY(launch_kernel(fp8_gemv_kernel<1>, grid, dim3(256), 0, st, true, A8, B8, sa, sb, p->D, p->M,
                                       p->N, p->K, p->output_dtype));
        else if (p->M == 2)
            LSG_CUDA_TRY(launch_kernel(fp8_gemv_kernel<2>, grid, dim3(256), 0, st, true, A8, B8, sa, sb, p->D, p->M,
                                       p->N, p->K, p->output_dtype));
        else
            LSG_CUDA_TRY(launch_kernel(fp8_gemv_kernel<4>, grid, dim3(256), 0, st, true, A8, B8, sa, sb, p->D, p->M,
                                       p->N, p->K, p->output_dtype));
        return LSG_OK;
    }
    const size_t need = lsg_fp8_gemm_workspace_bytes(p->M, p->N, p->K);
    if (!workspace || workspace_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "fp8_gemm: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(LSG_ERR_ALIGNMENT, "fp8_gemm: workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int M = p->M, N = p->N, K = p->K;
    uint8_t* base = static_cast<uint8_t*>(workspace);
    __half* a16 = reinterpret_cast<__half*>(base);
    __half* b16 = reinterpret_cast<__half*>(base + a256(static_cast<size_t>(M) * K * 2));
    rc = expand(static_cast<const uint8_t*>(p->A), nullptr, static_cast<const float*>(p->scale_A), nullptr, nullptr,
                a16, M, K, N, 1, M, 0, s);
    if (rc != LSG_OK) return rc;
    rc = expand(static_cast<const uint8_t*>(p->B), nullptr, static_cast<const float*>(p->scale_B), nullptr, nullptr,
                b16, N, K, N, 1, M, 1, s);
    if (rc != LSG_OK) return rc;
    return tc_gemm_f16(a16, M, b16, N, K, N, p->D, p->output_dtype, nullptr, M, nullptr, nullptr, 0, nullptr, s);
}

extern "C" size_t lsg_fp8_grouped_gemm_workspace_bytes(int total_tokens, int num_experts, int N, int K) {
    if (total_tokens <= 0 || num_experts <= 0 || N <= 0 || K <= 0) return 0;
    const size_t t_max = static_cast<size_t>((total_tokens + 127) / 128 + num_experts);
    return a256(2 * t_max * 4) + a256(static_cast<size_t>(total_tokens) * K * 2) +
           a256(static_cast<size_t>(num_experts) * N * K * 2);
}

extern "C" int lsg_fp8_grouped_gemm(const lsg_fp8_grouped_gemm_params* p, int total_tokens, void* workspace,
                                    size_t workspace_bytes, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "fp8_grouped_gemm: null params");
    if ((p->B_ptrs == nullptr) != (p->scale_B_ptrs == nullptr))
        return fail(LSG_ERR_INVALID, "FP8 grouped GEMM: B_ptrs and scale_B_ptrs must be both null or both non-null");
    if (p->num_experts <= 0 || total_tokens <= 0) return LSG_OK;
    if (p->N <= 0 || p->K <= 0 || p->K % 16 != 0)
        return fail(LSG_ERR_INVALID, "fp8_grouped_gemm: N must be positive and K a positive multiple of 16");
    int rc = check_out_dtype("fp8_grouped_gemm", p->output_dtype);
    if (rc != LSG_OK) return rc;
    if (!p->A_base || (!p->B_base && !p->B_ptrs) || !p->D_base || !p->scale_A_base ||
        (!p->scale_B_base && !p->scale_B_ptrs) || !p->expert_offsets)
        return fail(LSG_ERR_INVALID, "fp8_grouped_gemm: null pointer in params");
    const size_t need = lsg_fp8_grouped_gemm_workspace_bytes(total_tokens, p->num_experts, p->N, p->K);
    if (!workspace || workspace_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "fp8_grouped_gemm: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(LSG_ERR_ALIGNMENT, "fp8_grouped_gemm: workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int T = total_tokens, E = p->num_experts, N = p->N, K = p->K;
    const int t_max = (T + 127) / 128 + E;
    uint8_t* base = static_cast<uint8_t*>(workspace);
    int* tile_expert = reinterpret_cast<int*>(base);
    int* tile_mstart = tile_expert + t_max;
    __half* a16 = reinterpret_cast<__half*>(base + a256(2ull * t_max * 4));
    __half* b16 = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(a16) + a256(static_cast<size_t>(T) * K * 2));
    const int32_t* offs = p->expert_offsets;
    rc = build_mmq_tile_map(offs, E, 128, t_max, tile_expert, tile_mstart, s);
    if (rc != LSG_OK) return rc;
    rc = expand(static_cast<const uint8_t*>(p->A_base), nullptr, static_cast<const float*>(p->scale_A_base), nullptr,
                offs, a16, T, K, N, E, T, 0, s);
    if (rc != LSG_OK) return rc;
    rc = expand(static_cast<const uint8_t*>(p->B_base), p->B_ptrs, static_cast<const float*>(p->scale_B_base),
                p->scale_B_ptrs, offs, b16, static_cast<long long>(E) * N, K, N, E, T, 1, s);
    if (rc != LSG_OK) return rc;
    return tc_gemm_f16(a16, T, b16, static_cast<long long>(E) * N, K, N, p->D_base, p->output_dtype, nullptr, T,
                       tile_expert, tile_mstart, t_max, offs, s);
}
