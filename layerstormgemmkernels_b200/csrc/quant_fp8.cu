// Dynamic FP8 (e4m3) activation quantizer, one fp32 scale per (token, 128-column block).
//
// Results are bit-identical to the reference kernel dynamic_fp8_quant_kernel
// (csrc/smxx/quant/dynamic_fp8_quant.cu:38-112): scale = amax / 448 (1.0 when the block
// is all zero), values multiplied by the fp32 reciprocal 1.0f / scale (reciprocal, then
// multiply), clamped to +-448 and converted with round-to-nearest-even, saturating.  The
// maximum does not depend on the order it is taken in, so the thread layout is free.
// The kernel is bound by instruction issue, not by memory, unless the per-block work (index
// arithmetic, two IEEE divisions, the reduction) is spread over many values per lane: four
// lanes own one 128-column block, each four 16-byte pieces of it (piece l, l+4, l+8, l+12, so
// that the four lanes' loads of one step cover 64 contiguous bytes), eight blocks per warp.
// Rows that are not a multiple of eight values long, or unaligned tensors, take the older
// layout (sixteen lanes per block, scalar loads).
#include "common.cuh"
#include "host.h"

#include <cuda_fp8.h>

namespace lsg {

namespace {

constexpr int kFp8Block = 128;
constexpr int kFp8Warps = 8;

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

template <bool VEC>
__global__ void __launch_bounds__(kFp8Warps * 32)
dynamic_fp8_quant_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ out,
                         float* __restrict__ scales, int M, int K, int blocks_per_row,
                         int m_major) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    const int half = lane >> 4, hl = lane & 15;
    const long long gblk = (static_cast<long long>(blockIdx.x) * kFp8Warps + (threadIdx.x >> 5)) * 2 + half;
    const long long total = static_cast<long long>(M) * blocks_per_row;
    const bool live = gblk < total;
    const long long blk = live ? gblk : 0;
    // a 64-bit division costs about a hundred instructions; block counts fit 32 bits in practice
    const int row = total <= 0x7fffffffLL ? static_cast<int>(static_cast<unsigned>(blk) / static_cast<unsigned>(blocks_per_row))
                                          : static_cast<int>(blk / blocks_per_row);
    const int bc = static_cast<int>(blk - static_cast<long long>(row) * blocks_per_row);
    const int col0 = bc * kFp8Block + hl * 8;
    const size_t base = static_cast<size_t>(row) * K + col0;

    float v[8];
    if (VEC) {
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (col0 < K) raw = __ldg(reinterpret_cast<const uint4*>(in + base));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = (col0 + i < K) ? __bfloat162float(in[base + i]) : 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (!live) return;

    const float scale = (amax > 0.0f) ? (amax / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    if (hl == 0) {
        const size_t si = m_major ? (static_cast<size_t>(bc) * M + row)
                                  : (static_cast<size_t>(row) * blocks_per_row + bc);
        scales[si] = scale;
    }
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = fminf(fmaxf(v[i] * inv, -448.0f), 448.0f);
    if (VEC) {
        if (col0 < K) {
            uint2 o;
            o.x = pack_e4m3x4(s[0], s[1], s[2], s[3]);
            o.y = pack_e4m3x4(s[4], s[5], s[6], s[7]);
            *reinterpret_cast<uint2*>(out + base) = o;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (col0 + i < K)
                out[base + i] = static_cast<uint8_t>(
                    __nv_cvt_float_to_fp8(s[i], __NV_SATFINITE, __NV_E4M3));
        }
    }
}

// Four lanes per block, 32 values per lane.  K % 8 == 0, 16-byte aligned input, 8-byte aligned output.
__global__ void __launch_bounds__(kFp8Warps * 32)
dynamic_fp8_quant_wide_kernel(const __nv_bfloat16* __restrict__ in, uint8_t* __restrict__ out,
                              float* __restrict__ scales, int M, int K, int blocks_per_row, int m_major) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    const int ql = lane & 3;
    const long long gblk = (static_cast<long long>(blockIdx.x) * kFp8Warps + (threadIdx.x >> 5)) * 8 + (lane >> 2);
    const long long total = static_cast<long long>(M) * blocks_per_row;
    const bool live = gblk < total;
    const long long blk = live ? gblk : 0;
    const int row = total <= 0x7fffffffLL ? static_cast<int>(static_cast<unsigned>(blk) / static_cast<unsigned>(blocks_per_row))
                                          : static_cast<int>(blk / blocks_per_row);
    const int bc = static_cast<int>(blk - static_cast<long long>(row) * blocks_per_row);
    const int col0 = bc * kFp8Block + ql * 8;           // piece j starts at col0 + 32 j
    const size_t base = static_cast<size_t>(row) * K + col0;

    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        raw[j] = (col0 + 32 * j < K) ? __ldg(reinterpret_cast<const uint4*>(in + base + 32 * j)) : make_uint4(0, 0, 0, 0);
    float v[32];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[8 * j + 2 * i] = __uint_as_float(w[i] << 16);
            v[8 * j + 2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!live) return;

    const float scale = (amax > 0.0f) ? (amax / 448.0f) : 1.0f;
    const float inv = 1.0f / scale;
    if (ql == 0) {
        const size_t si = m_major ? (static_cast<size_t>(bc) * M + row)
                                  : (static_cast<size_t>(row) * blocks_per_row + bc);
        scales[si] = scale;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (col0 + 32 * j >= K) break;
        // the lower clamp also turns a NaN into -448 as the reference's fmaxf/fminf pair does;
        // the upper clamp is the converter's saturation
        float s[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] = fmaxf(v[8 * j + i] * inv, -448.0f);
        uint2 o;
        o.x = pack_e4m3x4(s[0], s[1], s[2], s[3]);
        o.y = pack_e4m3x4(s[4], s[5], s[6], s[7]);
        *reinterpret_cast<uint2*>(out + base + 32 * j) = o;
    }
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_dynamic_fp8_quant(const lsg_dynamic_fp8_quant_params* p, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "dynamic_fp8_quant: null params");
    if (p->num_tokens <= 0 || p->hidden_size <= 0) return LSG_OK;  // as the reference: nothing to do
    if (!p->input || !p->output || !p->scales)
        return fail(LSG_ERR_INVALID, "dynamic_fp8_quant: null pointer in params");
    const int M = p->num_tokens, K = p->hidden_size;
    const int bpr = (K + kFp8Block - 1) / kFp8Block;
    const long long total = static_cast<long long>(M) * bpr;
    const long long grid = (total + kFp8Warps * 2 - 1) / (kFp8Warps * 2);
    if (grid > 0x7fffffffLL) return fail(LSG_ERR_INVALID, "dynamic_fp8_quant: problem too large");
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(p->input) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p->output) & 7) == 0);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    auto in = static_cast<const __nv_bfloat16*>(p->input);
    auto out = static_cast<uint8_t*>(p->output);
    auto sc = static_cast<float*>(p->scales);
    if (vec)
        LSG_CUDA_TRY(launch_kernel(dynamic_fp8_quant_wide_kernel,
                                   dim3(static_cast<unsigned>((total + kFp8Warps * 8 - 1) / (kFp8Warps * 8))),
                                   dim3(kFp8Warps * 32), 0, s, true, in, out, sc, M, K, bpr,
                                   p->m_major_scales ? 1 : 0));
    else
        LSG_CUDA_TRY(launch_kernel(dynamic_fp8_quant_kernel<false>, dim3(static_cast<unsigned>(grid)),
                                   dim3(kFp8Warps * 32), 0, s, true, in, out, sc, M, K, bpr,
                                   p->m_major_scales ? 1 : 0));
    return LSG_OK;
}
