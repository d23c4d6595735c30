// Grouped NVFP4 activation quantizers: bf16 rows (already permuted by expert) ->
// e2m1 codes, two per byte, plus one ue4m3 scale per 16 values written in the
// 128-row x 4-group interleaved scale-factor layout block-scaled tensor-core GEMMs read.
//
// Bit-identical to the reference kernels bf16_to_nvfp4_grouped_kernel
// (csrc/smxx/quant/bf16_to_nvfp4_grouped.cu:16-97) and silu_mul_to_nvfp4_grouped_kernel
// (csrc/smxx/quant/silu_mul_to_nvfp4_grouped.cu:26-119), helpers in
// bf16_to_nvfp4_grouped_detail.cuh:30-92:
//   scale      = max(amax / (6 * is), 2^-9), stored as ue4m3 (clamped to [0, 480], RN)
//   code(v)    = sign | #{thresholds .25 .75 1.25 1.75 2.5 3.5 5 that |v| reaches},
//                v = x * (1 / (ue4m3(scale) * is))       (ties go up in magnitude; formed here
//                by the hardware converter on a value that cannot tie, see e2m1_untie)
//   SwiGLU     = bf16( (g * (0.5 * tanhf(0.5 g) + 0.5)) * u ) before quantization
// One thread per 16-value group (two 16-byte loads, one 8-byte store); a CTA covers up to
// 256 consecutive groups of one row and resolves the row's expert once.
#include "common.cuh"
#include "host.h"

#include <cuda_fp8.h>

namespace lsg {

namespace {

__device__ __forceinline__ int sf_offset_sm1xx(int row, int g, int groups_padded4) {
    // 512-byte atoms of 128 rows x 4 groups, atoms tiled row-major over (row/128, g/4);
    // inside an atom: (row % 32) * 16 + ((row % 128) / 32) * 4 + g % 4.
    const int tiles_g = groups_padded4 >> 2;
    const int atom = (row >> 7) * tiles_g + (g >> 2);
    const int r = row & 127;
    return atom * 512 + (r & 31) * 16 + (r >> 5) * 4 + (g & 3);
}

// The reference's code of a value is sign | #{thresholds .25 .75 1.25 1.75 2.5 3.5 5 that |v|
// reaches}: round to the nearest e2m1 magnitude with every tie going up.  The converter of the
// hardware rounds ties to even, so it is given a value that is never a tie: the lowest mantissa
// bit is set first.  A threshold (even bit pattern) then lies just above itself and goes up; the
// float just below a threshold already has that bit set and stays below; no other value can
// cross a threshold by one unit in the last place.  Three inputs need care: -0.0 and NaN, which
// the reference maps to code 0 (none of its comparisons holds), and infinities, whose bit
// pattern with the low bit set would be a NaN (clamped to +-8 first: the converter saturates
// to 6, code 7, like the comparisons).
__device__ __forceinline__ float e2m1_untie(float v) {
    const bool some = fabsf(v) > 0.0f;                       // false for +-0 and NaN
    const float c = fminf(fmaxf(v, -8.0f), 8.0f);
    return some ? __uint_as_float(__float_as_uint(c) | 1u) : 0.0f;
}

// Eight values -> eight 4-bit codes, value i in bits 4i..4i+3.
__device__ __forceinline__ uint32_t e2m1_codes8(const float* v, float inv) {
    float t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = e2m1_untie(v[i] * inv);
    uint32_t r;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}"
        : "=r"(r)
        : "f"(t[0]), "f"(t[1]), "f"(t[2]), "f"(t[3]), "f"(t[4]), "f"(t[5]), "f"(t[6]), "f"(t[7]));
    return r;
}

__device__ __forceinline__ float swiglu(float g, float u) {
    const float silu = g * (0.5f * tanhf(0.5f * g) + 0.5f);
    return silu * u;
}

// Which expert owns `row`: the last e with offsets[e] <= row < offsets[e+1].
__device__ __forceinline__ int expert_of_row(const int32_t* __restrict__ offs, int E, int row) {
    int lo = 0, hi = E;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (offs[mid + 1] <= row) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(256)
nvfp4_grouped_quant_kernel(const __nv_bfloat16* __restrict__ in, const __nv_bfloat16* __restrict__ up,
                           uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                           const int32_t* __restrict__ expert_offsets,
                           const int32_t* __restrict__ sf_offsets,
                           const float* __restrict__ input_scales, int T, int E, int K) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int row = blockIdx.y;
    const int gpr = K >> 4;
    // The group's values are fetched first: their addresses need nothing of the expert look-up
    // below, whose dependent loads would otherwise sit in front of them in every CTA.
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    const bool in_row = g < gpr;
    const size_t base = static_cast<size_t>(row) * K + static_cast<size_t>(in_row ? g : 0) * 16;
    uint4 ra = make_uint4(0, 0, 0, 0), rb = ra, ua = ra, ub = ra;
    if (in_row) {
        const uint4* p = reinterpret_cast<const uint4*>(in + base);
        ra = __ldg(p);
        rb = __ldg(p + 1);
        if (SWIGLU) {
            const uint4* q = reinterpret_cast<const uint4*>(up + base);
            ua = __ldg(q);
            ub = __ldg(q + 1);
        }
    }
    // The row's expert is the number of experts that end at or before it.  With at most one
    // expert per thread that is one load per thread and one counting barrier; a binary search
    // by one thread (seven dependent loads with the CTA waiting) only for more experts.
    int e = 0, e_start = 0, sf_base = 0;
    if (expert_offsets != nullptr) {
        if (E <= static_cast<int>(blockDim.x)) {
            const int t = threadIdx.x;
            e = __syncthreads_count(t < E && __ldg(expert_offsets + t + 1) <= row);
        } else {
            __shared__ int s_e;
            if (threadIdx.x == 0) s_e = expert_of_row(expert_offsets, E, row);
            __syncthreads();
            e = s_e;
        }
        e = min(e, E - 1);
        e_start = __ldg(expert_offsets + e);
        sf_base = __ldg(sf_offsets + e);
    }
    if (!in_row) return;
    const int local_row = row - e_start;
    float is = 1.0f;
    if (input_scales) {
        const float v = input_scales[e];
        if (v > 0.0f) is = v;
    }

    float x[16];
    {
        const uint32_t w[8] = {ra.x, ra.y, ra.z, ra.w, rb.x, rb.y, rb.z, rb.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    if (SWIGLU) {
        const uint32_t w[8] = {ua.x, ua.y, ua.z, ua.w, ub.x, ub.y, ub.z, ub.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float u0 = __uint_as_float(w[i] << 16), u1 = __uint_as_float(w[i] & 0xFFFF0000u);
            x[2 * i] = __bfloat162float(__float2bfloat16(swiglu(x[2 * i], u0)));
            x[2 * i + 1] = __bfloat162float(__float2bfloat16(swiglu(x[2 * i + 1], u1)));
        }
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));

    float scale = amax / (6.0f * is);
    scale = fmaxf(scale, 0.001953125f);  // 2^-9, the smallest positive ue4m3
    const float clamped = fminf(fmaxf(scale, 0.0f), 480.0f);
    const uint32_t sbits = static_cast<uint32_t>(
        __nv_cvt_float_to_fp8(clamped, __NV_SATFINITE, __NV_E4M3)) & 0xFFu;
    __nv_fp8_e4m3 f8;
    f8.__x = static_cast<__nv_fp8_storage_t>(sbits);
    float srepr = static_cast<float>(f8);
    srepr = fmaxf(srepr, 1e-12f);
    const int groups_padded4 = (gpr + 3) & ~3;
    scales[static_cast<size_t>(sf_base) * gpr + sf_offset_sm1xx(local_row, g, groups_padded4)] =
        static_cast<uint8_t>(sbits);

    const float inv = 1.0f / (srepr * is);
    const uint32_t lo = e2m1_codes8(x, inv), hi = e2m1_codes8(x + 8, inv);
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * (K >> 1) + static_cast<size_t>(g) * 8) =
        make_uint2(lo, hi);
}

// sf_offsets[e] = sum over experts before e of their row counts rounded up to 128
// (the reference computes this on the host: csrc/bindings_python.cu:312-326).
__global__ void nvfp4_sf_offsets_kernel(const int32_t* __restrict__ expert_offsets,
                                        int32_t* __restrict__ sf_offsets, int E) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int acc = 0;
    for (int e = 0; e <= E; ++e) {
        sf_offsets[e] = acc;
        if (e < E) acc += ((expert_offsets[e + 1] - expert_offsets[e] + 127) / 128) * 128;
    }
}

template <bool SWIGLU>
int launch_quant(const lsg_nvfp4_grouped_quant_params* p, const char* op, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "%s: null params", op);
    // the reference returns silently in these two cases (bf16_to_nvfp4_grouped.cu:101-102)
    if (p->K % 16 != 0) return LSG_OK;
    if (p->total_tokens <= 0) return LSG_OK;
    if (!p->input || (SWIGLU && !p->up) || !p->output_packed || !p->output_scales ||
        !p->expert_offsets || !p->sf_offsets)
        return fail(LSG_ERR_INVALID, "%s: null pointer in params", op);
    if ((reinterpret_cast<uintptr_t>(p->input) & 15) || (SWIGLU && (reinterpret_cast<uintptr_t>(p->up) & 15)) ||
        (reinterpret_cast<uintptr_t>(p->output_packed) & 7))
        return fail(LSG_ERR_ALIGNMENT, "%s: input must be 16-byte and output 8-byte aligned", op);
    const int gpr = p->K / 16;
    const int threads = gpr < 256 ? ((gpr + 31) / 32) * 32 : 256;
    dim3 grid((gpr + threads - 1) / threads, p->total_tokens);
    if (p->total_tokens > 65535) {
        // grid.y limit: fold rows into several launches
        return fail(LSG_ERR_UNSUPPORTED, "%s: more than 65535 rows per call is not supported", op);
    }
    LSG_CUDA_TRY(launch_kernel(nvfp4_grouped_quant_kernel<SWIGLU>, grid, dim3(threads), 0,
                               static_cast<cudaStream_t>(stream), true,
                               static_cast<const __nv_bfloat16*>(p->input),
                               static_cast<const __nv_bfloat16*>(p->up),
                               static_cast<uint8_t*>(p->output_packed),
                               static_cast<uint8_t*>(p->output_scales),
                               static_cast<const int32_t*>(p->expert_offsets),
                               static_cast<const int32_t*>(p->sf_offsets),
                               static_cast<const float*>(p->input_scales), p->total_tokens,
                               p->num_experts, p->K));
    return LSG_OK;
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_bf16_to_nvfp4_grouped(const lsg_nvfp4_grouped_quant_params* p, void* stream) {
    return launch_quant<false>(p, "bf16_to_nvfp4_grouped", stream);
}

extern "C" int lsg_silu_mul_to_nvfp4_grouped(const lsg_nvfp4_grouped_quant_params* p, void* stream) {
    return launch_quant<true>(p, "silu_mul_to_nvfp4_grouped", stream);
}

extern "C" int lsg_nvfp4_sf_offsets(const int32_t* expert_offsets, int32_t* sf_offsets,
                                    int num_experts, void* stream) {
    if (num_experts < 0 || !expert_offsets || !sf_offsets)
        return fail(LSG_ERR_INVALID, "nvfp4_sf_offsets: bad argument");
    nvfp4_sf_offsets_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(expert_offsets,
                                                                             sf_offsets, num_experts);
    LSG_CUDA_TRY(cudaGetLastError());
    return LSG_OK;
}

// Single-problem quantizer: x[M,K] bf16 -> e2m1 codes [M, K/2] + ue4m3 scales in the
// interleaved layout of an (M, K/16) scale matrix.  Replaces launch_bf16_to_nvfp4,
// csrc/smxx/quant/bf16_to_nvfp4.cu:76-140 (same arithmetic as the grouped kernel with one
// expert and no global input scale).  Padding entries of the scale buffer are not written.
extern "C" int lsg_bf16_to_nvfp4(const void* x_bf16, void* output_packed, void* output_scales, int M, int K,
                                 void* stream) {
    if (K % 16 != 0) return LSG_OK;   // as the reference: silently nothing (bf16_to_nvfp4.cu:137)
    if (M <= 0 || K <= 0) return LSG_OK;
    if (!x_bf16 || !output_packed || !output_scales) return fail(LSG_ERR_INVALID, "bf16_to_nvfp4: null pointer");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(output_packed) & 7))
        return fail(LSG_ERR_ALIGNMENT, "bf16_to_nvfp4: input must be 16-byte and output 8-byte aligned");
    if (M > 65535) return fail(LSG_ERR_UNSUPPORTED, "bf16_to_nvfp4: more than 65535 rows per call is not supported");
    const int gpr = K / 16;
    const int threads = gpr < 256 ? ((gpr + 31) / 32) * 32 : 256;
    dim3 grid((gpr + threads - 1) / threads, M);
    LSG_CUDA_TRY(launch_kernel(nvfp4_grouped_quant_kernel<false>, grid, dim3(threads), 0,
                               static_cast<cudaStream_t>(stream), true, static_cast<const __nv_bfloat16*>(x_bf16),
                               static_cast<const __nv_bfloat16*>(nullptr), static_cast<uint8_t*>(output_packed),
                               static_cast<uint8_t*>(output_scales), static_cast<const int32_t*>(nullptr),
                               static_cast<const int32_t*>(nullptr), static_cast<const float*>(nullptr), M, 1, K));
    return LSG_OK;
}

// NVFP4 weight [N, K/2] codes + raw row-major ue4m3 group scales [N, K/16] + global scalar
// -> bf16 [N, K]: value = (e2m1(code) * e4m3(scale)) * weight_scale_2, rounded to bf16.
// Replaces launch_nvfp4_dequant_bf16, csrc/smxx/quant/nvfp4_dequant_bf16.cu:41-121 (same
// products in the same order, hence the same bf16 bits).  One thread per 16-value group.
namespace lsg {
namespace {
__global__ void __launch_bounds__(256)
nvfp4_dequant_bf16_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales, float ws2,
                          __nv_bfloat16* __restrict__ out, long long groups) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long g = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (g >= groups) return;
    __nv_fp8_e4m3 f8;
    f8.__x = static_cast<__nv_fp8_storage_t>(scales[g]);
    const float gs = static_cast<float>(f8);
    const uint2 codes = *reinterpret_cast<const uint2*>(packed + g * 8);
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t byte = ((i < 4 ? codes.x : codes.y) >> (8 * (i & 3))) & 0xFFu;
        float v[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t c = h ? (byte >> 4) : (byte & 0xFu);
            const uint32_t m = c & 7u;
            const float mag = (m < 4u) ? 0.5f * static_cast<float>(m)
                                       : ((m == 4u) ? 2.0f : (m == 5u) ? 3.0f : (m == 6u) ? 4.0f : 6.0f);
            v[h] = ((c & 8u) ? -mag : mag) * gs * ws2;
        }
        const __nv_bfloat162 r = __floats2bfloat162_rn(v[0], v[1]);
        o[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + g * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}
}  // namespace
}  // namespace lsg

extern "C" int lsg_nvfp4_dequant_bf16(const void* input_packed, const void* scales, float weight_scale_2,
                                      void* output_bf16, int N, int K, void* stream) {
    if (N <= 0 || K <= 0) return LSG_OK;   // as the reference (nvfp4_dequant_bf16.cu:90)
    if (!input_packed || !scales || !output_bf16)
        return lsg::fail(LSG_ERR_INVALID, "launch_nvfp4_dequant_bf16: null pointer in params");
    if (K % 16 != 0)
        return lsg::fail(LSG_ERR_INVALID, "launch_nvfp4_dequant_bf16: K must be divisible by 16 (got %d)", K);
    if ((reinterpret_cast<uintptr_t>(input_packed) & 7) || (reinterpret_cast<uintptr_t>(output_bf16) & 15))
        return lsg::fail(LSG_ERR_ALIGNMENT, "nvfp4_dequant_bf16: input must be 8-byte and output 16-byte aligned");
    const long long groups = static_cast<long long>(N) * (K / 16);
    LSG_CUDA_TRY(lsg::launch_kernel(lsg::nvfp4_dequant_bf16_kernel, dim3(static_cast<unsigned>((groups + 255) / 256)),
                                    dim3(256), 0, static_cast<cudaStream_t>(stream), true,
                                    static_cast<const uint8_t*>(input_packed), static_cast<const uint8_t*>(scales),
                                    weight_scale_2, static_cast<__nv_bfloat16*>(output_bf16), groups));
    return LSG_OK;
}
