// Q8_1 activation quantizer: bf16 x[M,K] -> 36-byte blocks {fp16 d, fp16 sum, int8 q[32]}.
//
// Results are bit-identical to the reference kernel quantize_bf16_to_q8_1
// (csrc/sm120/gemm/gguf/gguf_mmvq.cu:42-63): d = amax / 127 as an IEEE fp32
// divide, q = rn(x / d) with the un-rounded fp32 d, the stored d rounded to
// fp16, and the block sum taken by the same 16-8-4-2-1 xor butterfly in fp32
// before rounding to fp16.  Four lanes own one block (eight values = one 16-byte
// load each); the reference launches one 32-thread CTA per block.
#include "common.cuh"
#include "formats.cuh"

namespace lsg {

namespace {

constexpr int kQuantThreads = 256;
constexpr int kQ8BatchMax = 8;

// Four lanes per 32-value block, eight consecutive values (one 16-byte load) per lane.
// The block sum is formed in exactly the order of the reference's xor butterfly
// (offsets 16, 8, 4, 2, 1 over lanes = elements): element pairs (i, i+16), then
// (i, i+8), (i, i+4), (i, i+2), (i, i+1).  With eight values per lane the first two
// levels are lane exchanges (lane+2, lane+1) and the last three are in-register.
// U vectors per thread, kQuantThreads apart (so that a warp's loads stay contiguous): all U loads
// are in flight before the first result is needed.  Large tensors take U = 4.
// One lane's share of a block: eight values (the 16 bytes `raw`) of task `tk` (block tk / 4, part
// tk % 4).  All four lanes of a block call this together; lanes that are not `live` take part
// in the exchanges and store nothing.
__device__ __forceinline__ void q8_1_emit(const uint4 raw, bool live, long long tk, uint8_t* __restrict__ y) {
    float v[8];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    // butterfly-ordered sum
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = v[i] + __shfl_xor_sync(0xffffffffu, v[i], 2);   // (i, i+16)
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = s[i] + __shfl_xor_sync(0xffffffffu, s[i], 1);   // (i, i+8)
    const float c0 = s[0] + s[4], c1 = s[1] + s[5], c2 = s[2] + s[6], c3 = s[3] + s[7];  // (i, i+4)
    const float sum = (c0 + c2) + (c1 + c3);                                             // (i, i+2), (i, i+1)
    if (!live) return;

    const float d = amax / 127.0f;
    const float rcp = (amax == 0.0f) ? 0.0f : 1.0f / d;
    uint32_t w0, w1;
    q8_round8(v, d, rcp, w0, w1);
    const long long blk = tk >> 2;
    const int part = static_cast<int>(tk & 3);
    uint32_t* out = reinterpret_cast<uint32_t*>(y + blk * kQ8_1Bytes);
    out[1 + 2 * part] = w0;
    out[2 + 2 * part] = w1;
    if (part == 0) {
        const __half2 ds = __halves2half2(__float2half(d), __float2half(sum));
        out[0] = *reinterpret_cast<const uint32_t*>(&ds);
    }
}

template <int U>
__device__ __forceinline__ void quantize_q8_1_body(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y,
                                                   long long n_blocks, long long cta) {
    const long long task0 = cta * (kQuantThreads * U) + threadIdx.x;
    uint4 raw[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const long long task = task0 + u * kQuantThreads;
        live[u] = task < n_blocks * 4;
        raw[u] = __ldg(reinterpret_cast<const uint4*>(x) + (live[u] ? task : 0));
    }
#pragma unroll
    for (int u = 0; u < U; ++u) q8_1_emit(raw[u], live[u], live[u] ? task0 + u * kQuantThreads : 0, y);
}

// Rows taken through a row map (row r of the output is row map[r] / top_k of x: the gather of
// an MoE layer folded into the quantizer), or formed on the way as bf16(silu(g) * u) from two
// tensors (the activation of an expert block folded into the quantizer of its down projection).
// Same bytes as the gather / activation kernel followed by the plain quantizer.
template <bool SILU>
__global__ void __launch_bounds__(kQuantThreads)
quantize_q8_1_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x2,
                          const int32_t* __restrict__ map, int top_k, uint8_t* __restrict__ y, int rows, int K) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int vpr = K >> 3;                                  // 16-byte vectors per row
    const long long task = static_cast<long long>(blockIdx.x) * kQuantThreads + threadIdx.x;
    const bool live = task < static_cast<long long>(rows) * vpr;
    const long long tk = live ? task : 0;
    const int row = static_cast<int>(tk / vpr), c = static_cast<int>(tk - static_cast<long long>(row) * vpr);
    const int src = map ? map[row] / top_k : row;
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(src) * K) + c);
    if (SILU) {
        const uint4 ur = __ldg(reinterpret_cast<const uint4*>(x2 + static_cast<size_t>(src) * K) + c);
        const uint32_t gw[4] = {raw.x, raw.y, raw.z, raw.w}, uw[4] = {ur.x, ur.y, ur.z, ur.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = silu_mul_bf16x2(gw[j], uw[j]);
        raw = make_uint4(o[0], o[1], o[2], o[3]);
    }
    q8_1_emit(raw, live, tk, y);
}

template <int U>
__global__ void __launch_bounds__(kQuantThreads)
quantize_q8_1_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, long long n_blocks) {
    pdl_launch_dependents();
    pdl_wait_prior();  // x may be the output of the previous kernel in the stream
    quantize_q8_1_body<U>(x, y, n_blocks, blockIdx.x);
}

// Large tensors: one lane per block.  With four lanes per block the kernel is bound by
// instruction issue (eighteen shuffles and two IEEE divisions per eight values); a lane that
// holds all 32 values of a block needs no shuffle, forms the sum in the same butterfly order in
// registers and divides once per 32 values.  The CTA's 256 blocks (9216 contiguous bytes) go
// through shared memory so that the stores are coalesced 4-byte words.
__global__ void __launch_bounds__(kQuantThreads)
quantize_q8_1_wide_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y, long long n_blocks) {
    __shared__ uint32_t stage[kQuantThreads * 9];
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long blk0 = static_cast<long long>(blockIdx.x) * kQuantThreads;
    const long long blk = blk0 + threadIdx.x;
    const bool live = blk < n_blocks;
    const uint4* src = reinterpret_cast<const uint4*>(x) + (live ? blk : 0) * 4;
    uint4 raw[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) raw[j] = __ldg(src + j);
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
    // the xor butterfly over 32 lanes, in registers: (i, i+16), (i, i+8), (i, i+4), (i, i+2), (i, i+1)
    float a[16], b[8], c[4];
#pragma unroll
    for (int i = 0; i < 16; ++i) a[i] = v[i] + v[i + 16];
#pragma unroll
    for (int i = 0; i < 8; ++i) b[i] = a[i] + a[i + 8];
#pragma unroll
    for (int i = 0; i < 4; ++i) c[i] = b[i] + b[i + 4];
    const float sum = (c[0] + c[2]) + (c[1] + c[3]);

    const float d = amax / 127.0f;
    const float rcp = (amax == 0.0f) ? 0.0f : 1.0f / d;
    uint32_t* out = stage + threadIdx.x * 9;
    const __half2 ds = __halves2half2(__float2half(d), __float2half(sum));
    out[0] = *reinterpret_cast<const uint32_t*>(&ds);
#pragma unroll
    for (int k = 0; k < 4; ++k) q8_round8(v + 8 * k, d, rcp, out[1 + 2 * k], out[2 + 2 * k]);
    __syncthreads();
    const long long left = n_blocks - blk0;
    const int words = static_cast<int>(left < kQuantThreads ? left : kQuantThreads) * 9;
    uint32_t* dst = reinterpret_cast<uint32_t*>(y + blk0 * kQ8_1Bytes);
    for (int i = threadIdx.x; i < words; i += kQuantThreads) dst[i] = stage[i];
}

// Several tensors in one launch (the distinct activations of a batch of projections whose inputs
// are all there when the call is made): CTAs [cta_end[t-1], cta_end[t]) quantize tensor t.
struct Q8BatchArgs {
    const __nv_bfloat16* x[kQ8BatchMax];
    uint8_t* y[kQ8BatchMax];
    long long n_blocks[kQ8BatchMax];
    int cta_end[kQ8BatchMax];
    int n;
};

__global__ void __launch_bounds__(kQuantThreads) quantize_q8_1_batch_kernel(const Q8BatchArgs a) {
    pdl_launch_dependents();
    pdl_wait_prior();
    int t = 0;
    while (t + 1 < a.n && static_cast<int>(blockIdx.x) >= a.cta_end[t]) ++t;
    const int first = t > 0 ? a.cta_end[t - 1] : 0;
    quantize_q8_1_body<1>(a.x[t], a.y[t], a.n_blocks[t], static_cast<long long>(blockIdx.x) - first);
}

}  // namespace

int quantize_q8_1_batch(int n, const void* const* x_bf16, void* const* q8_1_out, const int* M, const int* K,
                        cudaStream_t stream, bool pdl) {
    if (n <= 0) return LSG_OK;
    if (n > kQ8BatchMax) return fail(LSG_ERR_INVALID, "quantize_q8_1_batch: at most %d tensors, got %d", kQ8BatchMax, n);
    Q8BatchArgs a = {};
    long long ctas = 0;
    for (int i = 0; i < n; ++i) {
        if (M[i] <= 0 || K[i] <= 0 || K[i] % 32 != 0)
            return fail(LSG_ERR_INVALID, "quantize_q8_1_batch: bad shape of tensor %d (M=%d, K=%d)", i, M[i], K[i]);
        if (!x_bf16[i] || !q8_1_out[i]) return fail(LSG_ERR_INVALID, "quantize_q8_1_batch: null pointer");
        if ((reinterpret_cast<uintptr_t>(x_bf16[i]) & 15) || (reinterpret_cast<uintptr_t>(q8_1_out[i]) & 3))
            return fail(LSG_ERR_ALIGNMENT, "quantize_q8_1_batch: input must be 16-byte and output 4-byte aligned");
        a.x[i] = static_cast<const __nv_bfloat16*>(x_bf16[i]);
        a.y[i] = static_cast<uint8_t*>(q8_1_out[i]);
        a.n_blocks[i] = static_cast<long long>(M[i]) * (K[i] / 32);
        ctas += (a.n_blocks[i] * 4 + kQuantThreads - 1) / kQuantThreads;
        if (ctas > 0x7fffffffLL) return fail(LSG_ERR_INVALID, "quantize_q8_1_batch: too many blocks");
        a.cta_end[i] = static_cast<int>(ctas);
    }
    a.n = n;
    LSG_CUDA_TRY(launch_kernel(quantize_q8_1_batch_kernel, dim3(static_cast<unsigned>(ctas)), dim3(kQuantThreads), 0,
                               stream, pdl, a));
    return LSG_OK;
}

int quantize_q8_1_gather(const void* x_bf16, const int32_t* map, int top_k, void* q8_1_out, int rows, int K,
                          cudaStream_t stream, bool pdl) {
    if (rows <= 0) return LSG_OK;
    if (K <= 0 || K % 32 != 0 || top_k < 1) return fail(LSG_ERR_INVALID, "quantize_q8_1_gather: bad shape");
    if (!x_bf16 || !map || !q8_1_out) return fail(LSG_ERR_INVALID, "quantize_q8_1_gather: null pointer");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(q8_1_out) & 3))
        return fail(LSG_ERR_ALIGNMENT, "quantize_q8_1_gather: input must be 16-byte and output 4-byte aligned");
    const long long tasks = static_cast<long long>(rows) * (K / 8);
    LSG_CUDA_TRY(launch_kernel(quantize_q8_1_rows_kernel<false>, dim3(static_cast<unsigned>((tasks + kQuantThreads - 1) / kQuantThreads)),
                               dim3(kQuantThreads), 0, stream, pdl, static_cast<const __nv_bfloat16*>(x_bf16),
                               static_cast<const __nv_bfloat16*>(nullptr), map, top_k, static_cast<uint8_t*>(q8_1_out), rows, K));
    return LSG_OK;
}

int quantize_q8_1_silu_mul(const void* g_bf16, const void* u_bf16, void* q8_1_out, int rows, int K, cudaStream_t stream,
                           bool pdl) {
    if (rows <= 0) return LSG_OK;
    if (K <= 0 || K % 32 != 0) return fail(LSG_ERR_INVALID, "quantize_q8_1_silu_mul: bad shape");
    if (!g_bf16 || !u_bf16 || !q8_1_out) return fail(LSG_ERR_INVALID, "quantize_q8_1_silu_mul: null pointer");
    if (((reinterpret_cast<uintptr_t>(g_bf16) | reinterpret_cast<uintptr_t>(u_bf16)) & 15) ||
        (reinterpret_cast<uintptr_t>(q8_1_out) & 3))
        return fail(LSG_ERR_ALIGNMENT, "quantize_q8_1_silu_mul: inputs must be 16-byte and output 4-byte aligned");
    const long long tasks = static_cast<long long>(rows) * (K / 8);
    LSG_CUDA_TRY(launch_kernel(quantize_q8_1_rows_kernel<true>, dim3(static_cast<unsigned>((tasks + kQuantThreads - 1) / kQuantThreads)),
                               dim3(kQuantThreads), 0, stream, pdl, static_cast<const __nv_bfloat16*>(g_bf16),
                               static_cast<const __nv_bfloat16*>(u_bf16), static_cast<const int32_t*>(nullptr), 1,
                               static_cast<uint8_t*>(q8_1_out), rows, K));
    return LSG_OK;
}

int quantize_q8_1(const void* x_bf16, void* q8_1_out, int M, int K, cudaStream_t stream,
                  bool pdl) {
    if (M < 0 || K < 0) return fail(LSG_ERR_INVALID, "quantize_q8_1: negative shape");
    if (K % 32 != 0) return fail(LSG_ERR_INVALID, "quantize_q8_1: K must be divisible by 32, got K=%d", K);
    const long long n_blocks = static_cast<long long>(M) * (K / 32);
    if (n_blocks == 0) return LSG_OK;
    if (!x_bf16 || !q8_1_out) return fail(LSG_ERR_INVALID, "quantize_q8_1: null pointer");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(q8_1_out) & 3))
        return fail(LSG_ERR_ALIGNMENT, "quantize_q8_1: input must be 16-byte and output 4-byte aligned");
    if (n_blocks >= 2ll * kQuantThreads * sm_count()) {
        const long long ctas = (n_blocks + kQuantThreads - 1) / kQuantThreads;
        if (ctas > 0x7fffffffLL) return fail(LSG_ERR_INVALID, "quantize_q8_1: too many blocks");
        LSG_CUDA_TRY(launch_kernel(quantize_q8_1_wide_kernel, dim3(static_cast<unsigned>(ctas)), dim3(kQuantThreads), 0,
                                   stream, pdl, static_cast<const __nv_bfloat16*>(x_bf16),
                                   static_cast<uint8_t*>(q8_1_out), n_blocks));
        return LSG_OK;
    }
    const long long tasks = n_blocks * 4;
    const bool big = tasks >= 8ll * kQuantThreads * 4 * sm_count();   // enough CTAs left at four vectors per thread
    const int per_cta = kQuantThreads * (big ? 4 : 1);
    const long long grid = (tasks + per_cta - 1) / per_cta;
    if (grid > 0x7fffffffLL) return fail(LSG_ERR_INVALID, "quantize_q8_1: too many blocks");
    if (big)
        LSG_CUDA_TRY(launch_kernel(quantize_q8_1_kernel<4>, dim3(static_cast<unsigned>(grid)), dim3(kQuantThreads), 0,
                                   stream, pdl, static_cast<const __nv_bfloat16*>(x_bf16),
                                   static_cast<uint8_t*>(q8_1_out), n_blocks));
    else
        LSG_CUDA_TRY(launch_kernel(quantize_q8_1_kernel<1>, dim3(static_cast<unsigned>(grid)), dim3(kQuantThreads), 0,
                                   stream, pdl, static_cast<const __nv_bfloat16*>(x_bf16),
                                   static_cast<uint8_t*>(q8_1_out), n_blocks));
    return LSG_OK;
}

}  // namespace lsg
