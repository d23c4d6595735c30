// Q8_1 activation quantizer: bf16 x[M,K] -> 36-byte blocks {fp16 d, fp16 sum, int8 q[32]}.
//
// Results are bit-identical to the reference kernel quantize_bf16_to_q8_1
// (csrc/sm120/gemm/gguf/gguf_mmvq.cu:42-63): d = amax / 127 as an IEEE fp32
// divide, q = rn(x / d) with the un-rounded fp32 d, the stored d rounded to
// fp16, and the block sum taken by the same 16-8-4-2-1 xor butterfly in fp32
// before rounding to fp16.  One warp owns one block (lane = element), eight
// blocks per CTA; the reference launches one 32-thread CTA per block.
#include "common.cuh"
#include "formats.cuh"

namespace lsg {

namespace {

constexpr int kQuantWarps = 8;

__global__ void __launch_bounds__(kQuantWarps * 32)
quantize_q8_1_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ y,
                     long long n_blocks) {
    pdl_launch_dependents();
    pdl_wait_prior();  // x may be the output of the previous kernel in the stream
    const int lane = threadIdx.x & 31;
    const long long blk = static_cast<long long>(blockIdx.x) * kQuantWarps + (threadIdx.x >> 5);
    if (blk >= n_blocks) return;

    const float xi = __bfloat162float(x[blk * 32 + lane]);
    float amax = fabsf(xi);
    float sum = xi;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        sum += __shfl_xor_sync(0xffffffffu, sum, o);
    }
    const float d = amax / 127.0f;
    const int q = (amax == 0.0f) ? 0 : __float2int_rn(xi / d);

    uint8_t* out = y + blk * kQ8_1Bytes;
    reinterpret_cast<int8_t*>(out + 4)[lane] = static_cast<int8_t>(q);
    if (lane == 0) {
        *reinterpret_cast<__half2*>(out) = __halves2half2(__float2half(d), __float2half(sum));
    }
}

}  // namespace

int quantize_q8_1(const void* x_bf16, void* q8_1_out, int M, int K, cudaStream_t stream,
                  bool pdl) {
    if (M < 0 || K < 0) return fail(LSG_ERR_INVALID, "quantize_q8_1: negative shape");
    if (K % 32 != 0) return fail(LSG_ERR_INVALID, "quantize_q8_1: K must be divisible by 32, got K=%d", K);
    const long long n_blocks = static_cast<long long>(M) * (K / 32);
    if (n_blocks == 0) return LSG_OK;
    if (!x_bf16 || !q8_1_out) return fail(LSG_ERR_INVALID, "quantize_q8_1: null pointer");
    const long long grid = (n_blocks + kQuantWarps - 1) / kQuantWarps;
    if (grid > 0x7fffffffLL) return fail(LSG_ERR_INVALID, "quantize_q8_1: too many blocks");
    LSG_CUDA_TRY(launch_kernel(quantize_q8_1_kernel, dim3(static_cast<unsigned>(grid)),
                               dim3(kQuantWarps * 32), 0, stream, pdl,
                               static_cast<const __nv_bfloat16*>(x_bf16),
                               static_cast<uint8_t*>(q8_1_out), n_blocks));
    return LSG_OK;
}

}  // namespace lsg
