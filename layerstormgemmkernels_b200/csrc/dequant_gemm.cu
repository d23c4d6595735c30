// Lossless-activation GGUF GEMM ("Dequant" strategy): C = A(bf16) . dequant(W)^T
// with fp32 accumulation.  It exists as the golden the reference's own GPU tests
// compare the integer paths against (tests/test_gguf_mmvq.py:45-53,
// tests/test_gguf_grouped_gemm.py:129-159), not as a throughput path.
// Replaces launch_gguf_dequant_gemm (csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:309-325).
//
// One CTA computes a 32(M) x 32(N) output tile.  Per 256-value K step it
// expands 32 weight rows to fp32 in shared memory (one thread per block) and
// stages the matching bf16 activations; 256 threads then each accumulate a
// 2x2 patch with fmaf in ascending k, the same per-output order as the
// reference kernels (gguf_dequant_gemm.cu:94-142, 172-252).
#include "common.cuh"
#include "formats.cuh"
#include "host.h"

namespace lsg {

namespace {

constexpr int kTile = 32;
constexpr int kStep = 256;
constexpr int kPad = 4;

template <int T>
__global__ void __launch_bounds__(256)
dequant_gemm_kernel(const __nv_bfloat16* __restrict__ A, const uint8_t* __restrict__ W,
                    void* __restrict__ C, int M, int N, int K, int ldc, int out_f32) {
    using F = Fmt<T>;
    constexpr int BPS = kStep / F::VALS;  // blocks per K step per row
    extern __shared__ __align__(16) float dg_smem[];
    float (*sW)[kStep + kPad] = reinterpret_cast<float (*)[kStep + kPad]>(dg_smem);
    float (*sA)[kStep + kPad] = sW + kTile;

    const int tid = threadIdx.x;
    const int n0 = blockIdx.x * kTile, m0 = blockIdx.y * kTile;
    const int tx = tid & 15, ty = tid >> 4;
    const size_t row_bytes = static_cast<size_t>(K / F::VALS) * F::BYTES;

    float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += kStep) {
        const int kw = min(kStep, K - k0);
        for (int idx = tid; idx < kTile * BPS; idx += 256) {
            const int r = idx / BPS, b = idx % BPS;
            float* dst = &sW[r][b * F::VALS];
            if (n0 + r < N && b * F::VALS < kw) {
                const uint8_t* blk = W + static_cast<size_t>(n0 + r) * row_bytes +
                                     static_cast<size_t>(k0 / F::VALS + b) * F::BYTES;
                dequant_block<T>(blk, dst);
            } else {
                for (int i = 0; i < F::VALS; ++i) dst[i] = 0.0f;
            }
        }
        for (int idx = tid; idx < kTile * kStep; idx += 256) {
            const int r = idx / kStep, k = idx % kStep;
            sA[r][k] = (m0 + r < M && k < kw)
                           ? __bfloat162float(A[static_cast<size_t>(m0 + r) * K + k0 + k])
                           : 0.0f;
        }
        __syncthreads();
        for (int k = 0; k < kw; ++k) {
            const float a0 = sA[ty * 2][k], a1 = sA[ty * 2 + 1][k];
            const float w0 = sW[tx * 2][k], w1 = sW[tx * 2 + 1][k];
            acc[0][0] = fmaf(a0, w0, acc[0][0]);
            acc[0][1] = fmaf(a0, w1, acc[0][1]);
            acc[1][0] = fmaf(a1, w0, acc[1][0]);
            acc[1][1] = fmaf(a1, w1, acc[1][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + ty * 2 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int n = n0 + tx * 2 + j;
            if (n >= N) continue;
            const size_t o = static_cast<size_t>(m) * ldc + n;
            if (out_f32) static_cast<float*>(C)[o] = acc[i][j];
            else static_cast<__nv_bfloat16*>(C)[o] = __float2bfloat16_rn(acc[i][j]);
        }
    }
}

template <int T>
__global__ void dequant_blocks_kernel(const uint8_t* __restrict__ packed, float* __restrict__ out,
                                      long long n_blocks) {
    const long long b = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    float tmp[Fmt<T>::VALS];
    dequant_block<T>(packed + b * Fmt<T>::BYTES, tmp);
    for (int i = 0; i < Fmt<T>::VALS; ++i) out[b * Fmt<T>::VALS + i] = tmp[i];
}

template <int T>
int launch_dg(int M, int N, int K, const void* A, const void* W, void* C, int ldc, int out_f32,
              cudaStream_t stream) {
    auto kernel = dequant_gemm_kernel<T>;
    const size_t smem = 2 * sizeof(float) * kTile * (kStep + kPad);
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(smem)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    dim3 grid((N + kTile - 1) / kTile, (M + kTile - 1) / kTile);
    kernel<<<grid, 256, smem, stream>>>(static_cast<const __nv_bfloat16*>(A),
                                     static_cast<const uint8_t*>(W), C, M, N, K, ldc, out_f32);
    LSG_CUDA_TRY(cudaGetLastError());
    return LSG_OK;
}

template <int T>
int launch_db(const void* packed, float* out, long long n_blocks, cudaStream_t stream) {
    const long long grid = (n_blocks + 127) / 128;
    dequant_blocks_kernel<T><<<static_cast<unsigned>(grid), 128, 0, stream>>>(
        static_cast<const uint8_t*>(packed), out, n_blocks);
    LSG_CUDA_TRY(cudaGetLastError());
    return LSG_OK;
}

}  // namespace

int dequant_gemm(int type, int M, int N, int K, const void* A, const void* W, void* C, int ldc,
                 int out_f32, cudaStream_t stream) {
    if (M == 0 || N == 0) return LSG_OK;
    if (!A || !W || !C) return fail(LSG_ERR_INVALID, "gguf_dequant_gemm: null pointer");
    switch (type) {
        case 0: return launch_dg<0>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 1: return launch_dg<1>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 2: return launch_dg<2>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 3: return launch_dg<3>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 4: return launch_dg<4>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 5: return launch_dg<5>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 6: return launch_dg<6>(M, N, K, A, W, C, ldc, out_f32, stream);
        case 7: return launch_dg<7>(M, N, K, A, W, C, ldc, out_f32, stream);
    }
    return fail(LSG_ERR_UNSUPPORTED, "gguf_dequant_gemm: unknown type %d", type);
}

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_gguf_dequant_gemm(const lsg_gguf_mmvq_params* p, void* stream) {
    int rc = check_gemm_params("gguf_dequant_gemm", p);
    if (rc != LSG_OK) return rc;
    return dequant_gemm(p->type, p->M, p->N, p->K, p->A, p->B, p->C, p->N,
                        p->out_dtype == LSG_DTYPE_F32, static_cast<cudaStream_t>(stream));
}

extern "C" int lsg_gguf_dequant_blocks(const void* packed, float* out, int type,
                                       long long n_blocks, void* stream) {
    if (n_blocks == 0) return LSG_OK;
    if (!packed || !out || n_blocks < 0) return fail(LSG_ERR_INVALID, "gguf_dequant_blocks: bad argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (type) {
        case 0: return launch_db<0>(packed, out, n_blocks, s);
        case 1: return launch_db<1>(packed, out, n_blocks, s);
        case 2: return launch_db<2>(packed, out, n_blocks, s);
        case 3: return launch_db<3>(packed, out, n_blocks, s);
        case 4: return launch_db<4>(packed, out, n_blocks, s);
        case 5: return launch_db<5>(packed, out, n_blocks, s);
        case 6: return launch_db<6>(packed, out, n_blocks, s);
        case 7: return launch_db<7>(packed, out, n_blocks, s);
    }
    return fail(LSG_ERR_UNSUPPORTED, "gguf_dequant_blocks: unknown type %d", type);
}
