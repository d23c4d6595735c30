// Tensor-core path of the GGUF GEMMs on sm_100a: prefill ("mmq") and the grouped MoE
// GEMM when experts have many rows.
//
// Replaces the reference's int8 mma.sync kernels (csrc/sm120/gemm/gguf/mmq_mma/:
// mmq_kernel_32aligned.cuh:34-169, mmq_kernel_16subblock.cuh:36-155, launchers
// mmq_mma_dispatch.cu:52-91) and their grouped variants.  The reference multiplies int8
// tiles and rescales the int32 partial sums every 32 (or 16) values of K in registers:
//   C += dx[m,c] * (A[n,c] * dot_int8 + B[n,c] * sum qx[m,c]).
// With tcgen05 the accumulator lives in tensor memory, so a per-chunk rescale would mean
// draining it 128 times per row of a 4096-wide K.  This path therefore applies the scales
// BEFORE the multiply: both operands are turned into fp16 once per call,
//   w16[n,k] = fp16(A*Q + B)          (the weight's dequantized value)
//   x16[m,k] = fp16(d_x * q_x)        (the Q8_1 round trip of the activation)
// and one fp16 x fp16 -> fp32 tcgen05.mma sweep over the whole K does the rest.  The
// products are the same real numbers as the reference's, up to the fp16 rounding of each
// operand (2^-11 relative, unbiased), which lands far inside the 1e-3 bound.
//
// Kernel: persistent, warp-specialised.
//   warp 4      TMA producer: cp.async.bulk.tensor 2-D loads (128-byte swizzle) of a
//               128 x 64 activation tile and a 256 x 64 weight tile per stage, 4 stages;
//   warp 5      MMA issuer: one elected lane issues tcgen05.mma.cta_group::1.kind::f16
//               (M = 128, N = 256, K = 16) x 4 per stage, commits to the stage's "empty"
//               barrier, and after the last K block to the accumulator's "full" barrier;
//   warps 0-3   epilogue: tcgen05.ld of the 128 x 256 fp32 accumulator (each warp its 32
//               TMEM lanes), conversion, row-masked stores.  Two accumulators (2 x 256 of the
//               512 TMEM columns) let the epilogue of tile i overlap the MMAs of tile i+1.
// Work items are (m-tile, n-tile) pairs; m-tiles come either from a dense problem or from
// the device-built tile map of the grouped problem (routing.cu), so expert routing never
// touches the host.  Every mbarrier wait is time-limited; after a time-out all roles leave
// their loops, TMEM is freed, and the status word says so.
#include "common.cuh"
#include "formats.cuh"
#include "host.h"

#include "tcgen05.cuh"

namespace lsg {

using namespace tc;

namespace {

constexpr int BM = 128, BN = 256;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;   // 16 KB
constexpr int kBBytes = BN * BK * 2;   // 32 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTcThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kOutStageBytes = 4 * 32 * 128;   // 4 epilogue warps x 32 rows x 64 bf16: coalescing buffer of the gather route
constexpr int kTcSmem = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + kOutStageBytes;

struct TcArgs {
    void* C;                  // [rows, ldc] bf16 or f32
    int ldc;
    int out_f32;              // lsg_dtype of C: 0 bf16, 1 f32, 2 f16
    const float* alphas;      // optional per-expert output scale (grouped) or single value (dense)
    float alpha_host;         // output scale known on the host (used when alphas is null and it is not 1)
    void* const* C_ptrs;      // optional: n_out output matrices (this GPU's and its peers'), every tile is
    int n_out;                //   stored into each of them at column offset col_off (GEMM + all-gather)
    void* mc;                 // optional multicast address of those matrices: one multimem.st per 16 bytes
    int col_off;
    int K;
    int N;                    // columns of one problem (per expert)
    int n_tiles;              // ceil(N / BN)
    // dense: m_tiles = ceil(M / BM), tile_expert == nullptr
    // grouped: m_tiles = T_max, tile map and offsets on the device
    int m_tiles;
    int M;                    // dense: rows; grouped: total rows (for clamping)
    const int* tile_expert;
    const int* tile_mstart;
    const int* expert_offsets;
    unsigned int* status;
};

// ---------------------------------------------------------------------------
// The GEMM kernel
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kTcThreads, 1)
tc_gemm_f16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;   // [2]
    uint64_t* acc_empty = acc_full + 2;     // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* out_stage = smem + kStages * kStageBytes + 256;   // 16-byte aligned, behind the barriers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_wait_prior();  // operands were produced by the preparation kernels before this one

    const int kblocks = (a.K + BK - 1) / BK;
    const int total = a.m_tiles * a.n_tiles;

    if (warp == 4) {
        // ------------------------------ TMA producer ------------------------------
        // The whole warp walks the loop, one elected lane issues the copies (see the MMA issuer).
        {
            int s = 0;
            uint32_t lap = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok && !*abort_flag; w += gridDim.x) {
                const int t = w % a.m_tiles, j = w / a.m_tiles;
                int mstart = t * BM, brow0 = j * BN;
                if (a.tile_expert) {
                    const int e = a.tile_expert[t];
                    if (e < 0) continue;
                    mstart = a.tile_mstart[t];
                    brow0 = e * a.N + j * BN;
                }
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (lap > 0)
                        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty[s], (lap - 1) & 1, a.status, kDevWaitEmpty));
                    if (!ok) break;
                    uint8_t* sA = smem + s * kStageBytes;
                    uint8_t* sB = sA + kABytes;
                    if (elect_one()) {
                        mbar_arrive_expect_tx(&full[s], kStageBytes);
                        tma_load_2d(sA, &tmA, kb * BK, mstart, &full[s]);
                        tma_load_2d(sB, &tmB, kb * BK, brow0, &full[s]);
                    }
                    __syncwarp();
                    if (++s == kStages) {
                        s = 0;
                        ++lap;
                    }
                }
            }
            if (!ok) *abort_flag = 1;
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        // The whole warp walks the loop and one elected lane issues: descriptors and addresses
        // are then warp-uniform values (an issue inside a one-lane branch costs about three
        // times as long).
        constexpr uint32_t idesc = idesc_f16(BM, BN);
        int s = 0, tile_i = 0;
        uint32_t lap = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok && !*abort_flag; w += gridDim.x) {
            const int t = w % a.m_tiles;
            if (a.tile_expert && a.tile_expert[t] < 0) continue;
            const int ab = tile_i & 1;
            if (tile_i >= 2)
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&acc_empty[ab], ((tile_i >> 1) - 1) & 1, a.status, kDevWaitTmem));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + ab * BN;
            for (int kb = 0; kb < kblocks; ++kb) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&full[s], lap & 1, a.status, kDevWaitFull));
                if (!ok) break;
                tc_fence_after();
                const uint32_t sA = smem_u32(smem + s * kStageBytes);
                const uint64_t adesc = smem_desc_sw128(sA);
                const uint64_t bdesc = smem_desc_sw128(sA + kABytes);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        // 16 fp16 = 32 bytes further along K inside the swizzle atom: +2 in
                        // the (address >> 4) field of the descriptors
                        tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(&empty[s]);  // the stage is free once these MMAs have read it
                }
                __syncwarp();
                if (++s == kStages) {
                    s = 0;
                    ++lap;
                }
            }
            if (!ok) break;
            if (elect_one()) tc_commit(&acc_full[ab]);  // accumulator complete
            __syncwarp();
            ++tile_i;
        }
        if (!ok) *abort_flag = 1;
    } else {
        // ------------------------------ epilogue (warps 0-3) ----------------------
        int tile_i = 0;
        for (int w = blockIdx.x; w < total && !*abort_flag; w += gridDim.x) {
            const int t = w % a.m_tiles, j = w / a.m_tiles;
            int mstart = t * BM, mend = a.M;
            if (a.tile_expert) {
                const int e = a.tile_expert[t];
                if (e < 0) continue;
                mstart = a.tile_mstart[t];
                mend = a.expert_offsets[e + 1];
            }
            const int ab = tile_i & 1;
            // warp-uniform outcome: the tensor-memory loads below need the whole warp
            const bool landed = __all_sync(0xffffffffu,
                                           mbar_wait_bounded(&acc_full[ab], (tile_i >> 1) & 1, a.status, kDevWaitMma));
            if (!landed) {
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int row = mstart + warp * 32 + lane;
            const bool row_ok = row < mend;
            const int n0 = j * BN;
            float alpha = a.alpha_host;
            if (a.alphas) alpha = a.tile_expert ? a.alphas[a.tile_expert[t]] : a.alphas[0];
            const bool scaled = a.alphas != nullptr || alpha != 1.0f;
            // Gather route with 16-bit outputs: 64 columns at a time go through a swizzled
            // shared-memory buffer so that every store instruction writes four 128-byte row
            // segments (peer stores over NVLink travel as whole 128-byte packets instead of
            // 16-byte pieces).  Needs the whole tile inside the matrix and aligned rows.
            const bool staged_out = a.n_out > 0 && a.out_f32 != LSG_DTYPE_F32 && n0 + BN <= a.N &&
                                    ((a.ldc | a.col_off) & 7) == 0;
            if (staged_out) {
                const bool f16 = a.out_f32 == LSG_DTYPE_F16;
                const uint32_t buf = smem_u32(out_stage) + static_cast<uint32_t>(warp * 4096);
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    uint32_t pk[32];
#pragma unroll
                    for (int hc = 0; hc < 2; ++hc) {
                        uint32_t r[32];
                        tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + ab * BN + c + 32 * hc, r);
#pragma unroll
                        for (int h = 0; h < 16; ++h) {
                            const float v0 = __uint_as_float(r[2 * h]) * (scaled ? alpha : 1.0f);
                            const float v1 = __uint_as_float(r[2 * h + 1]) * (scaled ? alpha : 1.0f);
                            if (f16) {
                                const __half2 v = __floats2half2_rn(v0, v1);
                                pk[16 * hc + h] = *reinterpret_cast<const uint32_t*>(&v);
                            } else {
                                const __nv_bfloat162 v = __floats2bfloat162_rn(v0, v1);
                                pk[16 * hc + h] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                        }
                    }
                    __syncwarp();   // the previous 64 columns have been read out of the buffer
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(buf + lane * 128 + ((q ^ (lane & 7)) << 4)),
                                     "r"(pk[4 * q]), "r"(pk[4 * q + 1]), "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
                                     : "memory");
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3), q = lane & 7;
                        uint4 v;
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                                     : "r"(buf + rr * 128 + ((q ^ (rr & 7)) << 4)));
                        const int grow = mstart + warp * 32 + rr;
                        if (grow < mend) {
                            const size_t o = static_cast<size_t>(grow) * a.ldc + a.col_off + n0 + c + q * 8;
                            if (a.mc) {
                                // one store into the NVLink multicast object: the switch replicates it
                                // to every rank's copy of the output, this one included
                                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                                                 static_cast<uint16_t*>(a.mc) + o),
                                             "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                                             "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                                             : "memory");
                            } else {
                                for (int po = 0; po < a.n_out; ++po)
                                    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(a.C_ptrs[po]) + o) = v;
                            }
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + ab * BN + c, r);
                if (row_ok && n0 + c < a.N) {
                    if (scaled) {
#pragma unroll
                        for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) * alpha);
                    }
                    const size_t o = static_cast<size_t>(row) * a.ldc + a.col_off + n0 + c;
                    const int ncols = min(32, a.N - (n0 + c));
                    const int n_out = a.n_out > 0 ? a.n_out : 1;
                    if (a.out_f32 == LSG_DTYPE_F32) {
                        for (int po = 0; po < n_out; ++po) {
                            float* dst = static_cast<float*>(a.n_out > 0 ? a.C_ptrs[po] : a.C) + o;
                            if (ncols == 32 && ((a.ldc | a.col_off) & 3) == 0) {
#pragma unroll
                                for (int q = 0; q < 8; ++q)
                                    reinterpret_cast<uint4*>(dst)[q] =
                                        make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                            } else {
                                for (int q = 0; q < ncols; ++q) dst[q] = __uint_as_float(r[q]);
                            }
                        }
                    } else {
                        const bool f16 = a.out_f32 == LSG_DTYPE_F16;
                        uint32_t pk[16];
#pragma unroll
                        for (int h = 0; h < 16; ++h) {
                            const float v0 = __uint_as_float(r[2 * h]);
                            const float v1 = __uint_as_float(r[2 * h + 1]);
                            if (f16) {
                                const __half2 v = __floats2half2_rn(v0, v1);
                                pk[h] = *reinterpret_cast<const uint32_t*>(&v);
                            } else {
                                const __nv_bfloat162 v = __floats2bfloat162_rn(v0, v1);
                                pk[h] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                        }
                        for (int po = 0; po < n_out; ++po) {
                            uint16_t* dst = static_cast<uint16_t*>(a.n_out > 0 ? a.C_ptrs[po] : a.C) + o;
                            if (ncols == 32 && ((a.ldc | a.col_off) & 7) == 0) {
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    reinterpret_cast<uint4*>(dst)[q] =
                                        make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
                            } else {
                                for (int q = 0; q < ncols; ++q)
                                    dst[q] = static_cast<uint16_t>((q & 1) ? (pk[q >> 1] >> 16) : (pk[q >> 1] & 0xFFFFu));
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[ab]);
            ++tile_i;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Operand preparation
// ---------------------------------------------------------------------------
// Packed GGUF rows -> fp16 [rows, K].  One thread per 32 values.  With B_ptrs (grouped
// case) blockIdx.y is the expert and experts without rows are skipped.
template <int T>
__global__ void weights_to_f16_kernel(const uint8_t* __restrict__ W, const void* const* __restrict__ B_ptrs,
                                      const int32_t* __restrict__ expert_offsets, __half* __restrict__ out,
                                      int N, int K, long long n_blocks_per_matrix) {
    pdl_launch_dependents();
    pdl_wait_prior();
    using F = Fmt<T>;
    const int e = blockIdx.y;
    const uint8_t* base = W;
    if (B_ptrs) {
        if (expert_offsets[e + 1] - expert_offsets[e] <= 0) return;
        base = static_cast<const uint8_t*>(B_ptrs[e]);
        if (!base) return;
    }
    // one thread per 32 values: 64 contiguous bytes out per thread, 2 KB per warp
    constexpr int CPB = F::VALS / 32;
    const long long ch = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (ch >= n_blocks_per_matrix * CPB) return;
    const long long b = ch / CPB;
    const int c = static_cast<int>(ch - b * CPB);
    float v[32];
    dequant_chunk32<T>(base + b * F::BYTES, c, v);
    __half* dst = out + (static_cast<long long>(e) * N * K) + ch * 32;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
        uint32_t p[4];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            const __half2 hv = __floats2half2_rn(v[i + 2 * h], v[i + 2 * h + 1]);
            p[h] = *reinterpret_cast<const uint32_t*>(&hv);
        }
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(p[0], p[1], p[2], p[3]);
    }
}

// bf16 x[M,K] -> fp16 of the Q8_1 round trip: d_h * rn(x / d) with d = amax/127 per 32
// values and d_h its fp16 rounding (what the integer paths multiply by).  Four lanes per
// block, eight values per lane.
__global__ void __launch_bounds__(256)
x_q8_1_roundtrip_f16_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ out, long long n_blocks) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long task = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    const bool live = task < n_blocks * 4;
    const long long tk = live ? task : 0;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + tk);
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
    if (!live) return;
    const float d = amax / 127.0f;
    const float rcp = (amax == 0.0f) ? 0.0f : 1.0f / d;
    const float dh = __half2float(__float2half(d));
    uint32_t p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float r[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            r[h] = dh * q8_round_f(v[2 * i + h], d, rcp);   // same integer as rn(fl(x / d))
        }
        const __half2 hv = __floats2half2_rn(r[0], r[1]);
        p[i] = *reinterpret_cast<const uint32_t*>(&hv);
    }
    reinterpret_cast<uint4*>(out)[tk] = make_uint4(p[0], p[1], p[2], p[3]);
}

// ---------------------------------------------------------------------------
// Host
// ---------------------------------------------------------------------------
int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcArgs& a, int max_items, cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(tc_gemm_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    int grid = sm_count();
    if (grid > max_items) grid = max_items;
    if (grid < 1) grid = 1;
    LSG_CUDA_TRY(launch_kernel(tc_gemm_f16_kernel, dim3(grid), dim3(kTcThreads), kTcSmem, s, true, tmA, tmB, a));
    return LSG_OK;
}

template <int T>
int launch_w16(const void* W, const void* const* B_ptrs, const int32_t* offs, __half* out, int E, int N,
               int K, cudaStream_t s) {
    const long long nb = static_cast<long long>(N) * (K / Fmt<T>::VALS);
    const long long chunks = nb * (Fmt<T>::VALS / 32);
    dim3 grid(static_cast<unsigned>((chunks + 255) / 256), E);
    LSG_CUDA_TRY(launch_kernel(weights_to_f16_kernel<T>, grid, dim3(256), 0, s, true,
                               static_cast<const uint8_t*>(W), B_ptrs, offs, out, N, K, nb));
    return LSG_OK;
}

int weights_to_f16(int type, const void* W, const void* const* B_ptrs, const int32_t* offs, __half* out,
                   int E, int N, int K, cudaStream_t s) {
    switch (type) {
        case 0: return launch_w16<0>(W, B_ptrs, offs, out, E, N, K, s);
        case 1: return launch_w16<1>(W, B_ptrs, offs, out, E, N, K, s);
        case 2: return launch_w16<2>(W, B_ptrs, offs, out, E, N, K, s);
        case 3: return launch_w16<3>(W, B_ptrs, offs, out, E, N, K, s);
        case 4: return launch_w16<4>(W, B_ptrs, offs, out, E, N, K, s);
        case 5: return launch_w16<5>(W, B_ptrs, offs, out, E, N, K, s);
        case 6: return launch_w16<6>(W, B_ptrs, offs, out, E, N, K, s);
        case 7: return launch_w16<7>(W, B_ptrs, offs, out, E, N, K, s);
    }
    return fail(LSG_ERR_UNSUPPORTED, "gguf mmq: unknown type %d", type);
}

int x_to_f16(const void* x_bf16, __half* out, long long rows, int K, cudaStream_t s) {
    const long long nb = rows * (K / 32);
    if (nb == 0) return LSG_OK;
    LSG_CUDA_TRY(launch_kernel(x_q8_1_roundtrip_f16_kernel, dim3(static_cast<unsigned>((nb * 4 + 255) / 256)), dim3(256),
                               0, s, true, static_cast<const __nv_bfloat16*>(x_bf16), out, nb));
    return LSG_OK;
}

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

// Scratch of the tensor-core path: fp16 activations + fp16 weights of E matrices.
size_t mmq_scratch_bytes(long long rows, int K, int E, int N) {
    return align256(static_cast<size_t>(rows) * K * 2) + align256(static_cast<size_t>(E) * N * K * 2);
}

// Dense: C[M,N] = x16 . w16^T.
int mmq_dense(int type, int M, int N, int K, const void* A, const void* W, void* C, int out_f32, void* ws,
              size_t ws_bytes, cudaStream_t s, const MmqOutputs* outs) {
    if (M == 0 || N == 0) return LSG_OK;
    // Weights decoded inside the GEMM wherever that kernel has a decoder for the type: it reads
    // the packed weights once per token tile (up to 384 rows) and measured faster than one
    // expansion pass plus the plain fp16 GEMM at every M (14336 x 4096 Q4_K, M = 4096: 0.399 ms
    // against 0.489 ms).  The all-gather epilogue for large M stays with the prepared-operand
    // kernel, whose epilogue stores whole 128-byte segments into the peers.
    if (tc_fused_available(type) && (M <= 2048 || outs == nullptr || tc_fused_forced()))
        return tc_fused_dense(type, M, N, K, A, W, C, outs ? outs->ldc : N, out_f32 ? LSG_DTYPE_F32 : LSG_DTYPE_BF16,
                              ws, ws_bytes, s, outs);
    if (K % 8 != 0) return fail(LSG_ERR_UNSUPPORTED, "gguf_mmq: K must be a multiple of 8");
    const size_t need = mmq_scratch_bytes(M, K, 1, N);
    if (!ws || ws_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "gguf_mmq: workspace too small (have %zu, need %zu)",
                    ws ? ws_bytes : size_t(0), need);
    if (reinterpret_cast<uintptr_t>(ws) & 255) return fail(LSG_ERR_ALIGNMENT, "gguf_mmq: workspace must be 256-byte aligned");
    __half* x16 = static_cast<__half*>(ws);
    __half* w16 = reinterpret_cast<__half*>(static_cast<uint8_t*>(ws) + align256(static_cast<size_t>(M) * K * 2));
    int rc = x_to_f16(A, x16, M, K, s);
    if (rc != LSG_OK) return rc;
    rc = weights_to_f16(type, W, nullptr, nullptr, w16, 1, N, K, s);
    if (rc != LSG_OK) return rc;
    CUtensorMap tmA, tmB;
    rc = make_map(&tmA, x16, M, K, BM);
    if (rc != LSG_OK) return rc;
    rc = make_map(&tmB, w16, N, K, BN);
    if (rc != LSG_OK) return rc;
    TcArgs a = {};
    a.alpha_host = 1.0f;
    a.C = C; a.ldc = N; a.out_f32 = out_f32 ? LSG_DTYPE_F32 : LSG_DTYPE_BF16; a.K = K; a.N = N;
    if (outs) {
        a.C_ptrs = outs->C_ptrs; a.n_out = outs->n_out; a.col_off = outs->col_off; a.ldc = outs->ldc; a.mc = outs->mc_ptr;
    }
    a.n_tiles = (N + BN - 1) / BN;
    a.m_tiles = (M + BM - 1) / BM;
    a.M = M;
    a.status = device_status_word();
    return launch_tc(tmA, tmB, a, a.m_tiles * a.n_tiles, s);
}

// Grouped: rows routed by the device-built tile map (tile_m must be BM = 128).
int mmq_grouped(int type, int T, int E, int N, int K, const void* A, const void* const* B_ptrs,
                const int32_t* expert_offsets, void* D, int out_f32, const int* tile_expert,
                const int* tile_mstart, int t_max, void* scratch, size_t scratch_bytes, cudaStream_t s) {
    if (K % 8 != 0) return fail(LSG_ERR_UNSUPPORTED, "gguf grouped mmq: K must be a multiple of 8");
    const size_t need = mmq_scratch_bytes(T, K, E, N);
    if (!scratch || scratch_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "gguf grouped mmq: scratch too small (have %zu, need %zu)",
                    scratch ? scratch_bytes : size_t(0), need);
    __half* x16 = static_cast<__half*>(scratch);
    __half* w16 = reinterpret_cast<__half*>(static_cast<uint8_t*>(scratch) + align256(static_cast<size_t>(T) * K * 2));
    int rc = x_to_f16(A, x16, T, K, s);
    if (rc != LSG_OK) return rc;
    rc = weights_to_f16(type, nullptr, B_ptrs, expert_offsets, w16, E, N, K, s);
    if (rc != LSG_OK) return rc;
    CUtensorMap tmA, tmB;
    rc = make_map(&tmA, x16, T, K, BM);
    if (rc != LSG_OK) return rc;
    rc = make_map(&tmB, w16, static_cast<long long>(E) * N, K, BN);
    if (rc != LSG_OK) return rc;
    TcArgs a = {};
    a.alpha_host = 1.0f;
    a.C = D; a.ldc = N; a.out_f32 = out_f32 ? LSG_DTYPE_F32 : LSG_DTYPE_BF16; a.K = K; a.N = N;
    a.n_tiles = (N + BN - 1) / BN;
    a.m_tiles = t_max;
    a.M = T;
    a.tile_expert = tile_expert;
    a.tile_mstart = tile_mstart;
    a.expert_offsets = expert_offsets;
    a.status = device_status_word();
    return launch_tc(tmA, tmB, a, a.m_tiles * a.n_tiles, s);
}

// C = alpha * A16 . B16^T on prepared fp16 operands.  Dense when tile_expert is null
// (M rows), otherwise grouped through the device-built tile map; B16 then holds E
// matrices of N rows each.
int tc_gemm_f16(const void* A16, long long a_rows, const void* B16, long long b_rows, int K, int N,
                void* C, int out_dtype, const float* alphas, int M, const int* tile_expert,
                const int* tile_mstart, int t_max, const int32_t* expert_offsets, cudaStream_t s,
                float alpha_host) {
    CUtensorMap tmA, tmB;
    int rc = make_map(&tmA, A16, a_rows, K, BM);
    if (rc != LSG_OK) return rc;
    rc = make_map(&tmB, B16, b_rows, K, BN);
    if (rc != LSG_OK) return rc;
    TcArgs a = {};
    a.C = C; a.ldc = N; a.out_f32 = out_dtype; a.alphas = alphas; a.alpha_host = alpha_host; a.K = K; a.N = N;
    a.n_tiles = (N + BN - 1) / BN;
    a.m_tiles = tile_expert ? t_max : (M + BM - 1) / BM;
    a.M = M;
    a.tile_expert = tile_expert;
    a.tile_mstart = tile_mstart;
    a.expert_offsets = expert_offsets;
    a.status = device_status_word();
    if (a.m_tiles <= 0) return LSG_OK;
    return launch_tc(tmA, tmB, a, a.m_tiles * a.n_tiles, s);
}

}  // namespace lsg

using namespace lsg;

extern "C" size_t lsg_gguf_mmq_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    const size_t prepared = mmq_scratch_bytes(M, K, 1, N);
    const size_t fused = tc_fused_dense_scratch_bytes(M, N, K);
    return prepared > fused ? prepared : fused;
}

extern "C" int lsg_gguf_mmq(const lsg_gguf_mmvq_params* p, void* workspace, size_t workspace_bytes,
                            void* stream) {
    int rc = check_gemm_params("gguf_mmq", p);
    if (rc != LSG_OK) return rc;
    if (p->M == 0 || p->N == 0) return LSG_OK;
    if (!p->A || !p->B || !p->C) return fail(LSG_ERR_INVALID, "gguf_mmq: null pointer");
    return mmq_dense(p->type, p->M, p->N, p->K, p->A, p->B, p->C, p->out_dtype == LSG_DTYPE_F32, workspace,
                     workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" size_t lsg_gguf_gemm_bf16_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    return tc_fused_bf16_scratch_bytes(M, N, K);
}

extern "C" int lsg_gguf_gemm_bf16(const lsg_gguf_mmvq_params* p, void* workspace, size_t workspace_bytes,
                                  void* stream) {
    int rc = check_gemm_params("gguf_gemm_bf16", p);
    if (rc != LSG_OK) return rc;
    if (p->M == 0 || p->N == 0) return LSG_OK;
    if (!p->A || !p->B || !p->C) return fail(LSG_ERR_INVALID, "gguf_gemm_bf16: null pointer");
    return tc_fused_dense_bf16(p->type, p->M, p->N, p->K, p->A, p->B, p->C, p->N, p->out_dtype, workspace,
                               workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int lsg_gguf_mmq_gather_mc(const lsg_gguf_mmvq_params* p, void* const* C_ptrs, int n_out, int ldc,
                                      int col_offset, void* multicast_ptr, void* workspace, size_t workspace_bytes,
                                      void* stream) {
    int rc = check_gemm_params("gguf_mmq_gather", p);
    if (rc != LSG_OK) return rc;
    if (p->M == 0 || p->N == 0) return LSG_OK;
    if (!p->A || !p->B || !C_ptrs) return fail(LSG_ERR_INVALID, "gguf_mmq_gather: null pointer");
    if (n_out < 1 || n_out > 64 || col_offset < 0 || ldc < col_offset + p->N)
        return fail(LSG_ERR_INVALID, "gguf_mmq_gather: need 1 <= n_out <= 64 and col_offset + N <= ldc");
    if (reinterpret_cast<uintptr_t>(multicast_ptr) & 15)
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmq_gather: the multicast address must be 16-byte aligned");
    MmqOutputs outs = {C_ptrs, n_out, ldc, col_offset, multicast_ptr};
    return mmq_dense(p->type, p->M, p->N, p->K, p->A, p->B, nullptr, p->out_dtype == LSG_DTYPE_F32, workspace,
                     workspace_bytes, static_cast<cudaStream_t>(stream), &outs);
}

extern "C" int lsg_gguf_mmq_gather(const lsg_gguf_mmvq_params* p, void* const* C_ptrs, int n_out, int ldc,
                                   int col_offset, void* workspace, size_t workspace_bytes, void* stream) {
    return lsg_gguf_mmq_gather_mc(p, C_ptrs, n_out, ldc, col_offset, nullptr, workspace, workspace_bytes, stream);
}
