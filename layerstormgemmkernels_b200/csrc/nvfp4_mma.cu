// NVFP4 GEMM on the block-scaled tensor-core instruction of sm_100a:
//   D[m, n] = alpha * sum_k (a[m,k] * sfa[m, k/16]) * (b[n,k] * sfb[n, k/16])
// a, b: packed e2m1 (two per byte, low nibble = even k), sfa / sfb: one ue4m3 scale per 16
// values in the 128-row x 4-group interleaved layout, fp32 accumulation in tensor memory.
//
// This is the arithmetic the reference obtains from a CUTLASS block-scaled kernel for sm_120
// (csrc/sm120/gemm/nvfp4/nvfp4_grouped_gemm.cu:39-105, 227-365; nvfp4_gemm.cu:50-100), done
// here with tcgen05.mma.kind::mxf4nvf4.block_scale: the packed operands travel from HBM to
// shared memory by TMA exactly as the API hands them over (0.5 byte per value, no expanded
// copy anywhere), the scale factors by bulk copies of whole 512-byte atoms - the API's
// interleaved layout is, atom by atom, the layout tcgen05.cp wants - and from shared memory
// into tensor memory right before the MMAs that use them.
//
// Kernel: persistent, warp-specialised, one CTA per SM.  A work item is a 128-row token tile
// times a PAIR of neighbouring 128-column output tiles: the A tile is copied once and feeds two
// MMAs per K step (the kernel is bound by the bytes that come out of L2 and through shared
// memory, not by the tensor pipe; a pair moves 54 KB per stage for twice the work of 36 KB).
//   warp 4     producer (whole warp walks, an elected lane issues): per K tile of 256 values one
//              TMA box (128 rows x 128 bytes, 128-byte swizzle) of A and one per output tile of
//              B, plus the four scale atoms of each; 4 stages of 54 KB;
//   warp 5     MMA issuer (same form): 12 x tcgen05.cp (scale atoms -> tensor memory, replicated
//              over the four lane quadrants), then 2 x 4 tcgen05.mma (M = 128, N = 128, K = 64),
//              commit;
//   warps 0-3  epilogue: tcgen05.ld of the two 128 x 128 fp32 accumulators into packed 16-bit
//              registers (alpha applied), the accumulators are handed back to the MMA warp,
//              then row-masked 16-byte stores.
// Tensor memory: the pair's accumulators in columns 0..255, A scales in 256..271, B scales in
// 272..287 and 288..303 (four columns per MMA: lane r % 32 of every quadrant holds the sixteen
// bytes [row quadrant][K group] of rows r % 32 + 32 * {0,1,2,3}).
// A tile's rows are tokens (M side of the instruction), its columns weight rows: with
// tokens on the 128-lane side a thread's accumulator row is one output row and stores are
// contiguous.  Work items are (token tile, weight tile) pairs; token tiles come from a dense
// problem or from the device-built tile map of the grouped one.  Every wait is time-limited.
#include "common.cuh"
#include "host.h"
#include "tcgen05.cuh"

namespace lsg {

using namespace tc;

namespace {

constexpr int FM = 128, FN = 128;
constexpr int FKB = 128;                 // bytes of K per stage row = 256 values
// A CTA works on a pair of neighbouring 128-column output tiles that share their 128 rows of A:
// one copy of the A tile feeds two MMAs per K step, which takes a quarter off the bytes that come
// out of L2 and through shared memory per flop (the limit of this kernel, not the tensor pipe).
constexpr int kFStages = 4;
constexpr int kFABytes = FM * FKB;       // 16 KB
constexpr int kFBBytes = FN * FKB;       // 16 KB per output tile of the pair
constexpr int kFSfBytes = 4 * 512;       // four 128-row x 4-group atoms
constexpr int kFStageBytes = kFABytes + 2 * kFBBytes + 3 * kFSfBytes;   // 54 KB
constexpr int kFThreads = 192;
constexpr int kFTmemCols = 512;
constexpr int kFSfaCol = 256, kFSfbCol = 272;   // scales of A; of B, 16 columns per tile of the pair
constexpr int kFSmem = kFStages * kFStageBytes + 1024 + 256;

struct F4Args {
    void* D;
    int ldd;
    int out_dtype;
    const float* alphas;      // per expert (grouped) or null
    float alpha_host;
    const uint8_t* sfa;       // interleaved scale atoms of A
    const uint8_t* sfb;       // of B; expert e at sfb + e * sfb_expert_bytes
    long long sfb_expert_bytes;
    int K, N;
    int n_tiles, m_tiles;
    int M;
    const int* tile_expert;
    const int* tile_mstart;
    const int32_t* expert_offsets;
    const int32_t* sf_offsets;
    unsigned int* status;
};

// Shared-memory matrix descriptor of one scale atom for tcgen05.cp: 32 rows of 16 bytes, no
// swizzle, 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sf_atom(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;   // stride byte offset between 8-row groups
    d |= static_cast<uint64_t>(1) << 46;          // descriptor version
    return d;
}

__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}

__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// Instruction descriptor of kind::mxf4nvf4: A and B e2m1 (format 1), K-major, ue4m3 scales
// (format 0), scale-factor ids 0, K = 64.
__device__ __forceinline__ constexpr uint32_t idesc_nvf4(int m, int n) {
    return (1u << 7) | (1u << 10)                    // A, B format: E2M1
           | (static_cast<uint32_t>(n >> 3) << 17)   // N / 8
           | (0u << 23)                              // scale format UE4M3
           | (static_cast<uint32_t>(m >> 4) << 24);  // M / 16
}

__global__ void __launch_bounds__(kFThreads, 1)
nvfp4_mma_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const F4Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kFStages * kFStageBytes);
    uint64_t* empty = full + kFStages;
    uint64_t* acc_full = empty + kFStages;   // [2]
    uint64_t* acc_empty = acc_full + 2;      // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kFStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) tmem_alloc(tmem_slot, kFTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_wait_prior();

    const int ktiles = (a.K + 255) / 256;
    const int gpr = a.K >> 4;                        // scale groups per row (a multiple of 4)
    const long long sf_tile_bytes = 128ll * gpr;     // one 128-row tile of scale atoms
    const int n_pairs = (a.n_tiles + 1) >> 1;
    const int total = a.m_tiles * n_pairs;

    if (warp == 4) {
        // ------------------------------ producer ------------------------------
        // The whole warp walks the loop, one elected lane issues the copies of a stage
        // (see the MMA issuer for why).
        int s = 0;
        uint32_t lap = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok && !*abort_flag; w += gridDim.x) {
            const int t = w % a.m_tiles, j = 2 * (w / a.m_tiles);
            const bool two = j + 1 < a.n_tiles;
            int mstart = t * FM;
            long long brow0 = static_cast<long long>(j) * FN;
            const uint8_t* sfa_tile = a.sfa + static_cast<long long>(t) * sf_tile_bytes;
            const uint8_t* sfb_tile = a.sfb + static_cast<long long>(j) * sf_tile_bytes;
            if (a.tile_expert) {
                const int e = a.tile_expert[t];
                if (e < 0) continue;
                mstart = a.tile_mstart[t];
                brow0 += static_cast<long long>(e) * a.N;
                const int local_tile = (mstart - a.expert_offsets[e]) >> 7;
                sfa_tile = a.sfa + (static_cast<long long>(a.sf_offsets[e]) + 128ll * local_tile) * gpr;
                sfb_tile += static_cast<long long>(e) * a.sfb_expert_bytes;
            }
            for (int kt = 0; kt < ktiles; ++kt) {
                if (lap > 0)
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty[s], (lap - 1) & 1, a.status, kDevWaitEmpty));
                if (!ok) break;
                const int atoms = min(4, (a.K - kt * 256) >> 6);   // 64-value K blocks in this tile
                uint8_t* sA = smem + s * kFStageBytes;
                uint8_t* sB = sA + kFABytes;
                uint8_t* sSA = sB + 2 * kFBBytes;
                uint8_t* sSB = sSA + kFSfBytes;
                if (elect_one()) {
                    const uint32_t sfb = static_cast<uint32_t>(atoms * 512);
                    mbar_arrive_expect_tx(&full[s], static_cast<uint32_t>(kFABytes + kFBBytes + 2 * sfb +
                                                                        (two ? kFBBytes + sfb : 0)));
                    tma_load_2d(sA, &tmA, kt * FKB, mstart, &full[s]);
                    tma_load_2d(sB, &tmB, kt * FKB, static_cast<int>(brow0), &full[s]);
                    bulk_g2s(sSA, sfa_tile + static_cast<long long>(kt) * 2048, sfb, &full[s]);
                    bulk_g2s(sSB, sfb_tile + static_cast<long long>(kt) * 2048, sfb, &full[s]);
                    if (two) {
                        tma_load_2d(sB + kFBBytes, &tmB, kt * FKB, static_cast<int>(brow0) + FN, &full[s]);
                        bulk_g2s(sSB + kFSfBytes, sfb_tile + sf_tile_bytes + static_cast<long long>(kt) * 2048, sfb, &full[s]);
                    }
                }
                __syncwarp();
                if (++s == kFStages) {
                    s = 0;
                    ++lap;
                }
            }
        }
        if (!ok) *abort_flag = 1;
    } else if (warp == 5) {
        // ------------------------------ MMA issuer ------------------------------
        // The whole warp walks the loop and one elected lane issues: in converged code the
        // descriptors and addresses are warp-uniform values, and an issue costs about 20 cycles;
        // the same instructions inside a one-lane branch measured about 60 cycles each, which
        // with the scale copies and MMAs of a stage was three times the tensor time.
        constexpr uint32_t idesc = idesc_nvf4(FM, FN);
        int s = 0, tile_i = 0;
        uint32_t lap = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok && !*abort_flag; w += gridDim.x) {
            const int t = w % a.m_tiles, j = 2 * (w / a.m_tiles);
            if (a.tile_expert && a.tile_expert[t] < 0) continue;
            const bool two = j + 1 < a.n_tiles;
            // one accumulator pair: the epilogue releases it as soon as it has read it out
            if (tile_i >= 1)
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&acc_empty[0], (tile_i - 1) & 1, a.status, kDevWaitTmem));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base;
            for (int kt = 0; kt < ktiles; ++kt) {
                ok = __all_sync(0xffffffffu, mbar_wait_bounded(&full[s], lap & 1, a.status, kDevWaitFull));
                if (!ok) break;
                tc_fence_after();
                const int atoms = min(4, (a.K - kt * 256) >> 6);
                const uint32_t sA = smem_u32(smem + s * kFStageBytes);
                const uint32_t sSA = sA + kFABytes + 2 * kFBBytes, sSB = sSA + kFSfBytes;
                const uint64_t adesc = smem_desc_sw128(sA);
                const uint64_t bdesc = smem_desc_sw128(sA + kFABytes);
                const uint64_t bdesc1 = smem_desc_sw128(sA + kFABytes + kFBBytes);
                if (elect_one()) {
                    for (int k = 0; k < atoms; ++k) {
                        tc_cp_sf(tmem_base + kFSfaCol + 4 * k, smem_desc_sf_atom(sSA + 512 * k));
                        tc_cp_sf(tmem_base + kFSfbCol + 4 * k, smem_desc_sf_atom(sSB + 512 * k));
                        if (two) tc_cp_sf(tmem_base + kFSfbCol + 16 + 4 * k, smem_desc_sf_atom(sSB + kFSfBytes + 512 * k));
                    }
                    for (int k = 0; k < atoms; ++k) {
                        // 64 values = 32 bytes further along K inside the swizzle atom
                        const uint32_t acc = (kt | k) != 0 ? 1u : 0u;
                        tc_mma_nvf4(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, tmem_base + kFSfaCol + 4 * k,
                                    tmem_base + kFSfbCol + 4 * k, acc);
                        if (two)
                            tc_mma_nvf4(d_tmem + FN, adesc + 2 * k, bdesc1 + 2 * k, idesc, tmem_base + kFSfaCol + 4 * k,
                                        tmem_base + kFSfbCol + 16 + 4 * k, acc);
                    }
                    tc_commit(&empty[s]);
                }
                __syncwarp();
                if (++s == kFStages) {
                    s = 0;
                    ++lap;
                }
            }
            if (!ok) break;
            if (elect_one()) tc_commit(&acc_full[0]);
            __syncwarp();
            ++tile_i;
        }
        if (!ok) *abort_flag = 1;
    } else {
        // ------------------------------ epilogue (warps 0-3) ------------------------------
        int tile_i = 0;
        for (int w = blockIdx.x; w < total && !*abort_flag; w += gridDim.x) {
            const int t = w % a.m_tiles, j = 2 * (w / a.m_tiles);
            int mstart = t * FM, mend = a.M;
            float alpha = a.alpha_host;
            if (a.tile_expert) {
                const int e = a.tile_expert[t];
                if (e < 0) continue;
                mstart = min(a.tile_mstart[t], a.M);
                mend = min(a.expert_offsets[e + 1], a.M);
                if (a.alphas) alpha = a.alphas[e];
            } else if (a.alphas) {
                alpha = a.alphas[0];
            }
            const bool landed = __all_sync(0xffffffffu,
                                           mbar_wait_bounded(&acc_full[0], tile_i & 1, a.status, kDevWaitMma));
            if (!landed) {
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const int row = mstart + warp * 32 + lane;
            const bool row_ok = row < mend;
            const int n0 = j * FN;
            const int ncols_all = min(2 * FN, a.N - n0);           // live columns of the pair
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
            auto release = [&]() {
                tc_fence_before();
                __syncwarp();
                if (elect_one()) mbar_arrive(&acc_empty[0]);
            };
            const bool vec_ok = (a.ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(a.D) & 15) == 0 && (a.N & 31) == 0;
            if (a.out_dtype != LSG_DTYPE_F32 && vec_ok) {
                // 16-bit outputs: the whole pair is read out of tensor memory into packed registers
                // first, the accumulators are handed back to the MMA warp, and only then stored.
                const bool f16 = a.out_dtype == LSG_DTYPE_F16;
                uint32_t pk[8][16];
#pragma unroll
                for (int c8 = 0; c8 < 8; ++c8) {
                    if (c8 * 32 < ncols_all) {
                        uint32_t r[32];
                        tmem_ld32(t_lane + c8 * 32, r);
#pragma unroll
                        for (int h = 0; h < 16; ++h) {
                            const float v0 = __uint_as_float(r[2 * h]) * alpha;
                            const float v1 = __uint_as_float(r[2 * h + 1]) * alpha;
                            if (f16) {
                                const __half2 v = __floats2half2_rn(v0, v1);
                                pk[c8][h] = *reinterpret_cast<const uint32_t*>(&v);
                            } else {
                                const __nv_bfloat162 v = __floats2bfloat162_rn(v0, v1);
                                pk[c8][h] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                        }
                    }
                }
                release();
                if (row_ok) {
                    uint16_t* dst = static_cast<uint16_t*>(a.D) + static_cast<size_t>(row) * a.ldd + n0;
#pragma unroll
                    for (int c8 = 0; c8 < 8; ++c8) {
                        if (c8 * 32 < ncols_all) {
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                reinterpret_cast<uint4*>(dst + c8 * 32)[q] =
                                    make_uint4(pk[c8][4 * q], pk[c8][4 * q + 1], pk[c8][4 * q + 2], pk[c8][4 * q + 3]);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < 2 * FN; c += 32) {
                    if (c >= ncols_all) break;
                    uint32_t r[32];
                    tmem_ld32(t_lane + c, r);
                    if (row_ok) {
                        const size_t o = static_cast<size_t>(row) * a.ldd + n0 + c;
                        const int ncols = min(32, a.N - (n0 + c));
                        if (a.out_dtype == LSG_DTYPE_F32) {
                            float* dst = static_cast<float*>(a.D) + o;
                            for (int q = 0; q < ncols; ++q) dst[q] = __uint_as_float(r[q]) * alpha;
                        } else {
                            const bool f16 = a.out_dtype == LSG_DTYPE_F16;
                            uint16_t* dst = static_cast<uint16_t*>(a.D) + o;
                            for (int q = 0; q < ncols; ++q) {
                                const float v = __uint_as_float(r[q]) * alpha;
                                dst[q] = f16 ? __half_as_ushort(__float2half_rn(v)) : __bfloat16_as_ushort(__float2bfloat16_rn(v));
                            }
                        }
                    }
                }
                release();
            }
            ++tile_i;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kFTmemCols);
    }
}

// Packed e2m1 matrix [rows, K/2 bytes] -> tensor map with a (128 bytes x 128 rows) box.
int make_map_u8(CUtensorMap* map, const void* base, long long rows, int row_bytes) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(LSG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
    const cuuint32_t box[2] = {FKB, FM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LSG_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d", static_cast<int>(r));
    return LSG_OK;
}

}  // namespace

// The native route needs whole 64-value K blocks (so that scale atoms are whole), 16-byte
// aligned operands and scale buffers, and rows that are a multiple of 16 bytes.
bool nvfp4_mma_usable(const void* A, const void* B, const void* sfa, const void* sfb, int K) {
    static const bool off = [] {
        const char* e = getenv("LSG_NVFP4_NATIVE");
        return e && atoi(e) == 0;
    }();
    if (off || K <= 0 || K % 64 != 0) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                           reinterpret_cast<uintptr_t>(sfa) | reinterpret_cast<uintptr_t>(sfb);
    return (bits & 15) == 0;
}

// Dense (tile_expert == nullptr: M rows, one problem) or grouped (tile map of 128-row tiles).
int nvfp4_mma(const void* A, long long a_rows, const void* B, long long b_rows, const void* sfa, const void* sfb,
              long long sfb_expert_bytes, int K, int N, void* D, int out_dtype, const float* alphas, float alpha_host,
              int M, const int* tile_expert, const int* tile_mstart, int t_max, const int32_t* expert_offsets,
              const int32_t* sf_offsets, cudaStream_t s) {
    CUtensorMap tmA, tmB;
    int rc = make_map_u8(&tmA, A, a_rows, K / 2);
    if (rc != LSG_OK) return rc;
    rc = make_map_u8(&tmB, B, b_rows, K / 2);
    if (rc != LSG_OK) return rc;
    F4Args a = {};
    a.D = D; a.ldd = N; a.out_dtype = out_dtype; a.alphas = alphas; a.alpha_host = alpha_host;
    a.sfa = static_cast<const uint8_t*>(sfa); a.sfb = static_cast<const uint8_t*>(sfb);
    a.sfb_expert_bytes = sfb_expert_bytes;
    a.K = K; a.N = N; a.n_tiles = (N + FN - 1) / FN;
    a.m_tiles = tile_expert ? t_max : (M + FM - 1) / FM;
    a.M = M; a.tile_expert = tile_expert; a.tile_mstart = tile_mstart; a.expert_offsets = expert_offsets;
    a.sf_offsets = sf_offsets;
    a.status = device_status_word();
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(nvfp4_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmem));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const long long items = static_cast<long long>(a.m_tiles) * ((a.n_tiles + 1) / 2);
    int grid = sm_count();
    if (grid > items) grid = static_cast<int>(items);
    if (grid < 1) grid = 1;
    LSG_CUDA_TRY(launch_kernel(nvfp4_mma_kernel, dim3(grid), dim3(kFThreads), kFSmem, s, true, tmA, tmB, a));
    return LSG_OK;
}

}  // namespace lsg
