// GGUF mmvq for sm_100a: C[M,N] = Q8_1(A)[M,K] . decode(W)[N,K]^T, M small.
//
// Replaces gguf_mmvq_kernel / accumulate / reduce_store of the reference
// (csrc/sm120/gemm/gguf/gguf_mmvq.cu:69-112, gguf_mmvq_impl.cuh:43-100), which
// assigns one 128-thread CTA per output channel and walks the row with strided
// 4-byte loads.  This kernel is built for a bandwidth-bound part instead:
//
//   * one persistent CTA per SM owns a contiguous range of weight rows;
//   * a producer warp streams that range through a ring of shared-memory
//     stages with 1-D bulk (TMA) copies of whole row slabs - rows are
//     contiguous in memory, so a slab is one perfectly coalesced transfer
//     whatever the block size (17..210 bytes) - tracked by mbarriers;
//   * the Q8_1 activations are re-laid once per CTA into a planar,
//     bank-conflict-free shared-memory image with per-group sums, and for a
//     single row with short K they stay in registers for the whole kernel;
//   * consumer warps take `L` lanes per weight row (a whole warp for long
//     rows), decode chunks with packed-nibble tricks, dp4a against the
//     activations, and reduce with a halving butterfly that folds several
//     (row, batch-row) results per shuffle;
//   * the weight stream starts before griddepcontrol.wait, so under
//     programmatic dependent launch it overlaps the activation quantizer.
//
// The reduction order is fixed by the shape, so results are bit-reproducible
// run to run.  Every mbarrier wait is time-limited (common.cuh).
#pragma once

#include "common.cuh"
#include "formats.cuh"

namespace lsg {

constexpr int kMmvqMaxStages = 8;

struct MmvqArgs {
    const uint8_t* W;         // packed weight, 16-byte aligned
    const uint8_t* xq;        // Q8_1 blocks [M][K/32][36]
    void* C;                  // [M][ldc] bf16 or f32
    unsigned int* status;     // device status word
    int M, N, K;
    int ldc;                  // output row stride in elements
    int out_f32;              // 0: bf16, 1: f32
    int row_bytes;            // (K / VALS) * BYTES
    int slab_rows;            // rows per pipeline stage
    int stages;               // ring depth
    int stage_bytes;          // bytes reserved per stage (multiple of 128)
    int x_bytes;              // bytes of the activation image (multiple of 128)
};

// Per-type entry points, one translation unit each (mmvq_inst.cu).
#define LSG_CAT2(a, b) a##b
#define LSG_CAT(a, b) LSG_CAT2(a, b)
#define MMVQ_FN(name) LSG_CAT(LSG_CAT(mmvq_, name), LSG_CAT(_t, LSG_MMVQ_TYPE))
#define LSG_DECLARE_MMVQ(id)                                         \
    int mmvq_launch_t##id(MmvqArgs a, cudaStream_t stream, bool pdl); \
    int mmvq_max_rows_t##id(int K);
LSG_DECLARE_MMVQ(0) LSG_DECLARE_MMVQ(1) LSG_DECLARE_MMVQ(2) LSG_DECLARE_MMVQ(3)
LSG_DECLARE_MMVQ(4) LSG_DECLARE_MMVQ(5) LSG_DECLARE_MMVQ(6) LSG_DECLARE_MMVQ(7)

#if defined(__CUDACC__)

// Sizes of the activation image in shared memory, per activation row.
template <ChunkShape S> __host__ __device__ constexpr int x_row_bytes(int K) {
    // int8 values + fp32 d per 32 + fp32 d*sum per 32 (kPair/kBlock) or per 16 (kQuad)
    // rounded up so that every row image starts on a 16-byte boundary
    return (K + (K / 32) * 4 + (S == kQuad ? (K / 16) * 4 : (K / 32) * 4) + 15) & ~15;
}

// ---------------------------------------------------------------------------
// Activation image: build (once per CTA) and read (per chunk)
// ---------------------------------------------------------------------------
// Layout of one row: [planes of 16-byte units][d per 32-block][s].
//   kPair : 4 planes; unit (plane j, chunk c) = values 64c+16j ..  ; s per 32-block
//   kQuad : 4 planes; unit (plane q, chunk c=4sb+2ip+h) = values 256sb+128ip+32q+16h .. ;
//           s per (chunk, quad)
//   kBlock: 2 planes; unit (plane j, chunk c) = values 32c+16j .. ; s per 32-block
template <ChunkShape S>
__device__ __forceinline__ void build_x_image(uint8_t* img, const uint8_t* __restrict__ xq,
                                              int M, int K, int tid, int nthreads) {
    const int nb = K / 32;
    const int C = (S == kBlock) ? nb : K / 64;
    const int rowb = x_row_bytes<S>(K);
    for (int idx = tid; idx < M * nb; idx += nthreads) {
        const int m = idx / nb, b = idx - m * nb;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(xq + static_cast<size_t>(idx) * kQ8_1Bytes);
        const uint32_t ds = __ldg(src);
        const float d = fp16_bits_to_float(ds);
        uint4 u[2];
        u[0] = make_uint4(__ldg(src + 1), __ldg(src + 2), __ldg(src + 3), __ldg(src + 4));
        u[1] = make_uint4(__ldg(src + 5), __ldg(src + 6), __ldg(src + 7), __ldg(src + 8));
        int sum[2];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            int s = __dp4a(static_cast<int>(u[hf].x), 0x01010101, 0);
            s = __dp4a(static_cast<int>(u[hf].y), 0x01010101, s);
            s = __dp4a(static_cast<int>(u[hf].z), 0x01010101, s);
            s = __dp4a(static_cast<int>(u[hf].w), 0x01010101, s);
            sum[hf] = s;
        }
        uint8_t* row = img + static_cast<size_t>(m) * rowb;
        uint4* planes = reinterpret_cast<uint4*>(row);
        float* dvec = reinterpret_cast<float*>(row + K);
        float* svec = dvec + nb;
        dvec[b] = d;
        if (S == kPair) {
            const int c = b >> 1, j = (b & 1) * 2;
            planes[j * C + c] = u[0];
            planes[(j + 1) * C + c] = u[1];
            svec[b] = d * static_cast<float>(sum[0] + sum[1]);
        } else if (S == kBlock) {
            planes[b] = u[0];
            planes[C + b] = u[1];
            svec[b] = d * static_cast<float>(sum[0] + sum[1]);
        } else {
            // block b = 8sb + 4ip + q holds units h = 0, 1 of quad q
            const int sb = b >> 3, ip = (b >> 2) & 1, q = b & 3;
            const int c0 = 4 * sb + 2 * ip;
            planes[q * C + c0] = u[0];
            planes[q * C + c0 + 1] = u[1];
            svec[c0 * 4 + q] = d * static_cast<float>(sum[0]);
            svec[(c0 + 1) * 4 + q] = d * static_cast<float>(sum[1]);
        }
    }
}

template <ChunkShape S>
__device__ __forceinline__ void load_x_chunk(uint32_t row /*shared addr of the row image*/,
                                             int K, int c, XChunk<S>& x) {
    const int nb = K / 32;
    const int C = (S == kBlock) ? nb : K / 64;
    const uint32_t dvec = row + K;
    const uint32_t svec = dvec + nb * 4;
    if (S == kPair) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 v = lds128(row + (j * C + c) * 16);
            x.qs[4 * j] = v.x; x.qs[4 * j + 1] = v.y; x.qs[4 * j + 2] = v.z; x.qs[4 * j + 3] = v.w;
        }
        const uint2 d = lds64(dvec + c * 8), s = lds64(svec + c * 8);
        x.d[0] = __uint_as_float(d.x); x.d[1] = __uint_as_float(d.y);
        x.s[0] = __uint_as_float(s.x); x.s[1] = __uint_as_float(s.y);
    } else if (S == kQuad) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 v = lds128(row + (q * C + c) * 16);
            x.qs[4 * q] = v.x; x.qs[4 * q + 1] = v.y; x.qs[4 * q + 2] = v.z; x.qs[4 * q + 3] = v.w;
        }
        const uint4 d = lds128(dvec + (c >> 1) * 16), s = lds128(svec + c * 16);
        x.d[0] = __uint_as_float(d.x); x.d[1] = __uint_as_float(d.y);
        x.d[2] = __uint_as_float(d.z); x.d[3] = __uint_as_float(d.w);
        x.s[0] = __uint_as_float(s.x); x.s[1] = __uint_as_float(s.y);
        x.s[2] = __uint_as_float(s.z); x.s[3] = __uint_as_float(s.w);
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const uint4 v = lds128(row + (j * C + c) * 16);
            x.qs[4 * j] = v.x; x.qs[4 * j + 1] = v.y; x.qs[4 * j + 2] = v.z; x.qs[4 * j + 3] = v.w;
        }
        x.d[0] = __uint_as_float(lds32(dvec + c * 4));
        x.s[0] = __uint_as_float(lds32(svec + c * 4));
    }
}

// ---------------------------------------------------------------------------
// Halving butterfly: NV values per lane, summed over the L lanes of a group.
// Afterwards v[0] of lane l holds the group total of value (l % L) / (L / NV).
// NV and L are powers of two, NV <= L.
// ---------------------------------------------------------------------------
template <int NV, int L>
__device__ __forceinline__ void reduce_group(float (&v)[NV], int lane) {
    static_assert(NV <= L, "more values than lanes");
    if constexpr (NV > 1) {
        constexpr int stride = L / 2;
        const bool upper = (lane & stride) != 0;
        float h[NV / 2];
#pragma unroll
        for (int i = 0; i < NV / 2; ++i) {
            const float send = upper ? v[i] : v[i + NV / 2];
            const float keep = upper ? v[i + NV / 2] : v[i];
            h[i] = keep + __shfl_xor_sync(0xffffffffu, send, stride);
        }
        reduce_group<NV / 2, L / 2>(h, lane);
        v[0] = h[0];
    } else {
#pragma unroll
        for (int o = L / 2; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    }
}

__device__ __forceinline__ void store_out(void* C, int out_f32, size_t idx, float v) {
    if (out_f32) static_cast<float*>(C)[idx] = v;
    else static_cast<__nv_bfloat16*>(C)[idx] = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------------------
// The kernel
//   T    : lsg_gguf_type
//   MT   : activation rows per register pass (1, 2, 4, 8)
//   RW   : weight rows per lane group per pass (1 or 2)
//   L    : lanes per weight row (32, 8)
//   XREG : chunks of the single activation row kept in registers (0 = none)
// blockDim.x = 32 * (consumer warps + 1); the last warp is the producer.
// ---------------------------------------------------------------------------
template <int T, int MT, int RW, int L, int XREG>
__global__ void __launch_bounds__(512, 1) mmvq_kernel(const MmvqArgs a) {
    using F = Fmt<T>;
    using D = Mmvq<T>;
    constexpr ChunkShape S = F::SHAPE;
    constexpr int CHUNK_VALS = (S == kBlock) ? 32 : 64;
    constexpr int SUBS = 32 / L;        // lane groups per warp
    constexpr int RPP = SUBS * RW;      // rows per warp pass

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* x_img = smem;
    uint8_t* ring = smem + a.x_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(a.stages) * a.stage_bytes);
    uint64_t* empty = full + kMmvqMaxStages;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int n_cons_warps = (blockDim.x >> 5) - 1;
    const bool is_producer = (warp == n_cons_warps);

    // Contiguous row range of this CTA.
    const int row_begin = static_cast<int>((static_cast<long long>(a.N) * blockIdx.x) / gridDim.x);
    const int row_end = static_cast<int>((static_cast<long long>(a.N) * (blockIdx.x + 1)) / gridDim.x);
    const int n_slabs = (row_end - row_begin + a.slab_rows - 1) / a.slab_rows;

    if (tid == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], n_cons_warps);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (is_producer) {
        // ------------------------------------------------------------------
        // Producer: stream this CTA's rows, slab by slab, into the ring.
        // Weights are constants of the model, so this does not wait for the
        // previous kernel in the stream.
        // ------------------------------------------------------------------
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            const uintptr_t w_base = reinterpret_cast<uintptr_t>(a.W);
            const uintptr_t w_end_al = (w_base + static_cast<uintptr_t>(a.N) * a.row_bytes) & ~uintptr_t(15);
            for (int i = 0; i < n_slabs; ++i) {
                const int s = i % a.stages;
                if (i >= a.stages) {
                    const uint32_t parity = ((i / a.stages) - 1) & 1;
                    if (!mbar_wait_bounded(&empty[s], parity, a.status, kDevWaitEmpty)) break;
                }
                const int r0 = row_begin + i * a.slab_rows;
                const int r1 = min(r0 + a.slab_rows, row_end);
                const uintptr_t src_b = w_base + static_cast<uintptr_t>(r0) * a.row_bytes;
                const uintptr_t src_e = w_base + static_cast<uintptr_t>(r1) * a.row_bytes;
                const uintptr_t cp_b = src_b & ~uintptr_t(15);
                uintptr_t cp_e = (src_e + 15) & ~uintptr_t(15);
                uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
                if (cp_e > w_end_al) {
                    // Last rows of the matrix end off a 16-byte boundary: the
                    // bulk copy stops at the last whole 16 bytes and the
                    // remainder is moved with byte loads.
                    cp_e = w_end_al > cp_b ? w_end_al : cp_b;
                    for (uintptr_t p = cp_e; p < src_e; ++p)
                        dst[p - cp_b] = *reinterpret_cast<const uint8_t*>(p);
                }
                const uint32_t bytes = static_cast<uint32_t>(cp_e - cp_b);
                if (bytes > 0) {
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_g2s_hint(dst, reinterpret_cast<const void*>(cp_b), bytes, &full[s], policy);
                } else {
                    mbar_arrive(&full[s]);
                }
            }
        }
        return;
    }

    // ----------------------------------------------------------------------
    // Consumers
    // ----------------------------------------------------------------------
    pdl_wait_prior();  // activations (and the output buffer) belong to the stream order
    const int n_cons = n_cons_warps * 32;
    build_x_image<S>(x_img, a.xq, a.M, a.K, tid, n_cons);
    asm volatile("bar.sync 1, %0;" ::"r"(n_cons) : "memory");

    const int C = a.K / CHUNK_VALS;
    const int sub = lane / L;
    const int kl = lane % L;
    const uint32_t x_base = smem_u32(x_img);
    const int x_rowb = x_row_bytes<S>(a.K);

    XChunk<S> xr[XREG > 0 ? XREG : 1];
    if constexpr (XREG > 0) {
#pragma unroll
        for (int i = 0; i < XREG; ++i) {
            const int c = kl + L * i;
            if (c < C) load_x_chunk<S>(x_base, a.K, c, xr[i]);
        }
    }

    const uintptr_t w_base = reinterpret_cast<uintptr_t>(a.W);
    for (int i = 0; i < n_slabs; ++i) {
        const int s = i % a.stages;
        if (!mbar_wait_bounded(&full[s], (i / a.stages) & 1, a.status, kDevWaitFull)) return;

        const int r0 = row_begin + i * a.slab_rows;
        const int nrows = min(a.slab_rows, row_end - r0);
        const uintptr_t src_b = w_base + static_cast<uintptr_t>(r0) * a.row_bytes;
        const uint32_t slab = smem_u32(ring + static_cast<size_t>(s) * a.stage_bytes) +
                              static_cast<uint32_t>(src_b & 15);

        // Row groups are dealt to warps round-robin across the whole row range of the
        // CTA (not per slab), so that short slabs still keep every warp busy.
        const int groups_per_slab = (a.slab_rows + RPP - 1) / RPP;
        const int first_group = i * groups_per_slab;
        const int my_first = (warp + n_cons_warps - first_group % n_cons_warps) % n_cons_warps;
        for (int g = my_first * RPP; g < nrows; g += n_cons_warps * RPP) {
            int rloc[RW];
            uint32_t raddr[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                rloc[r] = g + sub * RW + r;
                raddr[r] = slab + static_cast<uint32_t>(min(rloc[r], nrows - 1)) * a.row_bytes;
            }
            for (int m0 = 0; m0 < a.M; m0 += MT) {
                float acc[RW * MT];
#pragma unroll
                for (int v = 0; v < RW * MT; ++v) acc[v] = 0.0f;

                if constexpr (XREG > 0) {
#pragma unroll
                    for (int it = 0; it < XREG; ++it) {
                        const int c = kl + L * it;
                        if (c < C) {
#pragma unroll
                            for (int r = 0; r < RW; ++r) {
                                typename D::W w;
                                D::load(raddr[r], c, w);
                                acc[r] += D::dot(w, xr[it]);
                            }
                        }
                    }
                } else {
                    for (int c = kl; c < C; c += L) {
                        typename D::W w[RW];
#pragma unroll
                        for (int r = 0; r < RW; ++r) D::load(raddr[r], c, w[r]);
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            // Rows past M re-read the last row; their results are dropped.
                            const int mm = min(m0 + m, a.M - 1);
                            XChunk<S> x;
                            load_x_chunk<S>(x_base + mm * x_rowb, a.K, c, x);
#pragma unroll
                            for (int r = 0; r < RW; ++r) acc[r * MT + m] += D::dot(w[r], x);
                        }
                    }
                }

                // Reduce over the L lanes of each group, NVB values at a time.
                constexpr int NV = RW * MT;
                constexpr int NVB = NV < L ? NV : L;
#pragma unroll
                for (int b0 = 0; b0 < NV; b0 += NVB) {
                    float v[NVB];
#pragma unroll
                    for (int k = 0; k < NVB; ++k) v[k] = acc[b0 + k];
                    reduce_group<NVB, L>(v, lane);
                    constexpr int LPV = L / NVB;  // lanes holding the same value
                    if ((kl % LPV) == 0) {
                        const int vi = b0 + kl / LPV;
                        const int r = vi / MT, m = vi % MT;
                        const int rl = g + sub * RW + r;
                        if (rl < nrows && m0 + m < a.M) {
                            store_out(a.C, a.out_f32,
                                      static_cast<size_t>(m0 + m) * a.ldc + (r0 + rl), v[0]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
    }
}

#endif  // __CUDACC__

}  // namespace lsg
