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
//     bank-conflict-free shared-memory image with per-group sums;
//   * consumer warps take `L` lanes per weight row (4..32, by row length),
//     each lane decoding whole super-blocks (mmvq_decode.cuh) and dp4a-ing
//     them against the activations, and reduce with a halving butterfly that
//     folds several (row, batch-row) results per shuffle;
//   * the weight stream starts before griddepcontrol.wait, so under
//     programmatic dependent launch it overlaps the activation quantizer.
//
// The reduction order is fixed by the shape, so results are bit-reproducible
// run to run.  Every mbarrier wait is time-limited (common.cuh).
#pragma once

#include "common.cuh"
#include "formats.cuh"
#include "mmvq_decode.cuh"

namespace lsg {

constexpr int kMmvqMaxStages = 8;
constexpr int kMmvqMaxExtra = 5;

struct MmvqArgs {
    const uint8_t* W;         // packed weight, 16-byte aligned
    const uint8_t* xq;        // Q8_1 blocks [M][K/32][36] (used when A is null)
    const __nv_bfloat16* A;   // bf16 activations [M][K]: quantized inside the kernel when set
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
    int debug_skip;           // bench builds (LSG_DEBUG_KNOBS) only: 1 = consumers skip the math
    int cons_warps;           // consumer warps per CTA (block = 32 * (cons_warps + 1))
    long long wait_limit;     // limit of every device-side wait, SM cycles (lsg_set_wait_limit_cycles)
    int drop_slab;            // failure-path test hook: CTA 0's producer never loads this slab (-1: none)
    // How the launch is ordered against the kernel in front of it in the stream (programmatic
    // dependent launch).  0: the kernel after this one may be scheduled at once, the activations
    // are read after the kernel in front has completed.  1 (first launch of a batch whose later
    // launches are of kind 2): the same wait, but the kernel after this one is released only
    // after the wait, so that nothing behind this launch runs before the work in front of the
    // batch has completed.  2 (a launch of a batch that reads and writes nothing an earlier
    // launch of the batch writes or reads): no wait before the activations are read - CTAs
    // start on the SMs the previous launch has left while its last CTAs still stream - and
    // the wait is made before the CTA exits, so that launches still complete in stream order.
    int dep_mode;
#ifdef LSG_MMVQ_TRACE
    unsigned long long* trace;  // [grid][16] nanosecond timestamps of the phases of each CTA
#endif
    // Division-free index arithmetic (set by finish_args): CTA b owns rows
    // [b*rows_q + min(b, rows_r), ...) and quotients by the two small divisors below
    // are taken with a multiply-high.
    int rows_q, rows_r;       // N / grid, N % grid
    int gps;                  // row groups per slab
    uint32_t gps_magic;       // ceil(2^32 / gps), 0 when gps == 1
    uint32_t stages_magic;    // ceil(2^32 / stages), 0 when stages == 1
    // Joined launch: up to five further weight matrices with the same type, K and batch rows
    // (the q, k, v or the gate, up projections of one input; with activations of their own,
    // Ax[j], any projections of that shape that do not depend on each other).  Matrix j owns
    // the CTAs from cta0x[j] up to the next matrix's first CTA; its output is [M][Nx[j]].
    // For joined launches rows_q / rows_r describe matrix 0 over its cta0x[0] CTAs.
    int n_extra;
    const uint8_t* Wx[kMmvqMaxExtra];
    const __nv_bfloat16* Ax[kMmvqMaxExtra];   // bf16 activations of matrix j (set when A is)
    const uint8_t* xqx[kMmvqMaxExtra];        // Q8_1 blocks of matrix j (set when A is null)
    void* Cx[kMmvqMaxExtra];
    int Nx[kMmvqMaxExtra];
    int cta0x[kMmvqMaxExtra];
    int rows_qx[kMmvqMaxExtra], rows_rx[kMmvqMaxExtra];
};

// n / d for 0 <= n < 65536 and 1 <= d < 65536 with magic = ceil(2^32 / d) (0 for d == 1):
// exact because n * (magic * d - 2^32) < n * d < 2^32.
inline uint32_t div_magic(int d) { return d <= 1 ? 0u : static_cast<uint32_t>((0x100000000ull + d - 1) / d); }
#if defined(__CUDACC__)
__device__ __forceinline__ int fast_div(int n, uint32_t magic) {
    return magic == 0u ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), magic));
}
#endif

// Fills the derived fields once grid, slab_rows and stages are known (rpp = rows per warp pass).
inline void finish_args(MmvqArgs& a, int grid, int rpp) {
    if (a.n_extra == 0) {
        a.rows_q = a.N / grid;
        a.rows_r = a.N % grid;
    }
    a.gps = (a.slab_rows + rpp - 1) / rpp;
    a.gps_magic = div_magic(a.gps);
    a.stages_magic = div_magic(a.stages);
}

// Launch geometry knobs (see lsg_mmvq_set_tuning in lsg.h).
struct MmvqTune {
    int warps;      // consumer warps per CTA, 1..15
    int ctas;       // CTAs of one launch per SM
    int stage_kb;   // target bytes per pipeline stage, in KiB
    int share;      // CTAs (of this and neighbouring launches) sharing an SM's shared memory
    int skip_math;  // measurement aid: stream the weights but skip the arithmetic
};

MmvqTune mmvq_tuning();  // current process-wide geometry, clamped to valid ranges (mmvq.cu)

// Per-type entry points, one translation unit each (mmvq_inst.cu).
#define LSG_CAT2(a, b) a##b
#define LSG_CAT(a, b) LSG_CAT2(a, b)
#define MMVQ_FN(name) LSG_CAT(LSG_CAT(mmvq_, name), LSG_CAT(_t, LSG_MMVQ_TYPE))
#define LSG_DECLARE_MMVQ(id)                                         \
    int mmvq_launch_t##id(MmvqArgs a, const MmvqTune& tn, cudaStream_t stream, bool pdl); \
    int mmvq_max_rows_t##id(int K);
LSG_DECLARE_MMVQ(0) LSG_DECLARE_MMVQ(1) LSG_DECLARE_MMVQ(2) LSG_DECLARE_MMVQ(3)
LSG_DECLARE_MMVQ(4) LSG_DECLARE_MMVQ(5) LSG_DECLARE_MMVQ(6) LSG_DECLARE_MMVQ(7)

#if defined(__CUDACC__)

// Bytes of one batch row's activation image.
template <int T> __host__ __device__ constexpr int x_row_bytes(int K) {
    return (K + (K / 32) * 4 + Mmvq<T>::NS * (K / Mmvq<T>::UV) * 4 + 15) & ~15;
}

// ---------------------------------------------------------------------------
// Activation image: Q8_1 blocks from global memory -> planar layout described
// in mmvq_decode.cuh.  One thread per Q8_1 block.
// ---------------------------------------------------------------------------
template <int T>
__device__ __forceinline__ void build_x_image(uint8_t* img, const uint8_t* __restrict__ xq,
                                              int M, int K, int tid, int nthreads) {
    using D = Mmvq<T>;
    constexpr int UVB = D::UV / 32;  // Q8_1 blocks per unit
    const int nb = K / 32;
    const int U = K / D::UV;
    const int rowb = x_row_bytes<T>(K);
    for (int idx = tid; idx < M * nb; idx += nthreads) {
        const int m = idx / nb, b = idx - m * nb;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(xq + static_cast<size_t>(idx) * kQ8_1Bytes);
        const float d = fp16_bits_to_float(__ldg(src));
        uint4 q[2];
        q[0] = make_uint4(__ldg(src + 1), __ldg(src + 2), __ldg(src + 3), __ldg(src + 4));
        q[1] = make_uint4(__ldg(src + 5), __ldg(src + 6), __ldg(src + 7), __ldg(src + 8));
        int sum[2];
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            int s = __dp4a(static_cast<int>(q[hf].x), 0x01010101, 0);
            s = __dp4a(static_cast<int>(q[hf].y), 0x01010101, s);
            s = __dp4a(static_cast<int>(q[hf].z), 0x01010101, s);
            s = __dp4a(static_cast<int>(q[hf].w), 0x01010101, s);
            sum[hf] = s;
        }
        uint8_t* row = img + static_cast<size_t>(m) * rowb;
        uint4* planes = reinterpret_cast<uint4*>(row);
        uint32_t* dvec = reinterpret_cast<uint32_t*>(row + K);
        uint32_t* svec = dvec + nb;
        const int u = b / UVB, jb = b % UVB;
        planes[(2 * jb) * U + u] = q[0];
        planes[(2 * jb + 1) * U + u] = q[1];
        if (UVB >= 4) dvec[((jb >> 2) * U + u) * 4 + (jb & 3)] = __float_as_uint(d);
        else dvec[u] = __float_as_uint(d);
        if (D::SUM == kSumF32Per32) {
            const uint32_t v = __float_as_uint(d * static_cast<float>(sum[0] + sum[1]));
            if (UVB >= 4) svec[((jb >> 2) * U + u) * 4 + (jb & 3)] = v;
            else svec[u] = v;
        } else if (D::SUM == kSumF32Per16 || D::SUM == kSumI32Per16) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int e = 2 * jb + hf;  // 16-value group of the unit
                const uint32_t v = (D::SUM == kSumI32Per16)
                                       ? static_cast<uint32_t>(sum[hf])
                                       : __float_as_uint(d * static_cast<float>(sum[hf]));
                svec[((e >> 2) * U + u) * 4 + (e & 3)] = v;
            }
        }
    }
}

// Same image straight from bf16 activations: the Q8_1 quantization of
// quantize_q8_1_kernel (d = amax/127, q = rn(x/d), d then rounded to fp16) done per CTA,
// without the round trip through global memory and without a launch of its own.  Four
// lanes share a 32-value block, eight values each.  Values are identical to the
// quantizer kernel's: max and the per-element division do not depend on the lane layout,
// and the block sum of the original values (the only order-dependent field of a Q8_1
// block) is not used by the mat-vec.
template <int T>
__device__ __forceinline__ void build_x_image_bf16(uint8_t* img, const __nv_bfloat16* __restrict__ A,
                                                   int M, int K, int tid, int nthreads) {
    using D = Mmvq<T>;
    constexpr int UVB = D::UV / 32;
    const int nb = K / 32;
    const int U = K / D::UV;
    const int rowb = x_row_bytes<T>(K);
    // Two lanes per 32-value block, sixteen values (two 16-byte loads) per lane: a 4096-wide
    // row is one trip of 256 tasks for the consumer threads, and the only index arithmetic is
    // shifts and divisions by compile-time constants.
    const int tasks = nb * 2;
    for (int m = 0; m < M; ++m) {
        const uint4* src = reinterpret_cast<const uint4*>(A + static_cast<size_t>(m) * K);
        uint8_t* row = img + static_cast<size_t>(m) * rowb;
        uint32_t* dvec = reinterpret_cast<uint32_t*>(row + K);
        uint32_t* svec = dvec + nb;
        for (int t0 = 0; t0 < tasks; t0 += nthreads) {
            const int idx = t0 + tid;
            const bool live = idx < tasks;
            const int task = live ? idx : 0;
            const uint4 r0 = __ldg(src + 2 * task), r1 = __ldg(src + 2 * task + 1);
            const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
            float x[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x[2 * i] = __uint_as_float(w[i] << 16);
                x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            const float d = amax / 127.0f;
            // q = rn(fl(x / d)) as the reference computes it, without sixteen IEEE divisions
            // (q8_round8: the quotient from the reciprocal and one exact remainder step)
            const float rcp = (amax == 0.0f) ? 0.0f : 1.0f / d;
            uint4 packed;
            q8_round8(x, d, rcp, packed.x, packed.y);
            q8_round8(x + 8, d, rcp, packed.z, packed.w);
            // sum of the sixteen int8 codes: four byte-wise dot products with ones
            const int sum16 = __dp4a(static_cast<int>(packed.x), 0x01010101,
                              __dp4a(static_cast<int>(packed.y), 0x01010101,
                              __dp4a(static_cast<int>(packed.z), 0x01010101,
                              __dp4a(static_cast<int>(packed.w), 0x01010101, 0))));
            const int sum32 = sum16 + __shfl_xor_sync(0xffffffffu, sum16, 1);
            if (!live) continue;
            const float dh = __half2float(__float2half(d));  // the mat-vec sees the fp16-rounded scale
            const int half = task & 1;
            const int b = task >> 1;
            const int u = b / UVB, jb = b % UVB;
            *reinterpret_cast<uint4*>(row + (static_cast<size_t>(2 * jb + half) * U + u) * 16) = packed;
            if (half == 0) {
                if (UVB >= 4) dvec[((jb >> 2) * U + u) * 4 + (jb & 3)] = __float_as_uint(dh);
                else dvec[u] = __float_as_uint(dh);
                if (D::SUM == kSumF32Per32) {
                    const uint32_t v = __float_as_uint(dh * static_cast<float>(sum32));
                    if (UVB >= 4) svec[((jb >> 2) * U + u) * 4 + (jb & 3)] = v;
                    else svec[u] = v;
                }
            }
            if (D::SUM == kSumF32Per16 || D::SUM == kSumI32Per16) {
                const int e = 2 * jb + half;
                const uint32_t v = (D::SUM == kSumI32Per16) ? static_cast<uint32_t>(sum16)
                                                            : __float_as_uint(dh * static_cast<float>(sum16));
                svec[((e >> 2) * U + u) * 4 + (e & 3)] = v;
            }
        }
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
// One row group x MT batch rows: dot every unit of the RW*SUBS rows of the group with
// the activation image, reduce over the L lanes of each row, store.
//   raddr   shared addresses of this lane group's RW rows (clamped to the slab)
//   xv      activation image view; xv.base / xv.mlast already set for this batch tile
//   rl0     first row of this lane group inside the slab; rows >= nrows are not stored
//   col0    output column of slab row 0;  mrow0 / mvalid  first output row and how many
// ---------------------------------------------------------------------------
template <int T, int MT, int RW, int L>
__device__ __forceinline__ void group_dot_store(const uint32_t (&raddr)[RW], const XView& xv, int lane,
                                                int rl0, int nrows, long long col0, int mrow0,
                                                int mvalid, void* C, int ldc, int out_f32,
                                                bool skip_math) {
    using D = Mmvq<T>;
    const int kl = lane % L;
    float acc[RW * MT];
#pragma unroll
    for (int v = 0; v < RW * MT; ++v) acc[v] = 0.0f;
    if (!skip_math)
        for (int u = kl; u < xv.U; u += L) D::template unit_dot<RW, MT>(raddr, u, xv, acc);

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
            const int rl = rl0 + r;
            if (rl < nrows && m < mvalid)
                store_out(C, out_f32, static_cast<size_t>(mrow0 + m) * ldc + (col0 + rl), v[0]);
        }
    }
}

// ---------------------------------------------------------------------------
// The kernel
//   T  : lsg_gguf_type
//   MT : batch rows per register pass (1, 2, 4, 8)
//   RW : weight rows per lane group per pass (1 or 2)
//   L  : lanes per weight row (4, 8, 16, 32)
// blockDim.x = 32 * (consumer warps + 1); the last warp is the producer.
// ---------------------------------------------------------------------------
// Development aid (-DLSG_MMVQ_TRACE): nanosecond timestamps of each CTA's phases, read back
// by a probe.  Compiled out of the library.
#ifdef LSG_MMVQ_TRACE
#define LSG_TRACE(slot) do { if (a.trace) a.trace[static_cast<size_t>(blockIdx.x) * 16 + (slot)] = global_timer_ns(); } while (0)
#define LSG_TRACE_MAX(slot) do { if (a.trace) atomicMax(&a.trace[static_cast<size_t>(blockIdx.x) * 16 + (slot)], global_timer_ns()); } while (0)
#define LSG_TRACE_MIN(slot) do { if (a.trace) atomicMin(&a.trace[static_cast<size_t>(blockIdx.x) * 16 + (slot)], global_timer_ns()); } while (0)
#define LSG_TRACE_ADD(slot, v) do { if (a.trace) atomicAdd(&a.trace[static_cast<size_t>(blockIdx.x) * 16 + (slot)], static_cast<unsigned long long>(v)); } while (0)
#define LSG_TRACE_CLK(var) const long long var = sm_clock()
#else
#define LSG_TRACE_ADD(slot, v) do { } while (0)
#define LSG_TRACE_CLK(var) do { } while (0)
#define LSG_TRACE(slot) do { } while (0)
#define LSG_TRACE_MAX(slot) do { } while (0)
#define LSG_TRACE_MIN(slot) do { } while (0)
#endif

#ifdef LSG_DEBUG_KNOBS
#define LSG_SKIP_MATH(a) ((a).debug_skip != 0)
#else
#define LSG_SKIP_MATH(a) false
#endif

template <int T, int MT, int RW, int L>
__global__ void __launch_bounds__(512, 1) mmvq_kernel(const MmvqArgs a) {
    using D = Mmvq<T>;
    constexpr int SUBS = 32 / L;    // lane groups per warp
    constexpr int RPP = SUBS * RW;  // rows per warp pass

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* x_img = smem;
    uint8_t* ring = smem + a.x_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(a.stages) * a.stage_bytes);
    uint64_t* empty = full + kMmvqMaxStages;
    int* next_group = reinterpret_cast<int*>(empty + kMmvqMaxStages);
    volatile int* slab_in_stage = next_group + 1;  // which slab each stage was last loaded with
    volatile int* released = slab_in_stage + kMmvqMaxStages;  // dep_mode 1: the consumers have passed their wait

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int n_cons_warps = (blockDim.x >> 5) - 1;
    const bool is_producer = (warp == n_cons_warps);

    // The matrix this CTA works on (joined launches) and its contiguous row range there.
    int bx = static_cast<int>(blockIdx.x);
    const uint8_t* Wm = a.W;
    const __nv_bfloat16* Am = a.A;
    const uint8_t* xqm = a.xq;
    void* Cm = a.C;
    int Nm = a.N, ldcm = a.ldc, rows_q = a.rows_q, rows_r = a.rows_r;
    if (a.n_extra > 0) {
        const int b = static_cast<int>(blockIdx.x);
        int jm = -1;
#pragma unroll
        for (int j = 0; j < kMmvqMaxExtra; ++j)
            if (j < a.n_extra && b >= a.cta0x[j]) jm = j;
        if (jm >= 0) {
            Wm = a.Wx[jm];
            Am = a.Ax[jm];
            xqm = a.xqx[jm];
            Cm = a.Cx[jm];
            Nm = ldcm = a.Nx[jm];
            rows_q = a.rows_qx[jm];
            rows_r = a.rows_rx[jm];
            bx = b - a.cta0x[jm];
        }
    }
    const int row_begin = bx * rows_q + min(bx, rows_r);
    const int row_end = row_begin + rows_q + (bx < rows_r ? 1 : 0);
    const int groups_per_slab = a.gps;

    const int n_slabs = (row_end - row_begin + a.slab_rows - 1) / a.slab_rows;

    // One lane per stage initialises its two barriers (a loop in a single thread would issue
    // them one after the other at the very start of every launch).
    if (tid == 0) LSG_TRACE(0);
    if (tid < kMmvqMaxStages) {
        if (tid < a.stages) {
            mbar_init(&full[tid], 1);
            mbar_init(&empty[tid], groups_per_slab);  // one arrival per row group
        }
        slab_in_stage[tid] = -1;
        if (tid == 0) *next_group = 0;
        mbar_fence_init();
    }
    if (tid == 0) *released = 0;
    __syncthreads();
    if (a.dep_mode != 1) pdl_launch_dependents();

    if (is_producer) {
        // ------------------------------------------------------------------
        // Producer: stream this CTA's rows, slab by slab, into the ring.
        // Weights are constants of the model, so this does not wait for the
        // previous kernel in the stream.
        // ------------------------------------------------------------------
        // The whole warp walks the loop with the same values in every lane and one elected
        // lane issues the copy: bulk copies and barrier operations take their operands from
        // warp-uniform registers, and inside a one-lane branch each of them costs several
        // times what it costs in converged code.
        const uint64_t policy = l2_policy_evict_first();
        const uintptr_t w_base = reinterpret_cast<uintptr_t>(Wm);
        const uintptr_t w_end_al = (w_base + static_cast<uintptr_t>(Nm) * a.row_bytes) & ~uintptr_t(15);
        int s = 0;
        uint32_t lap = 0;  // ring position of slab i: stage s, lap = i / stages
        bool trigger_due = a.dep_mode == 1;   // this warp releases the next kernel too, once the consumers have
        for (int i = 0; i < n_slabs; ++i, s = (s + 1 == a.stages) ? 0 : s + 1, lap += (s == 0)) {
            if (trigger_due && *released) {
                pdl_launch_dependents();
                trigger_due = false;
            }
            if (lap > 0 &&
                !__all_sync(0xffffffffu, mbar_wait_bounded(&empty[s], (lap - 1) & 1, a.status, kDevWaitEmpty, 2000u, a.wait_limit)))
                break;
            // Failure-path test hook: this slab is never loaded nor published, so its
            // consumers run into their wait limit, report and return.
            if (i == a.drop_slab && blockIdx.x == 0) break;
            const int r0 = row_begin + i * a.slab_rows;
            const int r1 = min(r0 + a.slab_rows, row_end);
            const uintptr_t src_b = w_base + static_cast<uintptr_t>(r0) * a.row_bytes;
            const uintptr_t src_e = w_base + static_cast<uintptr_t>(r1) * a.row_bytes;
            const uintptr_t cp_b = src_b & ~uintptr_t(15);
            uintptr_t cp_e = (src_e + 15) & ~uintptr_t(15);
            uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
            const bool ragged = cp_e > w_end_al;
            if (ragged) cp_e = w_end_al > cp_b ? w_end_al : cp_b;
            const uint32_t bytes = static_cast<uint32_t>(cp_e - cp_b);
            if (elect_one_lane()) {
                if (ragged) {
                    // Last rows of the matrix end off a 16-byte boundary: the bulk copy stops at
                    // the last whole 16 bytes and the remainder is moved with byte loads.
                    for (uintptr_t p = cp_e; p < src_e; ++p)
                        dst[p - cp_b] = *reinterpret_cast<const uint8_t*>(p);
                }
                slab_in_stage[s] = i;  // published before the arrive below (release)
                if (i == 0) LSG_TRACE(1);
                if (i == n_slabs - 1) LSG_TRACE(2);
                if (bytes > 0) {
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_g2s_hint(dst, reinterpret_cast<const void*>(cp_b), bytes, &full[s], policy);
                } else {
                    mbar_arrive(&full[s]);
                }
            }
            __syncwarp();
        }
        if (trigger_due) {
            // all slabs issued before the consumers were released: wait for them (bounded), then release
            const long long t0 = sm_clock();
            while (!*released && sm_clock() - t0 <= a.wait_limit) __nanosleep(64);
            pdl_launch_dependents();
        }
        return;
    }

    // ----------------------------------------------------------------------
    // Consumers
    // ----------------------------------------------------------------------
    const int n_cons = n_cons_warps * 32;
    if (a.dep_mode != 2) pdl_wait_prior();  // activations (and the output buffer) belong to the stream order
    if (a.dep_mode == 1) {
        pdl_launch_dependents();
        if (tid == 0) *released = 1;
    }
    if (tid == 0) LSG_TRACE(3);
    if (a.A) build_x_image_bf16<T>(x_img, Am, a.M, a.K, tid, n_cons);
    else build_x_image<T>(x_img, xqm, a.M, a.K, tid, n_cons);
    asm volatile("bar.sync 1, %0;" ::"r"(n_cons) : "memory");
    if (tid == 0) LSG_TRACE(4);

    const int sub = lane / L;
    XView xv;
    xv.rowb = x_row_bytes<T>(a.K);
    xv.d_off = a.K;
    xv.s_off = a.K + (a.K / 32) * 4;
    xv.U = a.K / D::UV;
    const uint32_t x_base = smem_u32(x_img);

    // Row groups (RPP rows each) are claimed from a CTA-wide queue in row order.  A
    // warp therefore waits on a stage only when it holds work in it, a short slab
    // never leaves warps polling, and the tail of the range balances itself.  Which
    // warp computes a group does not change its result.
    const uintptr_t w_base = reinterpret_cast<uintptr_t>(Wm);
    const int total_groups = n_slabs * groups_per_slab;
    for (;;) {
        LSG_TRACE_CLK(tc0);
        int gidx = 0;
        if (lane == 0) gidx = atomicAdd(next_group, 1);
        gidx = __shfl_sync(0xffffffffu, gidx, 0);
        if (gidx >= total_groups) break;
        if (gidx == 0 && lane == 0) LSG_TRACE(5);
        const int i = fast_div(gidx, a.gps_magic);
        const int g = (gidx - i * groups_per_slab) * RPP;
        const int lap = fast_div(i, a.stages_magic);
        const int s = i - lap * a.stages;
        const int r0 = row_begin + i * a.slab_rows;
        const int nrows = min(a.slab_rows, row_end - r0);
        // Every claim waits for its slab, including the groups past the end of a short
        // last slab: their arrival below must not fall into the stage's previous phase.
        // A parity wait alone cannot tell lap n of a stage from lap n-2, and a warp may
        // claim a group whose slab is more than a ring ahead of the slowest warp; so
        // first wait until the producer has started loading exactly this slab.
        if (slab_in_stage[s] != i) {
            const long long t0 = sm_clock();
            while (slab_in_stage[s] != i) {
                __nanosleep(64);
                if (sm_clock() - t0 > a.wait_limit) {
                    if (a.status) atomicCAS(a.status, 0u, static_cast<unsigned int>(kDevWaitFull));
                    return;
                }
            }
        }
        if (!mbar_wait_bounded(&full[s], lap & 1, a.status, kDevWaitFull, 2000u, a.wait_limit)) return;
        if (gidx == 0 && lane == 0) LSG_TRACE(6);
        LSG_TRACE_CLK(tc1);
        if (gidx == (n_slabs - 1) * groups_per_slab && lane == 0) LSG_TRACE(8);
        if (g < nrows) {
            const uintptr_t src_b = w_base + static_cast<uintptr_t>(r0) * a.row_bytes;
            const uint32_t slab = smem_u32(ring + static_cast<size_t>(s) * a.stage_bytes) +
                                  static_cast<uint32_t>(src_b & 15);
            uint32_t raddr[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r)
                raddr[r] = slab + static_cast<uint32_t>(min(g + sub * RW + r, nrows - 1)) * a.row_bytes;

            for (int m0 = 0; m0 < a.M; m0 += MT) {
                xv.base = x_base + m0 * xv.rowb;
                xv.mlast = a.M - 1 - m0;
                group_dot_store<T, MT, RW, L>(raddr, xv, lane, g + sub * RW, nrows, r0, m0,
                                              a.M - m0, Cm, ldcm, a.out_f32, LSG_SKIP_MATH(a));
            }
        }
        // Every stage collects one arrival per group, real or past the end.
        __syncwarp();
        if (elect_one_lane()) mbar_arrive(&empty[s]);
#ifdef LSG_MMVQ_TRACE
        if (lane == 0) {
            LSG_TRACE_CLK(tc2);
            LSG_TRACE_ADD(9, tc1 - tc0);
            LSG_TRACE_ADD(10, tc2 - tc1);
            LSG_TRACE_ADD(11, 1);
        }
#endif
    }
    if (lane == 0) LSG_TRACE_MAX(7);
    if (a.dep_mode == 2) pdl_wait_prior();
}

#endif  // __CUDACC__

}  // namespace lsg
