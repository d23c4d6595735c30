// Shared host/device helpers for the sm_100a kernels: status plumbing, bounded
// mbarrier waits, 1-D bulk (TMA) copies, programmatic-dependent-launch hooks.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/lsg.h"

namespace lsg {

// ---------------------------------------------------------------------------
// Host: error text + status helpers (defined in capi.cu)
// ---------------------------------------------------------------------------
int fail(int code, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
// Address of the per-device status word kernels report bounded-wait failures to.
unsigned int* device_status_word();
int sm_count();

#define LSG_CUDA_TRY(expr)                                        \
    do {                                                          \
        cudaError_t e__ = (expr);                                 \
        if (e__ != cudaSuccess) return ::lsg::cuda_fail(e__, #expr); \
    } while (0)

// Device status codes written to the status word.
enum : unsigned int {
    kDevOk = 0,
    kDevWaitFull = 1,   // consumer gave up waiting for a bulk copy to land
    kDevWaitEmpty = 2,  // producer gave up waiting for a stage to be released
    kDevWaitMma = 3,    // epilogue gave up waiting for tensor-core completion
    kDevWaitTmem = 4,
    kDevSlabTable = 5,   // grouped mat-vec: a CTA's slab table was too small for its rows
    kDevBarrier = 6,     // a cross-GPU flag barrier gave up waiting for a peer
    kDevEpOverflow = 7,  // an expert-parallel receive buffer was too small: rows were dropped
};

// Current limit of the device-side waits in SM cycles (lsg_set_wait_limit_cycles; capi.cu).
long long wait_limit_cycles();

#if defined(__CUDACC__)

// ---------------------------------------------------------------------------
// Device: small PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Height of the token tiles of an expert with m rows when its ceil(m / tile_m) tiles share the
// rows evenly: m / tiles rounded up to 16 (never more than tile_m, a multiple of 16).  The tile
// map builder and the kernels that consume balanced maps both use this.
__host__ __device__ __forceinline__ int balanced_tile_rows(int m, int tile_m) {
    const int tiles = (m + tile_m - 1) / tile_m;
    if (tiles <= 1) return tile_m;
    return (((m + tiles - 1) / tiles) + 15) & ~15;
}

// True in exactly one lane of a converged warp (all 32 lanes must call it).
__device__ __forceinline__ bool elect_one_lane() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// rn(fl(x / d)) as a float, for |x / d| <= 127, without a division per element.  t = x * fl(1/d)
// corrected once by its exact remainder, fma(fma(-t, d, x), fl(1/d), t), is the correctly
// rounded quotient when fl(1/d) is the correctly rounded reciprocal and nothing under- or
// overflows (the last step of the usual division sequence); four instructions and no branch.
// A test for "x * fl(1/d) is near a half-integer" would not do: with bf16 inputs x / d is an
// exact half-integer for one value in 250, and a warp would take the division for one value
// in eight.  Scales outside [1e-28, 1e30] (all-zero and infinite blocks among them, rcp = 0
// for the former) keep the older form.
__device__ __forceinline__ float q8_round_f(float x, float d, float rcp) {
    const float t = x * rcp;
    if (d >= 1e-28f && d <= 1e30f) return rintf(fmaf(fmaf(-t, d, x), rcp, t));
    float k = rintf(t);
    if (fabsf(t - k) > 0.4999f) k = rintf(x / d);
    return k;
}

// Two packed bf16 values: bf16( silu(g) * u ), silu(g) = g / (1 + exp(-g)) in fp32.
__device__ __forceinline__ uint32_t silu_mul_bf16x2(uint32_t gw, uint32_t uw) {
    float a[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const float gv = __uint_as_float(h ? (gw & 0xFFFF0000u) : (gw << 16));
        const float uv = __uint_as_float(h ? (uw & 0xFFFF0000u) : (uw << 16));
        a[h] = (gv / (1.0f + expf(-gv))) * uv;
    }
    const __nv_bfloat162 r = __floats2bfloat162_rn(a[0], a[1]);
    return *reinterpret_cast<const uint32_t*>(&r);
}

// max(a, b) that is NaN when either operand is.
__device__ __forceinline__ float max_nan(float a, float b) {
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

// Eight values of one Q8_1 block at once -> their int8 codes, values 0-3 in w0 and 4-7 in w1.
// Same integers as q8_round_f, i.e. rn(fl(x / d)).  With bf16 inputs x / d is an exact
// half-integer for one value in 250, so a test for "near a tie" sends most warps into the
// division; instead the quotient itself is formed exactly: t = x * fl(1/d) corrected once by
// its exact remainder, fma(fma(-t, d, x), fl(1/d), t), is the correctly rounded x / d when
// fl(1/d) is the correctly rounded reciprocal (the final step of the usual division
// sequence), as long as nothing under- or overflows.  It is rounded to an integer by adding
// 1.5 * 2^23; the low mantissa byte of that sum is the integer in two's complement, so no
// conversion instruction is needed.  Blocks whose scale is outside [1e-28, 1e30] (zero and
// infinite blocks among them) and groups with a NaN take the plain path.
__device__ __forceinline__ void q8_round8(const float* x, float d, float rcp, uint32_t& w0, uint32_t& w1) {
    const float magic = 12582912.0f;
    float km[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float t = x[i] * rcp;
        km[i] = fmaf(fmaf(-t, d, x[i]), rcp, t) + magic;
    }
    const float m = max_nan(max_nan(max_nan(km[0], km[1]), max_nan(km[2], km[3])),
                            max_nan(max_nan(km[4], km[5]), max_nan(km[6], km[7])));
    const bool redo = !(d >= 1e-28f && d <= 1e30f) || m != m;
    if (redo) {
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = static_cast<uint32_t>(static_cast<int>(q8_round_f(x[i], d, rcp))) & 0xFFu;
        w0 = q[0] | (q[1] << 8) | (q[2] << 16) | (q[3] << 24);
        w1 = q[4] | (q[5] << 8) | (q[6] << 16) | (q[7] << 24);
        return;
    }
    const uint32_t b[8] = {__float_as_uint(km[0]), __float_as_uint(km[1]), __float_as_uint(km[2]), __float_as_uint(km[3]),
                           __float_as_uint(km[4]), __float_as_uint(km[5]), __float_as_uint(km[6]), __float_as_uint(km[7])};
    w0 = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
    w1 = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
                 : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    // Makes barrier initialisation visible to the async (TMA) proxy.
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t hint_ns = 2000u) {
    uint32_t ok;
    // The third operand is a suspend-time hint in nanoseconds: the thread sleeps in
    // hardware until the phase completes or the hint runs out, instead of polling
    // and taking issue slots from the warps that have work.
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Time limit of every device-side wait, in SM clock cycles (about 0.2 s at 2 GHz).  Nothing
// in these kernels legitimately waits longer than a few microseconds; the limit only ever
// runs out when a copy or an MMA was mis-issued, and then the kernel reports and returns.
// The SM-local cycle counter is used because it is read in a few cycles; the global
// nanosecond timer is not, and a read of it would sit on the critical path of every wait
// that does not succeed at once.
// Kernels take the limit as a launch argument (wait_limit_cycles()); this is its default.
constexpr long long kWaitLimitCycles = 400000000ll;

__device__ __forceinline__ long long sm_clock() {
    long long t;
    asm volatile("mov.u64 %0, %clock64;" : "=l"(t));
    return t;
}

// Waits for the phase with the given parity to complete.  Returns false (after
// recording `code` in *status) when the time limit runs out.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  unsigned int* status, unsigned int code,
                                                  uint32_t hint_ns = 2000u,
                                                  long long limit = kWaitLimitCycles) {
    if (mbar_try_wait(bar, parity, hint_ns)) return true;
    const long long t0 = sm_clock();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
            if (mbar_try_wait(bar, parity, hint_ns)) return true;
        }
        if (sm_clock() - t0 > limit) {
            if (status) atomicCAS(status, 0u, code);
            return false;
        }
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// src, dst 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Same with an L2 eviction-priority hint (weights are streamed once).
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem,
                                              uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue now / wait until the previous kernel's memory is visible.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// dp4a with unsigned first operand (u8 x s8 -> s32).
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(int a, int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ float fp16_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xFFFFu)));
}

#endif  // __CUDACC__

// Launch helper: plain or with the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace lsg
