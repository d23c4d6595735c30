// Grouped (MoE) GGUF mat-vec: D[rows of expert e, :] = Q8_1(A[rows of e]) . decode(W_e)^T for
// every expert that has rows, in ONE launch, routed on the device.
//
// Replaces the reference's grouped decode kernels (gguf_mmvq_grouped_*_kernel,
// csrc/sm120/gemm/gguf/gguf_grouped_int.cu:90-653, launched as one warp or one CTA per
// (output channel, expert)).  Here the work list is a device-built segment list
// (routing.cu): segment = (expert, first row, rows <= image capacity).  The segments'
// weight rows form one virtual row space of n_segments * N rows, cut into equal
// contiguous ranges, one per persistent CTA, and streamed through the same bulk-copy
// ring as the single-weight kernel (mmvq.cuh).  A CTA rebuilds its activation image when
// its range crosses into another segment; within a segment, row groups are claimed from
// a queue.  Per-expert row counts are only known on the device, so the number of batch
// rows per register pass (1, 2, 4 or 8) is chosen per segment inside the kernel.
#pragma once

#include "mmvq.cuh"

namespace lsg {

constexpr int kGroupedMaxSlabs = 1024;  // slab table entries per CTA

struct GroupedArgs {
    const uint8_t* xq;          // Q8_1 blocks of all rows [T][K/32][36]
    const void* const* B_ptrs;  // [E] packed weights (device array of device pointers)
    const int* seg;             // [0] = n_segments, then (expert, first row, rows) triples
    void* D;                    // [T][N] bf16 or f32
    unsigned int* status;
    int N, K, out_f32;
    int row_bytes, slab_rows, stages, stage_bytes, x_bytes;
    int cons_warps;
};

// Per-type entry point (mmvq_inst.cu)
#define LSG_DECLARE_MMVQ_GROUPED(id)                                                       \
    int mmvq_grouped_launch_t##id(GroupedArgs a, const MmvqTune& tn, int max_segments,     \
                                  cudaStream_t stream, bool pdl);                          \
    int mmvq_grouped_max_rows_t##id(int K, const MmvqTune& tn);
LSG_DECLARE_MMVQ_GROUPED(0) LSG_DECLARE_MMVQ_GROUPED(1) LSG_DECLARE_MMVQ_GROUPED(2)
LSG_DECLARE_MMVQ_GROUPED(3) LSG_DECLARE_MMVQ_GROUPED(4) LSG_DECLARE_MMVQ_GROUPED(5)
LSG_DECLARE_MMVQ_GROUPED(6) LSG_DECLARE_MMVQ_GROUPED(7)

#if defined(__CUDACC__)

template <int T, int RW, int L>
__global__ void __launch_bounds__(512, 1) mmvq_grouped_kernel(const GroupedArgs a) {
    using D = Mmvq<T>;
    constexpr int SUBS = 32 / L;
    constexpr int RPP = SUBS * RW;

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* x_img = smem;
    uint8_t* ring = smem + a.x_bytes;
    uint64_t* full = reinterpret_cast<uint64_t*>(ring + static_cast<size_t>(a.stages) * a.stage_bytes);
    uint64_t* empty = full + kMmvqMaxStages;
    int* next_group = reinterpret_cast<int*>(empty + kMmvqMaxStages);
    int* n_slabs_sh = next_group + 1;
    volatile int* abort_flag = next_group + 2;  // set when a bounded wait ran out
    volatile int* slab_in_stage = next_group + 3;
    // slab table: (segment, first weight row, rows) per slab
    int* slab_tab = const_cast<int*>(slab_in_stage) + kMmvqMaxStages;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int n_cons_warps = (blockDim.x >> 5) - 1;
    const bool is_producer = (warp == n_cons_warps);
    const int groups_per_slab = (a.slab_rows + RPP - 1) / RPP;

    pdl_launch_dependents();
    pdl_wait_prior();  // the segment list and the activations come from earlier kernels

    if (tid == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], groups_per_slab);
            slab_in_stage[s] = -1;
        }
        *next_group = 0;
        *abort_flag = 0;
        mbar_fence_init();
        // This CTA's range of the virtual row space, cut into slabs that never cross a
        // segment boundary.
        const long long V = static_cast<long long>(a.seg[0]) * a.N;
        const long long vb = V * blockIdx.x / gridDim.x, ve = V * (blockIdx.x + 1) / gridDim.x;
        int n = 0;
        for (long long cur = vb; cur < ve && n < kGroupedMaxSlabs;) {
            const int sg = static_cast<int>(cur / a.N);
            const int n0 = static_cast<int>(cur - static_cast<long long>(sg) * a.N);
            long long rows = a.slab_rows;
            if (rows > a.N - n0) rows = a.N - n0;
            if (rows > ve - cur) rows = ve - cur;
            slab_tab[3 * n] = sg;
            slab_tab[3 * n + 1] = n0;
            slab_tab[3 * n + 2] = static_cast<int>(rows);
            cur += rows;
            ++n;
            if (n == kGroupedMaxSlabs && cur < ve && a.status) atomicCAS(a.status, 0u, static_cast<unsigned int>(kDevSlabTable));
        }
        *n_slabs_sh = n;
    }
    __syncthreads();
    const int n_slabs = *n_slabs_sh;

    if (is_producer) {
        // The whole warp walks the loop with the same values in every lane; one elected lane
        // issues the copy (bulk copies and barrier operations take warp-uniform operands and
        // cost several times as much inside a one-lane branch).
        const uint64_t policy = l2_policy_evict_first();
        int s = 0;
        uint32_t lap = 0;
        for (int i = 0; i < n_slabs; ++i) {
            if (lap > 0) {
                const bool ok = __all_sync(0xffffffffu, !*abort_flag && mbar_wait_bounded(&empty[s], (lap - 1) & 1, a.status, kDevWaitEmpty));
                if (!ok) {
                    *abort_flag = 1;
                    break;
                }
            }
            const int sg = slab_tab[3 * i], n0 = slab_tab[3 * i + 1], rows = slab_tab[3 * i + 2];
            const int e = a.seg[1 + 3 * sg];
            const uintptr_t w_base = reinterpret_cast<uintptr_t>(a.B_ptrs[e]);
            const uintptr_t w_end_al = (w_base + static_cast<uintptr_t>(a.N) * a.row_bytes) & ~uintptr_t(15);
            const uintptr_t src_b = w_base + static_cast<uintptr_t>(n0) * a.row_bytes;
            const uintptr_t src_e = src_b + static_cast<uintptr_t>(rows) * a.row_bytes;
            uintptr_t cp_b = src_b & ~uintptr_t(15);
            uintptr_t cp_e = (src_e + 15) & ~uintptr_t(15);
            uint8_t* dst = ring + static_cast<size_t>(s) * a.stage_bytes;
            const bool unaligned = (w_base & 15) != 0;
            const bool ragged = !unaligned && cp_e > w_end_al;
            if (unaligned) cp_e = cp_b;
            else if (ragged) cp_e = w_end_al > cp_b ? w_end_al : cp_b;
            const uint32_t bytes = static_cast<uint32_t>(cp_e - cp_b);
            if (elect_one_lane()) {
                if (unaligned) {
                    // Weights must be 16-byte aligned for bulk copies; fall back to byte
                    // loads for such an expert rather than read before its buffer.
                    for (uintptr_t p = src_b; p < src_e; ++p)
                        dst[(p - src_b) + (src_b & 15)] = *reinterpret_cast<const uint8_t*>(p);
                } else if (ragged) {
                    for (uintptr_t p = cp_e; p < src_e; ++p)
                        dst[p - cp_b] = *reinterpret_cast<const uint8_t*>(p);
                }
                slab_in_stage[s] = i;
                if (bytes > 0) {
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_g2s_hint(dst, reinterpret_cast<const void*>(cp_b), bytes, &full[s], policy);
                } else {
                    mbar_arrive(&full[s]);
                }
            }
            __syncwarp();
            if (++s == a.stages) {
                s = 0;
                ++lap;
            }
        }
        return;
    }

    // ----------------------------------------------------------------------
    // Consumers: segment by segment
    // ----------------------------------------------------------------------
    const int n_cons = n_cons_warps * 32;
    const int sub = lane / L;
    XView xv;
    xv.rowb = x_row_bytes<T>(a.K);
    xv.d_off = a.K;
    xv.s_off = a.K + (a.K / 32) * 4;
    xv.U = a.K / D::UV;
    const uint32_t x_base = smem_u32(x_img);
    const size_t xq_row = static_cast<size_t>(a.K / 32) * kQ8_1Bytes;

    int sl = 0;
    while (sl < n_slabs) {
        const int sg = slab_tab[3 * sl];
        int sl_end = sl + 1;
        while (sl_end < n_slabs && slab_tab[3 * sl_end] == sg) ++sl_end;
        const int arow0 = a.seg[2 + 3 * sg], mcount = a.seg[3 + 3 * sg];

        asm volatile("bar.sync 1, %0;" ::"r"(n_cons) : "memory");  // previous image no longer read
        build_x_image<T>(x_img, a.xq + static_cast<size_t>(arow0) * xq_row, mcount, a.K, tid, n_cons);
        if (tid == 0) *next_group = 0;
        asm volatile("bar.sync 1, %0;" ::"r"(n_cons) : "memory");

        const int seg_groups = (sl_end - sl) * groups_per_slab;
        for (;;) {
            int gidx = 0;
            if (lane == 0) gidx = atomicAdd(next_group, 1);
            gidx = __shfl_sync(0xffffffffu, gidx, 0);
            if (gidx >= seg_groups) break;
            const int i = sl + gidx / groups_per_slab;
            const int g = (gidx % groups_per_slab) * RPP;
            const int s = i % a.stages;
            const int n0 = slab_tab[3 * i + 1], nrows = slab_tab[3 * i + 2];
            // After a wait has run out the warps keep walking the loops (the named
            // barriers above need every warp) but no longer wait or compute.
            bool ok = *abort_flag == 0;
            if (ok && slab_in_stage[s] != i) {
                const long long t0 = sm_clock();
                while (slab_in_stage[s] != i && *abort_flag == 0) {
                    __nanosleep(64);
                    if (sm_clock() - t0 > kWaitLimitCycles) {
                        if (a.status) atomicCAS(a.status, 0u, static_cast<unsigned int>(kDevWaitFull));
                        *abort_flag = 1;
                    }
                }
                ok = *abort_flag == 0;
            }
            if (ok && !mbar_wait_bounded(&full[s], (i / a.stages) & 1, a.status, kDevWaitFull)) {
                *abort_flag = 1;
                ok = false;
            }
            if (ok && g < nrows) {
                const int e = a.seg[1 + 3 * sg];
                const uintptr_t src_b = reinterpret_cast<uintptr_t>(a.B_ptrs[e]) +
                                        static_cast<uintptr_t>(n0) * a.row_bytes;
                const uint32_t slab = smem_u32(ring + static_cast<size_t>(s) * a.stage_bytes) +
                                      static_cast<uint32_t>(src_b & 15);
                uint32_t raddr[RW];
#pragma unroll
                for (int r = 0; r < RW; ++r)
                    raddr[r] = slab + static_cast<uint32_t>(min(g + sub * RW + r, nrows - 1)) * a.row_bytes;
                for (int m0 = 0; m0 < mcount; m0 += 8) {
                    const int rem = mcount - m0;
                    xv.base = x_base + m0 * xv.rowb;
                    xv.mlast = rem - 1;
                    if (rem == 1)
                        group_dot_store<T, 1, RW, L>(raddr, xv, lane, g + sub * RW, nrows, n0, arow0 + m0,
                                                     rem, a.D, a.N, a.out_f32, false);
                    else if (rem == 2)
                        group_dot_store<T, 2, RW, L>(raddr, xv, lane, g + sub * RW, nrows, n0, arow0 + m0,
                                                     rem, a.D, a.N, a.out_f32, false);
                    else if (rem <= 4)
                        group_dot_store<T, 4, RW, L>(raddr, xv, lane, g + sub * RW, nrows, n0, arow0 + m0,
                                                     rem, a.D, a.N, a.out_f32, false);
                    else
                        group_dot_store<T, 8, RW, L>(raddr, xv, lane, g + sub * RW, nrows, n0, arow0 + m0,
                                                     rem, a.D, a.N, a.out_f32, false);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }
        sl = sl_end;
    }
}

#endif  // __CUDACC__

}  // namespace lsg
