// Device-side routing metadata for the grouped (MoE) GEMMs: everything is derived from
// expert_offsets on the GPU, so the grouped calls never synchronize with the host and
// can be captured in a CUDA graph.
//
//   * active expert list  - ascending indices of experts with rows, -1 padded to `cap`;
//     same contents as the reference's build_active_expert_list
//     (csrc/sm120/gemm/gguf/gguf_grouped_int.cu:156-187);
//   * m-tile map          - tile t -> (expert, first row), -1 padded to T_max; same
//     contents as build_mmq_tile_map (gguf_grouped_int.cu:46-66);
//   * segment list        - (expert, first row, rows) pieces of at most `max_rows` rows,
//     the work list of the grouped mat-vec kernel (no counterpart in the reference).
//
// One warp does each scan with ballots / prefix sums; expert counts are a few hundred.
#include "common.cuh"
#include "host.h"

namespace lsg {

namespace {

__global__ void active_expert_list_kernel(const int32_t* __restrict__ offs, int E, int cap,
                                          int* __restrict__ active) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    int written = 0;
    for (int base = 0; base < E && written < cap; base += 32) {
        const int e = base + lane;
        const bool has = e < E && (offs[e + 1] - offs[e]) > 0;
        const unsigned m = __ballot_sync(0xffffffffu, has);
        if (has) {
            const int slot = written + __popc(m & ((1u << lane) - 1u));
            if (slot < cap) active[slot] = e;
        }
        written += __popc(m);
    }
    for (int s = written + lane; s < cap; s += 32) active[s] = -1;
}

// `rows` bounds every offset (callers whose offsets come from another GPU's counts pass the
// row capacity of their buffers; INT_MAX leaves the offsets as they are).
// balanced: an expert's tiles share its rows evenly (height = rows / tiles, rounded up to 16)
// instead of full tiles followed by a remainder; the consumer derives the same height.
__global__ void mmq_tile_map_kernel(const int32_t* __restrict__ offs, int E, int tile_m, int T_max, int rows,
                                    int balanced, int* __restrict__ tile_expert, int* __restrict__ tile_mstart) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    int t0 = 0;  // tiles emitted so far (warp-uniform)
    for (int base = 0; base < E; base += 32) {
        const int e = base + lane;
        int off = 0, nt = 0, height = tile_m;
        if (e < E) {
            off = min(offs[e], rows);
            const int m = min(offs[e + 1], rows) - off;
            nt = m > 0 ? (m + tile_m - 1) / tile_m : 0;
            if (balanced && nt > 0) height = balanced_tile_rows(m, tile_m);
        }
        // exclusive prefix sum of nt over the warp
        int incl = nt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        const int first = t0 + incl - nt;
        for (int i = 0; i < nt; ++i) {
            const int t = first + i;
            if (t < T_max) {
                tile_expert[t] = e;
                tile_mstart[t] = off + i * height;
            }
        }
        t0 += __shfl_sync(0xffffffffu, incl, 31);
    }
    for (int t = t0 + lane; t < T_max; t += 32) {
        tile_expert[t] = -1;
        tile_mstart[t] = 0;
    }
}

// seg[0] = number of segments; then triples (expert, first row, rows).  Experts with a
// null weight pointer are skipped, as the reference's host loop skips them
// (gguf_grouped_gemm.cu:114-118 with B_e == nullptr guarded in the engine).
__global__ void segment_list_kernel(const int32_t* __restrict__ offs, const void* const* __restrict__ B_ptrs,
                                    int E, int max_rows, int max_segments, int rows, int* __restrict__ seg) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    int s0 = 0;
    for (int base = 0; base < E; base += 32) {
        const int e = base + lane;
        int off = 0, m = 0, ns = 0;
        if (e < E) {
            off = min(offs[e], rows);
            m = min(offs[e + 1], rows) - off;
            if (m < 0 || B_ptrs[e] == nullptr) m = 0;
            ns = (m + max_rows - 1) / max_rows;
        }
        int incl = ns;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        const int first = s0 + incl - ns;
        for (int i = 0; i < ns; ++i) {
            const int s = first + i;
            if (s < max_segments) {
                seg[1 + 3 * s] = e;
                seg[2 + 3 * s] = off + i * max_rows;
                seg[3 + 3 * s] = min(max_rows, m - i * max_rows);
            }
        }
        s0 += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) seg[0] = min(s0, max_segments);
}

}  // namespace

int build_active_expert_list(const int32_t* offs, int E, int cap, int* active, cudaStream_t s) {
    if (cap <= 0) return LSG_OK;
    LSG_CUDA_TRY(launch_kernel(active_expert_list_kernel, dim3(1), dim3(32), 0, s, true, offs, E, cap,
                               active));
    return LSG_OK;
}

int build_mmq_tile_map(const int32_t* offs, int E, int tile_m, int T_max, int* tile_expert,
                       int* tile_mstart, cudaStream_t s, int rows, bool balanced) {
    if (T_max <= 0) return LSG_OK;
    LSG_CUDA_TRY(launch_kernel(mmq_tile_map_kernel, dim3(1), dim3(32), 0, s, true, offs, E, tile_m,
                               T_max, rows, balanced ? 1 : 0, tile_expert, tile_mstart));
    return LSG_OK;
}

int build_segment_list(const int32_t* offs, const void* const* B_ptrs, int E, int max_rows,
                       int max_segments, int* seg, cudaStream_t s, int rows) {
    LSG_CUDA_TRY(launch_kernel(segment_list_kernel, dim3(1), dim3(32), 0, s, true, offs, B_ptrs, E,
                               max_rows, max_segments, rows, seg));
    return LSG_OK;
}

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_build_active_expert_list(const int32_t* expert_offsets, int num_experts, int cap,
                                            int32_t* active_experts, void* stream) {
    if (num_experts < 0 || cap < 0 || !expert_offsets || (cap > 0 && !active_experts))
        return fail(LSG_ERR_INVALID, "build_active_expert_list: bad argument");
    return build_active_expert_list(expert_offsets, num_experts, cap, active_experts,
                                    static_cast<cudaStream_t>(stream));
}

extern "C" int lsg_build_mmq_tile_map(const int32_t* expert_offsets, int num_experts, int tile_m,
                                      int t_max, int32_t* tile_expert, int32_t* tile_mstart,
                                      void* stream) {
    if (num_experts < 0 || tile_m <= 0 || t_max < 0 || !expert_offsets ||
        (t_max > 0 && (!tile_expert || !tile_mstart)))
        return fail(LSG_ERR_INVALID, "build_mmq_tile_map: bad argument");
    return build_mmq_tile_map(expert_offsets, num_experts, tile_m, t_max, tile_expert, tile_mstart,
                              static_cast<cudaStream_t>(stream));
}
