// Expert-parallel MoE exchange over peer memory (NVLink / NVSwitch): the dispatch and the
// return of the routed rows are plain kernels that store straight into the destination
// GPU's buffer, instead of two all-to-all collectives with a host round trip for their split
// sizes and a regrouping pass on each side.  The reference has no multi-GPU code; this defines
// that layer for one node, one process per GPU.
//
// Every rank r owns experts [r*per, (r+1)*per).  Buffers the ranks share (symmetric
// allocations; each rank holds the peers' addresses in a device array):
//   counts table  int32 [world][E]   row s = rows rank s sends per global expert
//   receive buffer bf16 [capacity][H] rows for this rank's experts, grouped by
//                                    (local expert, source rank)
//   return buffer  bf16 [P][H]       expert outputs back at the sender, in the sender's
//                                    sorted-by-expert row order
// Per layer: publish counts (stores into every peer's table) | barrier | plan (every rank
// derives all offsets from the complete table, no communication) | send rows (gather from the
// token matrix + peer stores) | barrier | expert block on the receive buffer | return rows
// (peer stores) | barrier.  The barriers are the caller's (stream-ordered, between kernels);
// no kernel here waits for another GPU, and all peer accesses are stores.
#include "common.cuh"
#include "host.h"

namespace lsg {

namespace {

// counts of this rank -> row `rank` of every peer's table.
__global__ void __launch_bounds__(256)
ep_publish_counts_kernel(const int32_t* __restrict__ offs, int E, int rank, int world,
                         int32_t* const* __restrict__ tabs) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= E * world) return;
    const int peer = i / E, e = i - peer * E;
    tabs[peer][static_cast<size_t>(rank) * E + e] = offs[e + 1] - offs[e];
}

// One CTA of 1024 threads; E <= 1024, world * per = E.
//   send_base[e]            row in rank (e / per)'s receive buffer where this rank's block for
//                           global expert e starts
//   dst_start[el*world + s] start of block (local expert el, source s) in this rank's
//                           receive buffer; local_offsets[el] = dst_start[el*world]
//   ret_base[el*world + s]  row in source s's return buffer where that block goes back
//                           (= exclusive scan of s's counts at global expert rank*per + el)
//   info[0] = rows received (never more than the capacity), info[1] = 1 if some rank's receive
//   buffer is too small for what the ranks send it
// Overflow: every start and offset written here is clamped to `capacity`, so whatever runs on
// the receive buffer afterwards stays inside it; rows that do not fit are dropped at the
// sender (ep_send_rows_kernel zeroes their slots of the return buffer, so a dropped row
// contributes nothing to the combine) and the device status word reports kDevEpOverflow.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int32_t* __restrict__ tab, int rank, int world, int E, int capacity,
               int32_t* __restrict__ send_base, int32_t* __restrict__ local_offsets, int32_t* __restrict__ dst_start,
               int32_t* __restrict__ ret_base, int32_t* __restrict__ info, unsigned int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int wsum[32];
    __shared__ int colsum[1024];   // rows for global expert e over all sources
    __shared__ int overflow;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per = E / world;
    if (tid == 0) overflow = 0;
    // per-expert totals and, for this rank as a source, the rows of lower-ranked sources
    int total_e = 0, before_me = 0;
    if (tid < E) {
        for (int s = 0; s < world; ++s) {
            const int c = tab[static_cast<size_t>(s) * E + tid];
            if (s < rank) before_me += c;
            total_e += c;
        }
        colsum[tid] = total_e;
    }
    __syncthreads();
    // exclusive scan of the totals inside each destination rank's expert range
    if (tid < E) {
        const int d = tid / per, el = tid - d * per;
        int base = 0;
        for (int j = 0; j < el; ++j) base += colsum[d * per + j];
        send_base[tid] = base + before_me;
        if (el == per - 1 && base + total_e > capacity) overflow = 1;
    }
    // this rank as a receiver: blocks (el, s) in destination order
    const int B = per * world;
    int v = 0;
    if (tid < B) {
        const int el = tid / world, s = tid - el * world;
        v = tab[static_cast<size_t>(s) * E + rank * per + el];
    }
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = wsum[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += u;
        }
        wsum[lane] = w;
    }
    __syncthreads();
    const int excl = (warp > 0 ? wsum[warp - 1] : 0) + incl - v;
    if (tid < B) {
        const int el = tid / world, s = tid - el * world;
        dst_start[tid] = min(excl, capacity);
        if (s == 0) local_offsets[el] = min(excl, capacity);
        if (tid == B - 1) {
            local_offsets[per] = min(excl + v, capacity);
            info[0] = min(excl + v, capacity);
        }
        // where the block goes back: source s's rows for experts below rank*per + el
        int back = 0;
        const int ge = rank * per + el;
        for (int j = 0; j < ge; ++j) back += tab[static_cast<size_t>(s) * E + j];
        ret_base[tid] = back;
    }
    __syncthreads();
    if (tid == 0) {
        info[1] = overflow;
        if (overflow && status) atomicCAS(status, 0u, static_cast<unsigned int>(kDevEpOverflow));
    }
}

// Rows per CTA of the two copy kernels.  Two rows and at most 32 registers per thread, so that a
// copy CTA fits on an SM next to a resident 448-thread, 128-register GEMM CTA (57,344 + 8,192 =
// the whole register file) and an exchange on a second stream can run under the expert GEMMs.
constexpr int kEpRows = 2;

// Index of the last segment whose start is <= i, for nondecreasing starts[0..n): the number of
// starts that are <= i, minus one, counted by the whole CTA (one or a few loads per thread and
// one reduction) instead of a binary search per thread.  Uniform over the CTA.
__device__ __forceinline__ int segment_of(const int32_t* __restrict__ starts, int n, int i, int* s_count) {
    if (threadIdx.x == 0) *s_count = 0;
    __syncthreads();
    int c = 0;
    for (int t = threadIdx.x; t < n; t += blockDim.x) c += (__ldg(starts + t) <= i) ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(s_count, c);
    __syncthreads();
    return max(*s_count - 1, 0);
}

// Sorted row i (expert e, j-th row of e) -> row send_base[e] + j of rank e / per.
// A CTA copies kEpRows consecutive sorted rows: the expert of the first one is counted once,
// the following rows walk on from it; every thread has kEpRows independent 16-byte loads in
// flight before the stores into the destination GPUs' receive buffers.
__global__ void __launch_bounds__(256, 8)
ep_send_rows_kernel(const uint4* __restrict__ hidden, const int32_t* __restrict__ perm,
                    const int32_t* __restrict__ offs, const int32_t* __restrict__ send_base, int P, int top_k,
                    int vpr, int E, int per, uint4* const* __restrict__ recv, int capacity,
                    uint4* __restrict__ back_local, int le_lo, int le_hi) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int s_count;
    const int i0 = blockIdx.x * kEpRows;
    int e = segment_of(offs, E, i0, &s_count);   // last expert whose first row is <= i0
    int token[kEpRows], row[kEpRows], dst[kEpRows];
#pragma unroll
    for (int j = 0; j < kEpRows; ++j) {
        const int i = i0 + j;
        token[j] = -1;
        row[j] = 0;
        dst[j] = 0;
        if (i < P) {
            while (e + 1 < E && __ldg(offs + e + 1) <= i) ++e;
            dst[j] = e / per;
            const int le = e - dst[j] * per;   // the expert's index on its rank: only the group [le_lo, le_hi) travels
            if (le >= le_lo && le < le_hi) {
                row[j] = __ldg(send_base + e) + (i - __ldg(offs + e));
                token[j] = __ldg(perm + i) / top_k;
            }
        }
    }
    for (int v = threadIdx.x; v < vpr; v += blockDim.x) {
        uint4 val[kEpRows];
#pragma unroll
        for (int j = 0; j < kEpRows; ++j)
            val[j] = (token[j] >= 0 && row[j] < capacity) ? __ldg(hidden + static_cast<size_t>(token[j]) * vpr + v)
                                                          : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < kEpRows; ++j) {
            if (token[j] < 0) continue;
            if (row[j] < capacity) {
                recv[dst[j]][static_cast<size_t>(row[j]) * vpr + v] = val[j];
            } else if (back_local) {
                // no room at the destination: nothing comes back for this row, so its slot of this
                // rank's return buffer is cleared instead of keeping the previous layer's contents
                back_local[static_cast<size_t>(i0 + j) * vpr + v] = val[j];
            }
        }
    }
}

// Received row r of block (el, s) -> row ret_base[block] + j of source s's return buffer.
__global__ void __launch_bounds__(256, 8)
ep_return_rows_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ dst_start,
                      const int32_t* __restrict__ ret_base, const int32_t* __restrict__ info, int world, int B,
                      int vpr, int capacity, uint4* const* __restrict__ back,
                      const int32_t* __restrict__ local_offsets, int le_lo, int le_hi) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int s_count;
    int rows = min(__ldg(info), capacity);
    int first = 0;
    if (local_offsets) {   // only the rows of the local experts [le_lo, le_hi)
        first = min(__ldg(local_offsets + le_lo), rows);
        rows = min(__ldg(local_offsets + le_hi), rows);
    }
    const int r0 = first + blockIdx.x * kEpRows;
    if (r0 >= rows) return;   // uniform over the CTA
    int b = segment_of(dst_start, B, r0, &s_count);
    int row[kEpRows], dst[kEpRows];
#pragma unroll
    for (int j = 0; j < kEpRows; ++j) {
        const int r = r0 + j;
        row[j] = -1;
        dst[j] = 0;
        if (r < rows) {
            while (b + 1 < B && __ldg(dst_start + b + 1) <= r) ++b;
            row[j] = __ldg(ret_base + b) + (r - __ldg(dst_start + b));
            dst[j] = b % world;
        }
    }
    for (int v = threadIdx.x; v < vpr; v += blockDim.x) {
        uint4 val[kEpRows];
#pragma unroll
        for (int j = 0; j < kEpRows; ++j)
            val[j] = row[j] >= 0 ? __ldg(y + static_cast<size_t>(r0 + j) * vpr + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < kEpRows; ++j)
            if (row[j] >= 0) back[dst[j]][static_cast<size_t>(row[j]) * vpr + v] = val[j];
    }
}

// Cross-GPU barrier on the stream, owned by this library: every rank holds a flag array
// uint32 [world + 1] in peer-accessible memory (entry p = the last barrier rank p has arrived
// at, entry world = this rank's own count).  Arriving = storing the new count into entry
// `rank` of every peer's array (release, system scope, after a system-wide fence so that the
// peer stores of the kernels before it are visible first); waiting = polling the local array
// until every entry has reached the count, for at most `limit` SM cycles, after which the
// kernel records kDevBarrier in the status word and returns - a rank that never arrives costs
// its peers the limit, not a hung GPU.  Counts only grow, so a rank that is one barrier ahead
// cannot be mistaken for one that is behind.  mode: 1 arrive, 2 wait, 3 both.
__global__ void __launch_bounds__(64)
ep_barrier_kernel(uint32_t* const* __restrict__ flags, int rank, int world, int mode, long long limit,
                  unsigned int* __restrict__ status) {
    pdl_launch_dependents();
    pdl_wait_prior();
    uint32_t* mine = flags[rank];
    __shared__ uint32_t count;
    if (threadIdx.x == 0) {
        uint32_t c = *reinterpret_cast<volatile uint32_t*>(mine + world);
        if (mode & 1) {
            ++c;
            *reinterpret_cast<volatile uint32_t*>(mine + world) = c;
        }
        count = c;
    }
    __syncthreads();
    const uint32_t c = count;
    const int p = threadIdx.x;
    if (p >= world) return;
    if (mode & 1) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flags[p] + rank), "r"(c) : "memory");
    }
    if (mode & 2) {
        const long long t0 = sm_clock();
        for (;;) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine + p) : "memory");
            if (static_cast<int32_t>(v - c) >= 0) break;
            if (sm_clock() - t0 > limit) {
                if (status) atomicCAS(status, 0u, static_cast<unsigned int>(kDevBarrier));
                return;
            }
            __nanosleep(100);
        }
    }
}

int check_world(const char* op, int E, int world) {
    if (world < 1 || E < 1 || E > 1024 || E % world != 0)
        return fail(LSG_ERR_INVALID, "%s: need 1 <= num_experts <= 1024 divisible by the world size (E=%d, world=%d)", op, E,
                    world);
    return LSG_OK;
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_ep_publish_counts(const int32_t* expert_offsets, int num_experts, int rank, int world,
                                     void* const* counts_table_ptrs, void* stream) {
    int rc = check_world("ep_publish_counts", num_experts, world);
    if (rc != LSG_OK) return rc;
    if (rank < 0 || rank >= world || !expert_offsets || !counts_table_ptrs)
        return fail(LSG_ERR_INVALID, "ep_publish_counts: bad rank or null pointer");
    const int n = num_experts * world;
    LSG_CUDA_TRY(launch_kernel(ep_publish_counts_kernel, dim3((n + 255) / 256), dim3(256), 0,
                               static_cast<cudaStream_t>(stream), true, expert_offsets, num_experts, rank, world,
                               reinterpret_cast<int32_t* const*>(counts_table_ptrs)));
    return LSG_OK;
}

extern "C" int lsg_ep_plan(const int32_t* counts_table, int rank, int world, int num_experts, int capacity,
                           int32_t* send_base, int32_t* local_offsets, int32_t* dst_start, int32_t* ret_base,
                           int32_t* info, void* stream) {
    int rc = check_world("ep_plan", num_experts, world);
    if (rc != LSG_OK) return rc;
    if (rank < 0 || rank >= world || capacity < 0 || !counts_table || !send_base || !local_offsets || !dst_start ||
        !ret_base || !info)
        return fail(LSG_ERR_INVALID, "ep_plan: bad rank, negative capacity or null pointer");
    LSG_CUDA_TRY(launch_kernel(ep_plan_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), true,
                               counts_table, rank, world, num_experts, capacity, send_base, local_offsets, dst_start,
                               ret_base, info, device_status_word()));
    return LSG_OK;
}

extern "C" int lsg_ep_send_rows_group(const void* hidden_bf16, const int32_t* perm, const int32_t* expert_offsets,
                                      const int32_t* send_base, int num_pairs, int top_k, int H, int num_experts,
                                      int world, void* const* recv_buf_ptrs, int capacity, void* back_local,
                                      int local_expert_lo, int local_expert_hi, void* stream) {
    int rc = check_world("ep_send_rows", num_experts, world);
    if (rc != LSG_OK) return rc;
    if (num_pairs <= 0) return LSG_OK;
    if (!hidden_bf16 || !perm || !expert_offsets || !send_base || !recv_buf_ptrs || top_k < 1)
        return fail(LSG_ERR_INVALID, "ep_send_rows: null pointer or bad top_k");
    if (local_expert_lo < 0 || local_expert_hi > num_experts / world || local_expert_lo > local_expert_hi)
        return fail(LSG_ERR_INVALID, "ep_send_rows: bad local expert range [%d, %d)", local_expert_lo, local_expert_hi);
    if (H % 8 != 0 || (reinterpret_cast<uintptr_t>(hidden_bf16) & 15))
        return fail(LSG_ERR_ALIGNMENT, "ep_send_rows: H must be a multiple of 8 and buffers 16-byte aligned");
    const int vpr = H / 8;
    const int threads = vpr >= 256 ? 256 : ((vpr + 31) / 32) * 32;
    LSG_CUDA_TRY(launch_kernel(ep_send_rows_kernel, dim3(static_cast<unsigned>((num_pairs + kEpRows - 1) / kEpRows)), dim3(threads), 0,
                               static_cast<cudaStream_t>(stream), true, static_cast<const uint4*>(hidden_bf16), perm,
                               expert_offsets, send_base, num_pairs, top_k, vpr, num_experts, num_experts / world,
                               reinterpret_cast<uint4* const*>(recv_buf_ptrs), capacity,
                               static_cast<uint4*>(back_local), local_expert_lo, local_expert_hi));
    return LSG_OK;
}

extern "C" int lsg_ep_send_rows(const void* hidden_bf16, const int32_t* perm, const int32_t* expert_offsets,
                                const int32_t* send_base, int num_pairs, int top_k, int H, int num_experts, int world,
                                void* const* recv_buf_ptrs, int capacity, void* back_local, void* stream) {
    return lsg_ep_send_rows_group(hidden_bf16, perm, expert_offsets, send_base, num_pairs, top_k, H, num_experts, world,
                                  recv_buf_ptrs, capacity, back_local, 0, world > 0 ? num_experts / world : 0, stream);
}

extern "C" int lsg_ep_return_rows_group(const void* y_bf16, const int32_t* dst_start, const int32_t* ret_base,
                                        const int32_t* info, int world, int experts_per_rank, int H, int capacity,
                                        void* const* back_buf_ptrs, const int32_t* local_offsets, int local_expert_lo,
                                        int local_expert_hi, void* stream) {
    if (world < 1 || experts_per_rank < 1 || world * experts_per_rank > 1024)
        return fail(LSG_ERR_INVALID, "ep_return_rows: need 1 <= world * experts_per_rank <= 1024");
    if (capacity <= 0) return LSG_OK;
    if (!y_bf16 || !dst_start || !ret_base || !info || !back_buf_ptrs)
        return fail(LSG_ERR_INVALID, "ep_return_rows: null pointer");
    if (local_offsets && (local_expert_lo < 0 || local_expert_hi > experts_per_rank || local_expert_lo > local_expert_hi))
        return fail(LSG_ERR_INVALID, "ep_return_rows: bad local expert range [%d, %d)", local_expert_lo, local_expert_hi);
    if (H % 8 != 0 || (reinterpret_cast<uintptr_t>(y_bf16) & 15))
        return fail(LSG_ERR_ALIGNMENT, "ep_return_rows: H must be a multiple of 8 and buffers 16-byte aligned");
    const int vpr = H / 8;
    const int threads = vpr >= 256 ? 256 : ((vpr + 31) / 32) * 32;
    LSG_CUDA_TRY(launch_kernel(ep_return_rows_kernel, dim3(static_cast<unsigned>((capacity + kEpRows - 1) / kEpRows)), dim3(threads), 0,
                               static_cast<cudaStream_t>(stream), true, static_cast<const uint4*>(y_bf16), dst_start,
                               ret_base, info, world, world * experts_per_rank, vpr, capacity,
                               reinterpret_cast<uint4* const*>(back_buf_ptrs), local_offsets, local_expert_lo,
                               local_expert_hi));
    return LSG_OK;
}

extern "C" int lsg_ep_return_rows(const void* y_bf16, const int32_t* dst_start, const int32_t* ret_base,
                                  const int32_t* info, int world, int experts_per_rank, int H, int capacity,
                                  void* const* back_buf_ptrs, void* stream) {
    return lsg_ep_return_rows_group(y_bf16, dst_start, ret_base, info, world, experts_per_rank, H, capacity,
                                    back_buf_ptrs, nullptr, 0, experts_per_rank, stream);
}

extern "C" int lsg_ep_barrier(void* const* flag_ptrs, int rank, int world, int mode, void* stream) {
    if (world < 1 || world > 64 || rank < 0 || rank >= world || !flag_ptrs || mode < 1 || mode > 3)
        return fail(LSG_ERR_INVALID, "ep_barrier: need 1 <= world <= 64, 0 <= rank < world, mode 1..3, flag pointers");
    LSG_CUDA_TRY(launch_kernel(ep_barrier_kernel, dim3(1), dim3(64), 0, static_cast<cudaStream_t>(stream), true,
                               reinterpret_cast<uint32_t* const*>(flag_ptrs), rank, world, mode, wait_limit_cycles(),
                               device_status_word()));
    return LSG_OK;
}
