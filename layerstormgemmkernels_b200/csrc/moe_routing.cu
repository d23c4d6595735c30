// MoE routing for the grouped GEMMs: router softmax + top-k + renormalisation, the stable
// permutation that groups (token, slot) pairs by expert, row gather ("permute") and the
// weighted combine ("unpermute").  The reference has none of this - its grouped operators
// take rows that are already permuted plus expert_offsets (gguf_grouped_gemm.h:20-24,
// grouped_gemm.h:24-25) - so the definition these kernels follow is the usual one:
//   p = softmax(logits, -1);  (w, idx) = topk(p, k);  w /= sum(w)
//   pairs (token, slot) in token-major order, stably sorted by idx -> permutation
//   expert_offsets = [0, cumsum(bincount(idx))]
// Everything stays on the device (no host synchronisation).
#include "common.cuh"
#include "host.h"

namespace lsg {

namespace {

constexpr int kMaxTopK = 16;

// One warp per token, PER experts per lane (E <= 32 * PER <= 1024).
template <int PER>
__global__ void __launch_bounds__(256)
moe_route_kernel(const float* __restrict__ logits, int T, int E, int k, int32_t* __restrict__ topk_idx,
                 float* __restrict__ topk_w) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const float* row = logits + static_cast<size_t>(t) * E;
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? row[e] : -INFINITY;
        mx = fmaxf(mx, v[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int e = i * 32 + lane;
        v[i] = e < E ? expf(v[i] - mx) : -1.0f;  // -1 marks "not a candidate"
        if (e < E) sum += v[i];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    // k rounds of arg-max over the remaining candidates; ties go to the lower expert id
    float wsel[kMaxTopK];
    int isel[kMaxTopK];
    float wsum = 0.0f;
    for (int r = 0; r < k; ++r) {
        float best = -2.0f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * 32 + lane;
            if (v[i] > best) { best = v[i]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (i * 32 + lane == bi) v[i] = -1.0f;
        wsel[r] = best * inv;
        isel[r] = bi;
        wsum += wsel[r];
    }
    if (lane == 0) {
        for (int r = 0; r < k; ++r) {
            topk_idx[static_cast<size_t>(t) * k + r] = isel[r];
            topk_w[static_cast<size_t>(t) * k + r] = wsel[r] / wsum;
        }
    }
}

// Stable grouping of the pairs by expert as a counting sort over chunks of 256 pairs:
//   1. per-chunk histogram over the experts,
//   2. per expert, exclusive scan of the histograms over the chunks (in place) and the
//      exclusive scan of the totals over the experts (= expert_offsets),
//   3. per chunk, each pair's rank among the earlier pairs of the same expert:
//      earlier chunks (step 2), earlier warps of the chunk, earlier lanes of the warp.
// Pairs whose expert id lies outside [0, E) are ignored.
constexpr int kChunk = 256;

__global__ void __launch_bounds__(kChunk)
moe_chunk_hist_kernel(const int32_t* __restrict__ idx, int P, int E, int32_t* __restrict__ hist) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int h[1024];
    for (int e = threadIdx.x; e < E; e += kChunk) h[e] = 0;
    __syncthreads();
    const int i = blockIdx.x * kChunk + threadIdx.x;
    if (i < P) {
        const int e = idx[i];
        if (e >= 0 && e < E) atomicAdd(&h[e], 1);
    }
    __syncthreads();
    // laid out [expert][chunk]: the scan below reads consecutive chunks of one expert
    for (int e = threadIdx.x; e < E; e += kChunk) hist[static_cast<size_t>(e) * gridDim.x + blockIdx.x] = h[e];
}

// One CTA of 1024 threads (E <= 1024).  Phase 1: warp w scans the chunk histograms of experts
// w, w + 32, ... (lanes = 32 consecutive chunks, warp prefix sum, carry between groups of 32
// chunks) and leaves the expert's total in shared memory.  Phase 2: thread e takes part in the
// exclusive scan of the totals over the experts.
__global__ void __launch_bounds__(1024)
moe_chunk_scan_kernel(int32_t* __restrict__ hist, int n_chunks, int E, int32_t* __restrict__ offsets) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int totals[1024];
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int e = warp; e < E; e += 32) {
        int carry = 0;
        // up to 128 chunks are fetched before the first scan step: the loads of an expert's row
        // are contiguous and independent, only the carry is sequential
        int pre[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = j * 32 + lane;
            pre[j] = c < n_chunks ? hist[static_cast<size_t>(e) * n_chunks + c] : 0;
        }
        for (int c0 = 0; c0 < n_chunks; c0 += 32) {
            const int c = c0 + lane;
            const size_t at = static_cast<size_t>(e) * n_chunks + c;
            int v;
            if (c0 < 128) {
                const int j = c0 >> 5;
                v = j == 0 ? pre[0] : (j == 1 ? pre[1] : (j == 2 ? pre[2] : pre[3]));
            } else {
                v = c < n_chunks ? hist[at] : 0;
            }
            int incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += u;
            }
            if (c < n_chunks) hist[at] = carry + incl - v;
            carry += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) totals[e] = carry;
    }
    __syncthreads();
    const int e = tid;
    const int total = e < E ? totals[e] : 0;
    int incl = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = wsum[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        wsum[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int before = warp > 0 ? wsum[warp - 1] : 0;
    if (e < E) offsets[e] = before + incl - total;
    if (e == E - 1) offsets[E] = before + incl;
}

// perm[row] = pair, inv[pair] = row.
__global__ void __launch_bounds__(kChunk)
moe_place_kernel(const int32_t* __restrict__ idx, int P, int E, const int32_t* __restrict__ chunk_base,
                 const int32_t* __restrict__ offsets, int32_t* __restrict__ perm, int32_t* __restrict__ inv) {
    pdl_launch_dependents();
    pdl_wait_prior();
    extern __shared__ int whist[];  // [8 warps][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < (kChunk / 32) * E; j += kChunk) whist[j] = 0;
    __syncthreads();
    const int i = blockIdx.x * kChunk + threadIdx.x;
    int e = i < P ? idx[i] : -1;
    if (e >= E) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) whist[warp * E + e] = __popc(same);
    __syncthreads();
    if (e >= 0) {
        int before = 0;
        for (int w = 0; w < warp; ++w) before += whist[w * E + e];
        const int row = offsets[e] + chunk_base[static_cast<size_t>(e) * gridDim.x + blockIdx.x] + before + rank;
        perm[row] = i;
        inv[i] = row;
    }
}

// The three steps above in one CTA, for P <= 1024 pairs (decode-sized batches, where three
// dependent launches cost more than the work): thread i owns pair i; per-warp histograms in
// shared memory ([warps][E], the caller checks that they fit), their sum over the warps per
// expert, the exclusive scan over the experts, then each pair's row.
__global__ void __launch_bounds__(1024)
moe_permutation_small_kernel(const int32_t* __restrict__ idx, int P, int E, int32_t* __restrict__ offsets,
                             int32_t* __restrict__ perm, int32_t* __restrict__ inv) {
    pdl_launch_dependents();
    pdl_wait_prior();
    extern __shared__ int whist[];  // [n_warps][E]
    __shared__ int totals[1024];
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_warps = (P + 31) >> 5;
    for (int j = tid; j < n_warps * E; j += 1024) whist[j] = 0;
    __syncthreads();
    int e = tid < P ? idx[tid] : -1;
    if (e >= E) e = -1;
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) whist[warp * E + e] = __popc(same);
    __syncthreads();
    // thread x: total of expert x, and the warps' counts turned into exclusive prefixes
    int total = 0;
    if (tid < E) {
        for (int w = 0; w < n_warps; ++w) {
            const int v = whist[w * E + tid];
            whist[w * E + tid] = total;
            total += v;
        }
    }
    int incl = total;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = wsum[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        wsum[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int before = warp > 0 ? wsum[warp - 1] : 0;
    if (tid < E) {
        totals[tid] = before + incl - total;
        offsets[tid] = before + incl - total;
    }
    if (tid == E - 1) offsets[E] = before + incl;
    __syncthreads();
    if (e >= 0) {
        const int row = totals[e] + whist[warp * E + e] + rank;
        perm[row] = tid;
        inv[tid] = row;
    }
}

// out[row, :] = hidden[perm[row] / k, :]   (bf16 rows, 16-byte vectors)
__global__ void __launch_bounds__(256)
moe_gather_kernel(const uint4* __restrict__ hidden, const int32_t* __restrict__ perm, int k, int rows,
                  int vec_per_row, uint4* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<long long>(rows) * vec_per_row) return;
    const int row = static_cast<int>(i / vec_per_row), c = static_cast<int>(i - static_cast<long long>(row) * vec_per_row);
    out[i] = __ldg(hidden + static_cast<size_t>(perm[row] / k) * vec_per_row + c);
}

// out[t, :] = sum_s w[t, s] * y[inv[t * k + s], :], slots in order, fp32 accumulate.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ inv,
                   const float* __restrict__ w, int T, int k, int H, __nv_bfloat16* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int hv = H >> 1;
    if (i >= static_cast<long long>(T) * hv) return;
    const int t = static_cast<int>(i / hv), c = static_cast<int>(i - static_cast<long long>(t) * hv);
    float a0 = 0.0f, a1 = 0.0f;
    for (int s = 0; s < k; ++s) {
        const int row = inv[static_cast<size_t>(t) * k + s];
        const float ws = w[static_cast<size_t>(t) * k + s];
        const __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(y + static_cast<size_t>(row) * H)[c];
        a0 = fmaf(ws, __bfloat162float(v.x), a0);
        a1 = fmaf(ws, __bfloat162float(v.y), a1);
    }
    reinterpret_cast<__nv_bfloat162*>(out + static_cast<size_t>(t) * H)[c] = __floats2bfloat162_rn(a0, a1);
}

// The same for H a multiple of 8 and 16-byte aligned rows: one token per blockIdx.x, one 16-byte
// vector (eight columns) per thread and slot, the k slot rows of a vector in flight together;
// same sum order (slots ascending, fmaf in fp32), hence the same bits.
template <int KMAX>
__global__ void __launch_bounds__(256)
moe_combine_vec_kernel(const uint4* __restrict__ y, const int32_t* __restrict__ inv, const float* __restrict__ w,
                       int k, int vpr, uint4* __restrict__ out) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int t = blockIdx.x;
    for (int v = threadIdx.x; v < vpr; v += blockDim.x) {
        uint4 r[KMAX];
        float ws[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
            if (s < k) {
                const int row = __ldg(inv + static_cast<size_t>(t) * k + s);
                ws[s] = __ldg(w + static_cast<size_t>(t) * k + s);
                r[s] = __ldg(y + static_cast<size_t>(row) * vpr + v);
            }
        }
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
            if (s < k) {
                const uint32_t q[4] = {r[s].x, r[s].y, r[s].z, r[s].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] = fmaf(ws[s], __uint_as_float(q[i] << 16), acc[2 * i]);
                    acc[2 * i + 1] = fmaf(ws[s], __uint_as_float(q[i] & 0xFFFF0000u), acc[2 * i + 1]);
                }
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            o[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        out[static_cast<size_t>(t) * vpr + v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// Expert-parallel receive side: rows arrive grouped by (source rank, local expert); the
// grouped GEMM wants them grouped by (local expert, source rank).  counts[s * per + e] = rows
// from source s for local expert e.  One CTA: exclusive scans of the block sizes in both
// orders.  starts_recv[s * per + e], starts_dst[e * world + s], local_offsets[per + 1].
__global__ void __launch_bounds__(1024)
ep_block_starts_kernel(const int32_t* __restrict__ counts, int world, int per, int32_t* __restrict__ starts_recv,
                       int32_t* __restrict__ starts_dst, int32_t* __restrict__ local_offsets) {
    pdl_launch_dependents();
    pdl_wait_prior();
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int B = world * per;
    for (int pass = 0; pass < 2; ++pass) {
        // pass 0: receive order (s, e); pass 1: destination order (e, s)
        int v = 0;
        if (tid < B) v = pass == 0 ? counts[tid] : counts[(tid % world) * per + tid / world];
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
            if (pass == 0) starts_recv[tid] = excl;
            else {
                starts_dst[tid] = excl;
                if (tid % world == 0) local_offsets[tid / world] = excl;
                if (tid == B - 1) local_offsets[per] = excl + v;
            }
        }
        __syncthreads();
    }
}

// order[i] = receive-order row of destination row i; inv_order[that row] = i.
__global__ void __launch_bounds__(256)
ep_order_kernel(const int32_t* __restrict__ counts, const int32_t* __restrict__ starts_recv,
                const int32_t* __restrict__ starts_dst, int world, int per, int rows, int32_t* __restrict__ order,
                int32_t* __restrict__ inv_order) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= rows) return;
    const int B = world * per;
    // last destination block whose start is <= i and that is not empty before i
    int lo = 0, hi = B - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (starts_dst[mid] <= i) lo = mid;
        else hi = mid - 1;
    }
    const int e = lo / world, s_rank = lo % world;
    const int b = s_rank * per + e;
    const int src = starts_recv[b] + (i - starts_dst[lo]);
    order[i] = src;
    inv_order[src] = i;
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_moe_route(const float* logits, int num_tokens, int num_experts, int top_k,
                             int32_t* topk_idx, float* topk_weights, void* stream) {
    if (num_tokens <= 0) return LSG_OK;
    if (!logits || !topk_idx || !topk_weights) return fail(LSG_ERR_INVALID, "moe_route: null pointer");
    if (num_experts < 1 || num_experts > 1024 || top_k < 1 || top_k > kMaxTopK || top_k > num_experts)
        return fail(LSG_ERR_INVALID, "moe_route: need 1 <= top_k <= min(16, E) and E <= 1024 (E=%d, k=%d)",
                    num_experts, top_k);
    const dim3 rg((num_tokens + 7) / 8), rb(256);
    if (num_experts <= 128)
        LSG_CUDA_TRY(launch_kernel(moe_route_kernel<4>, rg, rb, 0,
                               static_cast<cudaStream_t>(stream), true, logits, num_tokens, num_experts,
                               top_k, topk_idx, topk_weights));
    else if (num_experts <= 256)
        LSG_CUDA_TRY(launch_kernel(moe_route_kernel<8>, rg, rb, 0,
                               static_cast<cudaStream_t>(stream), true, logits, num_tokens, num_experts,
                               top_k, topk_idx, topk_weights));
    else
        LSG_CUDA_TRY(launch_kernel(moe_route_kernel<32>, rg, rb, 0,
                               static_cast<cudaStream_t>(stream), true, logits, num_tokens, num_experts,
                               top_k, topk_idx, topk_weights));
    return LSG_OK;
}

extern "C" long long lsg_moe_permutation_scratch_ints(int num_tokens, int top_k, int num_experts) {
    if (num_tokens < 0 || top_k < 0 || num_experts < 1) return 0;
    const long long P = static_cast<long long>(num_tokens) * top_k;
    const long long n_chunks = P > 0 ? (P + kChunk - 1) / kChunk : 1;
    return n_chunks * num_experts;
}

extern "C" int lsg_moe_permutation(const int32_t* topk_idx, int num_tokens, int top_k, int num_experts,
                                   int32_t* expert_offsets, int32_t* perm, int32_t* inv_perm,
                                   int32_t* counts_scratch, void* stream) {
    if (num_experts < 1) return fail(LSG_ERR_INVALID, "moe_permutation: num_experts must be positive");
    if (!expert_offsets || !counts_scratch) return fail(LSG_ERR_INVALID, "moe_permutation: null pointer");
    const int P = num_tokens * top_k;
    if (P > 0 && (!topk_idx || !perm || !inv_perm)) return fail(LSG_ERR_INVALID, "moe_permutation: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (num_experts > 1024) return fail(LSG_ERR_INVALID, "moe_permutation: at most 1024 experts (E=%d)", num_experts);
    if (P > 0 && P <= 1024 && static_cast<long long>((P + 31) / 32) * num_experts <= 10240) {
        LSG_CUDA_TRY(launch_kernel(moe_permutation_small_kernel, dim3(1), dim3(1024),
                                   static_cast<size_t>((P + 31) / 32) * num_experts * sizeof(int), s, true, topk_idx,
                                   P, num_experts, expert_offsets, perm, inv_perm));
        return LSG_OK;
    }
    const int n_chunks = P > 0 ? (P + kChunk - 1) / kChunk : 1;
    LSG_CUDA_TRY(launch_kernel(moe_chunk_hist_kernel, dim3(n_chunks), dim3(kChunk), 0, s, true, topk_idx, P,
                               num_experts, counts_scratch));
    LSG_CUDA_TRY(launch_kernel(moe_chunk_scan_kernel, dim3(1), dim3(1024), 0, s, true, counts_scratch, n_chunks,
                               num_experts, expert_offsets));
    if (P > 0)
        LSG_CUDA_TRY(launch_kernel(moe_place_kernel, dim3(n_chunks), dim3(kChunk),
                                   static_cast<size_t>(kChunk / 32) * num_experts * sizeof(int), s, true, topk_idx,
                                   P, num_experts, static_cast<const int32_t*>(counts_scratch),
                                   static_cast<const int32_t*>(expert_offsets), perm, inv_perm));
    return LSG_OK;
}

extern "C" int lsg_moe_permute(const void* hidden_bf16, const int32_t* perm, int rows, int top_k, int H,
                               void* out_bf16, void* stream) {
    if (rows <= 0) return LSG_OK;
    if (!hidden_bf16 || !perm || !out_bf16) return fail(LSG_ERR_INVALID, "moe_permute: null pointer");
    if (H % 8 != 0 || (reinterpret_cast<uintptr_t>(hidden_bf16) & 15) || (reinterpret_cast<uintptr_t>(out_bf16) & 15))
        return fail(LSG_ERR_ALIGNMENT, "moe_permute: H must be a multiple of 8 and buffers 16-byte aligned");
    const int vpr = H / 8;
    const long long total = static_cast<long long>(rows) * vpr;
    LSG_CUDA_TRY(launch_kernel(moe_gather_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0,
                               static_cast<cudaStream_t>(stream), true, static_cast<const uint4*>(hidden_bf16),
                               perm, top_k, rows, vpr, static_cast<uint4*>(out_bf16)));
    return LSG_OK;
}

extern "C" int lsg_moe_unpermute(const void* y_bf16, const int32_t* inv_perm, const float* topk_weights,
                                 int num_tokens, int top_k, int H, void* out_bf16, void* stream) {
    if (num_tokens <= 0) return LSG_OK;
    if (!y_bf16 || !inv_perm || !topk_weights || !out_bf16) return fail(LSG_ERR_INVALID, "moe_unpermute: null pointer");
    if (H % 2 != 0) return fail(LSG_ERR_INVALID, "moe_unpermute: H must be even");
    if (H % 8 == 0 && top_k <= 8 && ((reinterpret_cast<uintptr_t>(y_bf16) | reinterpret_cast<uintptr_t>(out_bf16)) & 15) == 0) {
        const int vpr = H / 8;
        const int threads = vpr >= 256 ? 256 : ((vpr + 31) / 32) * 32;
        LSG_CUDA_TRY(launch_kernel(moe_combine_vec_kernel<8>, dim3(static_cast<unsigned>(num_tokens)), dim3(threads), 0,
                                   static_cast<cudaStream_t>(stream), true, static_cast<const uint4*>(y_bf16), inv_perm,
                                   topk_weights, top_k, vpr, static_cast<uint4*>(out_bf16)));
        return LSG_OK;
    }
    const long long total = static_cast<long long>(num_tokens) * (H / 2);
    LSG_CUDA_TRY(launch_kernel(moe_combine_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0,
                               static_cast<cudaStream_t>(stream), true, static_cast<const __nv_bfloat16*>(y_bf16),
                               inv_perm, topk_weights, num_tokens, top_k, H, static_cast<__nv_bfloat16*>(out_bf16)));
    return LSG_OK;
}

extern "C" int lsg_ep_expert_order(const int32_t* recv_counts, int world, int experts_per_rank, int rows,
                                   int32_t* local_offsets, int32_t* order, int32_t* inv_order,
                                   int32_t* scratch, void* stream) {
    const long long B = static_cast<long long>(world) * experts_per_rank;
    if (world < 1 || experts_per_rank < 1 || B > 1024)
        return fail(LSG_ERR_INVALID, "ep_expert_order: need 1 <= world * experts_per_rank <= 1024");
    if (rows < 0) return fail(LSG_ERR_INVALID, "ep_expert_order: negative row count");
    if (!recv_counts || !local_offsets || !scratch || (rows > 0 && (!order || !inv_order)))
        return fail(LSG_ERR_INVALID, "ep_expert_order: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int32_t* starts_recv = scratch;
    int32_t* starts_dst = scratch + B;
    LSG_CUDA_TRY(launch_kernel(ep_block_starts_kernel, dim3(1), dim3(1024), 0, s, true, recv_counts, world,
                               experts_per_rank, starts_recv, starts_dst, local_offsets));
    if (rows > 0)
        LSG_CUDA_TRY(launch_kernel(ep_order_kernel, dim3((rows + 255) / 256), dim3(256), 0, s, true, recv_counts,
                                   static_cast<const int32_t*>(starts_recv), static_cast<const int32_t*>(starts_dst),
                                   world, experts_per_rank, rows, order, inv_order));
    return LSG_OK;
}
