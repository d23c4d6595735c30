// GGUF grouped GEMM (one MoE projection over E experts; rows already permuted by expert).
// Host side: validation, workspace carving, strategy / force routing.
//
// Replaces gguf_grouped_gemm_workspace_bytes, launch_gguf_grouped_gemm,
// launch_gguf_grouped_gemm_int_forced, launch_gguf_grouped_gemm_hostloop
// (csrc/sm120/gemm/gguf/gguf_grouped_gemm.cu:28-150) and launch_gguf_grouped_int
// (gguf_grouped_int.cu:925-995) with the same routing rules:
//   strategy Dequant, or force = hostloop  -> per-expert host loop (one D2H copy + sync)
//   strategy Int, force auto/mmvq/mmq      -> device-routed, no host sync, capturable
//   auto picks the tensor-core path when total_tokens / num_experts > 8.
#include "mmvq_grouped.cuh"
#include "host.h"

#include <vector>

namespace lsg {

namespace {

struct WsLayout {
    size_t q8_bytes, active_off, seg_off, tile_off, total;
    int cap, max_segments, tmax64;
};

// Workspace: [Q8_1 of all rows][active list: cap ints][segment list: 1 + 3*max_segments ints]
//            [m-tile map: 2 * T_max(64) ints]
WsLayout ws_layout(int T, int K, int E) {
    WsLayout w = {};
    w.q8_bytes = static_cast<size_t>(T) * (K / 32) * kQ8_1Bytes;
    w.cap = E < T ? E : T;
    w.max_segments = E + T;  // one segment per expert plus one per extra image-full of rows
    w.tmax64 = (T + 63) / 64 + (E > 0 ? E : 0);
    w.active_off = (w.q8_bytes + 15) & ~size_t(15);
    w.seg_off = w.active_off + ((static_cast<size_t>(w.cap) * 4 + 15) & ~size_t(15));
    w.tile_off = w.seg_off + ((static_cast<size_t>(1 + 3 * w.max_segments) * 4 + 15) & ~size_t(15));
    w.total = (w.tile_off + 2ull * w.tmax64 * 4 + 255) & ~size_t(255);
    return w;
}

int grouped_dispatch(int type, const GroupedArgs& a, const MmvqTune& tn, int max_segments,
                     cudaStream_t s) {
    switch (type) {
        case 0: return mmvq_grouped_launch_t0(a, tn, max_segments, s, true);
        case 1: return mmvq_grouped_launch_t1(a, tn, max_segments, s, true);
        case 2: return mmvq_grouped_launch_t2(a, tn, max_segments, s, true);
        case 3: return mmvq_grouped_launch_t3(a, tn, max_segments, s, true);
        case 4: return mmvq_grouped_launch_t4(a, tn, max_segments, s, true);
        case 5: return mmvq_grouped_launch_t5(a, tn, max_segments, s, true);
        case 6: return mmvq_grouped_launch_t6(a, tn, max_segments, s, true);
        case 7: return mmvq_grouped_launch_t7(a, tn, max_segments, s, true);
    }
    return fail(LSG_ERR_UNSUPPORTED, "gguf_grouped_gemm: unknown type %d", type);
}

int grouped_max_rows(int type, int K, const MmvqTune& tn) {
    switch (type) {
        case 0: return mmvq_grouped_max_rows_t0(K, tn);
        case 1: return mmvq_grouped_max_rows_t1(K, tn);
        case 2: return mmvq_grouped_max_rows_t2(K, tn);
        case 3: return mmvq_grouped_max_rows_t3(K, tn);
        case 4: return mmvq_grouped_max_rows_t4(K, tn);
        case 5: return mmvq_grouped_max_rows_t5(K, tn);
        case 6: return mmvq_grouped_max_rows_t6(K, tn);
        case 7: return mmvq_grouped_max_rows_t7(K, tn);
    }
    return 1;
}

int check_common(const lsg_gguf_grouped_gemm_params* p) {
    if (!p) return fail(LSG_ERR_INVALID, "gguf_grouped_gemm: null params");
    const int qk = gguf_block_values(p->type);
    if (qk == 0) return fail(LSG_ERR_UNSUPPORTED, "gguf_grouped_gemm: unknown GGUF type %d", p->type);
    if (p->out_dtype != LSG_DTYPE_BF16 && p->out_dtype != LSG_DTYPE_F32)
        return fail(LSG_ERR_UNSUPPORTED, "gguf_grouped_gemm: out_dtype must be bf16 or f32");
    return LSG_OK;
}

// The grouped mat-vec over a device-built segment list: activations quantized into the
// workspace (skipped when `xq_ready`: the caller, or the call in front with the same A_base, K
// and workspace, left them there) and segments built from the offsets (skipped when
// `seg_ready`: the call in front had the same offsets and K and skipped the same experts - the
// caller guarantees that an expert has a weight here when it had one there), then one launch.
int grouped_matvec_tail(const lsg_gguf_grouped_gemm_params* p, int T, uint8_t* base, const WsLayout& w,
                        cudaStream_t s, bool xq_ready, bool seg_ready) {
    int rc = LSG_OK;
    if (!xq_ready) {
        rc = quantize_q8_1(p->A_base, base, T, p->K, s, true);
        if (rc != LSG_OK) return rc;
    }
    int* seg = reinterpret_cast<int*>(base + w.seg_off);
    const MmvqTune tn = mmvq_tuning();
    const int max_rows = grouped_max_rows(p->type, p->K, tn);
    if (!seg_ready) {
        rc = build_segment_list(static_cast<const int32_t*>(p->expert_offsets), p->B_ptrs, p->num_experts,
                                max_rows, w.max_segments, seg, s, T);
        if (rc != LSG_OK) return rc;
    }
    GroupedArgs a = {};
    a.xq = base;
    a.B_ptrs = p->B_ptrs;
    a.seg = seg;
    a.D = p->D_base;
    a.status = device_status_word();
    a.N = p->N;
    a.K = p->K;
    a.out_f32 = p->out_dtype == LSG_DTYPE_F32;
    // upper bound of live segments: each expert contributes ceil(M_e / max_rows) <= 1 + M_e / max_rows
    long long bound = static_cast<long long>(p->num_experts < T ? p->num_experts : T) + T / max_rows;
    if (bound > w.max_segments) bound = w.max_segments;
    return grouped_dispatch(p->type, a, tn, static_cast<int>(bound), s);
}

// Device-routed integer path.
int grouped_int(const lsg_gguf_grouped_gemm_params* p, int T, void* ws, size_t ws_bytes, int force,
                cudaStream_t s) {
    if (p->num_experts <= 0 || T <= 0) return LSG_OK;  // nothing to do, as the reference
    if (p->K % 32 != 0 || p->K % gguf_block_values(p->type) != 0)
        return fail(LSG_ERR_INVALID, "GGUF grouped int: K must be divisible by %d", gguf_block_values(p->type));
    if (!ws) return fail(LSG_ERR_WORKSPACE, "GGUF grouped int: workspace required");
    if (!p->A_base || !p->D_base || !p->expert_offsets || !p->B_ptrs)
        return fail(LSG_ERR_INVALID, "GGUF grouped GEMM: null A/D/expert_offsets/B_ptrs");
    const WsLayout w = ws_layout(T, p->K, p->num_experts);
    if (ws_bytes < w.total)
        return fail(LSG_ERR_WORKSPACE, "GGUF grouped int: workspace too small (have %zu, need %zu)",
                    ws_bytes, w.total);
    uint8_t* base = static_cast<uint8_t*>(ws);
    int rc = LSG_OK;

    // As the reference (gguf_grouped_int.cu:947-950): tensor cores when there are more
    // than 8 rows per expert on average, unless forced either way.  The tensor-core path
    // needs the larger workspace of lsg_gguf_grouped_gemm_workspace_bytes_ex; without it
    // the grouped mat-vec kernel, which is correct for any rows-per-expert, does the work.
    bool use_mmq = (T / p->num_experts) > 8;
    if (force == LSG_GGUF_FORCE_MMVQ) use_mmq = false;
    if (force == LSG_GGUF_FORCE_MMQ) use_mmq = true;
    int* tile_expert = reinterpret_cast<int*>(base + w.tile_off);
    // Preferred: weights decoded inside the GEMM (needs only the fp16 activations as scratch).
    if (use_mmq && tc_fused_available(p->type) &&
        ws_bytes >= w.total + tc_fused_grouped_scratch_bytes(T, p->num_experts, p->N, p->K)) {
        const int tile_m = tc_fused_grouped_tile_m(T, p->num_experts);   // 64, 128 or 256
        const int t_max = (T + tile_m - 1) / tile_m + p->num_experts;
        int* tile_mstart = tile_expert + t_max;  // t_max(tile_m >= 64) <= t_max(64): fits the reserved map
        rc = build_mmq_tile_map(static_cast<const int32_t*>(p->expert_offsets), p->num_experts, tile_m,
                                t_max, tile_expert, tile_mstart, s, T, true);
        if (rc != LSG_OK) return rc;
        return tc_fused_grouped(p->type, T, p->num_experts, p->N, p->K, p->A_base, p->B_ptrs,
                                static_cast<const int32_t*>(p->expert_offsets), p->D_base, p->out_dtype,
                                tile_expert, tile_mstart, t_max, tile_m, base + w.total, ws_bytes - w.total, s);
    }
    const size_t mmq_need = mmq_scratch_bytes(T, p->K, p->num_experts, p->N);
    if (use_mmq && ws_bytes >= w.total + mmq_need && (p->K % 8) == 0) {
        const int tile_m = 128;
        const int t_max = (T + tile_m - 1) / tile_m + p->num_experts;
        int* tile_mstart = tile_expert + t_max;  // t_max(128) <= t_max(64): fits the reserved map
        rc = build_mmq_tile_map(static_cast<const int32_t*>(p->expert_offsets), p->num_experts, tile_m,
                                t_max, tile_expert, tile_mstart, s, T);
        if (rc != LSG_OK) return rc;
        return mmq_grouped(p->type, T, p->num_experts, p->N, p->K, p->A_base, p->B_ptrs,
                           static_cast<const int32_t*>(p->expert_offsets), p->D_base,
                           p->out_dtype == LSG_DTYPE_F32, tile_expert, tile_mstart, t_max,
                           base + w.total, ws_bytes - w.total, s);
    }
    return grouped_matvec_tail(p, T, base, w, s, false, false);
}

// Host per-expert loop: the golden of both strategies and the Dequant implementation.
int grouped_hostloop(const lsg_gguf_grouped_gemm_params* p, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (p->num_experts <= 0) return LSG_OK;
    if (!p->B_ptrs)
        return fail(LSG_ERR_INVALID, "GGUF grouped GEMM: B_ptrs required (scattered per-expert blocks)");
    if (!p->A_base || !p->D_base || !p->expert_offsets)
        return fail(LSG_ERR_INVALID, "GGUF grouped GEMM: null A/D/expert_offsets");
    const int qk = gguf_block_values(p->type);
    if (p->K % qk != 0)
        return fail(LSG_ERR_INVALID, "GGUF grouped GEMM: K=%d must be divisible by the block size %d",
                    p->K, qk);
    const int E = p->num_experts;
    std::vector<int32_t> offs(E + 1);
    std::vector<const void*> ptrs(E);
    LSG_CUDA_TRY(cudaMemcpyAsync(offs.data(), p->expert_offsets, (E + 1) * sizeof(int32_t),
                                 cudaMemcpyDeviceToHost, s));
    LSG_CUDA_TRY(cudaMemcpyAsync(ptrs.data(), p->B_ptrs, E * sizeof(void*), cudaMemcpyDeviceToHost, s));
    LSG_CUDA_TRY(cudaStreamSynchronize(s));
    const size_t out_elem = p->out_dtype == LSG_DTYPE_F32 ? 4 : 2;
    for (int e = 0; e < E; ++e) {
        const int off = offs[e], M_e = offs[e + 1] - off;
        if (M_e <= 0 || ptrs[e] == nullptr) continue;
        const uint8_t* A_e = static_cast<const uint8_t*>(p->A_base) + static_cast<size_t>(off) * p->K * 2;
        uint8_t* D_e = static_cast<uint8_t*>(p->D_base) + static_cast<size_t>(off) * p->N * out_elem;
        int rc;
        if (p->strategy == LSG_GGUF_STRATEGY_DEQUANT) {
            rc = dequant_gemm(p->type, M_e, p->N, p->K, A_e, ptrs[e], D_e, p->N,
                              p->out_dtype == LSG_DTYPE_F32, s);
        } else {
            const size_t need = static_cast<size_t>(M_e) * (p->K / 32) * kQ8_1Bytes;
            if (!ws || ws_bytes < need)
                return fail(LSG_ERR_WORKSPACE,
                            "GGUF grouped GEMM (Int): workspace too small (have %zu, need %zu)",
                            ws ? ws_bytes : size_t(0), need);
            rc = quantize_q8_1(A_e, ws, M_e, p->K, s, false);
            if (rc == LSG_OK)
                rc = mmvq_q8_1(p->type, M_e, p->N, p->K, ptrs[e], ws, D_e, p->N,
                               p->out_dtype == LSG_DTYPE_F32, s, false);
        }
        if (rc != LSG_OK) return rc;
    }
    return LSG_OK;
}

}  // namespace

// The mat-vec route of lsg_gguf_grouped_gemm for a caller inside the library that runs several
// projections of the same rows through the same workspace (gate and up of an expert block):
// `xq_ready` skips the activation quantizer (the Q8_1 blocks of all T rows are at the start of
// the workspace already) and `seg_ready` the segment list (every expert with rows has all its
// weights: lsg_gguf_moe_ffn's contract).  A_base may be null with `xq_ready`.
int grouped_gemm_matvec(const lsg_gguf_grouped_gemm_params* p, int T, void* ws, size_t ws_bytes, cudaStream_t s,
                        bool xq_ready, bool seg_ready) {
    int rc = check_common(p);
    if (rc != LSG_OK) return rc;
    if (p->num_experts <= 0 || T <= 0) return LSG_OK;
    if (p->K % 32 != 0 || p->K % gguf_block_values(p->type) != 0)
        return fail(LSG_ERR_INVALID, "GGUF grouped int: K must be divisible by %d", gguf_block_values(p->type));
    if (!ws) return fail(LSG_ERR_WORKSPACE, "GGUF grouped int: workspace required");
    if ((!p->A_base && !xq_ready) || !p->D_base || !p->expert_offsets || !p->B_ptrs)
        return fail(LSG_ERR_INVALID, "GGUF grouped GEMM: null A/D/expert_offsets/B_ptrs");
    const WsLayout w = ws_layout(T, p->K, p->num_experts);
    if (ws_bytes < w.total)
        return fail(LSG_ERR_WORKSPACE, "GGUF grouped int: workspace too small (have %zu, need %zu)", ws_bytes, w.total);
    return grouped_matvec_tail(p, T, static_cast<uint8_t*>(ws), w, s, xq_ready, seg_ready);
}

}  // namespace lsg

using namespace lsg;

extern "C" size_t lsg_gguf_grouped_gemm_workspace_bytes(int total_tokens, int K, int num_experts) {
    if (total_tokens <= 0 || K <= 0) return 0;
    return ws_layout(total_tokens, K, num_experts < 0 ? 0 : num_experts).total;
}

extern "C" size_t lsg_gguf_grouped_gemm_workspace_bytes_ex(int total_tokens, int K, int num_experts,
                                                           int N) {
    if (total_tokens <= 0 || K <= 0) return 0;
    const int E = num_experts < 0 ? 0 : num_experts;
    return ws_layout(total_tokens, K, E).total + mmq_scratch_bytes(total_tokens, K, E, N < 0 ? 0 : N);
}

extern "C" int lsg_gguf_grouped_gemm(const lsg_gguf_grouped_gemm_params* p, int total_tokens,
                                     void* workspace, size_t workspace_bytes, int force, void* stream) {
    int rc = check_common(p);
    if (rc != LSG_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (force < 0 || force > 3) return fail(LSG_ERR_INVALID, "gguf_grouped_gemm: force must be 0..3");
    if (p->strategy == LSG_GGUF_STRATEGY_DEQUANT || force == LSG_GGUF_FORCE_HOSTLOOP)
        return grouped_hostloop(p, workspace, workspace_bytes, s);
    if (p->strategy != LSG_GGUF_STRATEGY_INT)
        return fail(LSG_ERR_INVALID, "gguf_grouped_gemm: strategy must be 0 (Dequant) or 1 (Int)");
    return grouped_int(p, total_tokens, workspace, workspace_bytes, force, s);
}
