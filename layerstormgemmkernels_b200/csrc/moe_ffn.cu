// Expert feed-forward block of a SwiGLU MoE layer over rows already grouped by expert:
//   D = down( silu(gate(x)) * up(x) ),   silu(g) = g / (1 + exp(-g)),
// i.e. the three grouped GEMMs a caller of the reference issues through
// gguf_grouped_gemm (csrc/bindings_python.cu:552-611) with the activation in between,
// as ONE call.  The reference fuses the activation with the quantizer only on its NVFP4
// path (launch_silu_mul_to_nvfp4_grouped, csrc/smxx/quant/bf16_to_nvfp4_grouped.cu); this is
// the same idea for GGUF weights.  Numerics: gate and up outputs rounded to bf16, the
// activation computed in fp32 and rounded to bf16, then the usual Q8_1 activation
// quantization of the down projection - what the three separate calls produce.
//
// Two routes:
//   * tensor cores with the weights decoded inside the GEMM (tc_fused.cu): one activation
//     preparation, gate and up in one launch, SwiGLU fused into the preparation of the down
//     GEMM's operand, one tile map for both launches;
//   * otherwise (types without an in-kernel decoder, or few rows per expert) the three
//     grouped GEMMs of this library back to back with a SwiGLU kernel in between.
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "formats.cuh"
#include "host.h"

namespace lsg {

namespace {

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// act = bf16( silu(g) * u ), eight values per thread.
__global__ void __launch_bounds__(256)
silu_mul_bf16_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ out, long long n_vec) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= n_vec) return;
    const uint4 gr = __ldg(g + i), ur = __ldg(u + i);
    const uint32_t gw[4] = {gr.x, gr.y, gr.z, gr.w}, uw[4] = {ur.x, ur.y, ur.z, ur.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = silu_mul_bf16x2(gw[j], uw[j]);
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

// Average rows per expert up to which the block is composed from the grouped mat-vec kernels.
std::atomic<int>& matvec_rows() {
    static std::atomic<int> rows([] {
        const char* e = getenv("LSG_MOE_MATVEC_ROWS");
        return e ? atoi(e) : 8;
    }());
    return rows;
}

struct FfnLayout {
    size_t gather_off, gather_bytes;  // routed rows of the composed route when the call carries a permutation
    size_t map_off, map_bytes;      // tile map of the tensor-core route
    size_t fused_off, fused_bytes;  // scratch of the tensor-core route
    size_t g_off, u_off, act_off;   // bf16 [T, I] buffers of the composed route
    size_t grouped_off, grouped_bytes;
    size_t total;
};

FfnLayout ffn_layout(int T, int H, int I, int E) {
    FfnLayout l = {};
    const size_t t_max64 = static_cast<size_t>((T + 63) / 64 + E);
    l.map_off = 0;
    l.map_bytes = align256(2 * t_max64 * sizeof(int));
    l.fused_off = l.map_bytes;
    l.fused_bytes = tc_fused_moe_ffn_scratch_bytes(T, H, I);
    // composed route shares the space after the map
    const size_t ti = align256(static_cast<size_t>(T) * I * 2);
    l.g_off = l.map_bytes;
    l.u_off = l.g_off + ti;
    l.act_off = l.u_off + ti;
    l.grouped_off = l.act_off + ti;
    const size_t g1 = lsg_gguf_grouped_gemm_workspace_bytes_ex(T, H, E, I);
    const size_t g2 = lsg_gguf_grouped_gemm_workspace_bytes_ex(T, I, E, H);
    l.grouped_bytes = align256(g1 > g2 ? g1 : g2);
    // the composed route gathers the routed rows first (it serves decode-sized batches only,
    // so this is small); the tensor-core route reads the tokens through the permutation
    l.gather_off = l.grouped_off + l.grouped_bytes;
    l.gather_bytes = (T / E > 8) ? 0 : align256(static_cast<size_t>(T) * H * 2);
    const size_t composed = l.gather_off + l.gather_bytes;
    const size_t fused = l.fused_off + l.fused_bytes;
    l.total = composed > fused ? composed : fused;
    return l;
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" size_t lsg_gguf_moe_ffn_workspace_bytes(int total_tokens, int H, int I, int num_experts) {
    if (total_tokens <= 0 || H <= 0 || I <= 0 || num_experts <= 0) return 0;
    return ffn_layout(total_tokens, H, I, num_experts).total;
}

extern "C" int lsg_gguf_moe_ffn_set_matvec_rows(int rows) {
    return matvec_rows().exchange(rows, std::memory_order_relaxed);
}

extern "C" int lsg_gguf_moe_ffn(const lsg_gguf_moe_ffn_params* p, int total_tokens, void* workspace,
                                size_t workspace_bytes, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "gguf_moe_ffn: null params");
    const int qk = gguf_block_values(p->type);
    if (qk == 0) return fail(LSG_ERR_UNSUPPORTED, "gguf_moe_ffn: unknown GGUF type %d", p->type);
    if (p->out_dtype != LSG_DTYPE_BF16 && p->out_dtype != LSG_DTYPE_F32)
        return fail(LSG_ERR_UNSUPPORTED, "gguf_moe_ffn: out_dtype must be bf16 or f32");
    if (total_tokens < 0 || p->num_experts < 0 || p->H <= 0 || p->I <= 0)
        return fail(LSG_ERR_INVALID, "gguf_moe_ffn: negative or zero shape");
    if (total_tokens == 0 || p->num_experts == 0) return LSG_OK;
    if (p->H % qk != 0 || p->I % qk != 0 || p->H % 32 != 0 || p->I % 32 != 0)
        return fail(LSG_ERR_INVALID, "gguf_moe_ffn: H=%d and I=%d must be divisible by the block size %d (and by 32)",
                    p->H, p->I, qk);
    if (!p->A_base || !p->D_base || !p->expert_offsets || !p->gate_ptrs || !p->up_ptrs || !p->down_ptrs)
        return fail(LSG_ERR_INVALID, "gguf_moe_ffn: null A/D/expert_offsets/weight pointer arrays");
    if (p->perm && p->top_k < 1) return fail(LSG_ERR_INVALID, "gguf_moe_ffn: top_k must be >= 1 with a permutation");
    const int T = total_tokens, E = p->num_experts, H = p->H, I = p->I;
    const FfnLayout l = ffn_layout(T, H, I, E);
    if (!workspace || workspace_bytes < l.total)
        return fail(LSG_ERR_WORKSPACE, "gguf_moe_ffn: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), l.total);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(LSG_ERR_ALIGNMENT, "gguf_moe_ffn: workspace must be 256-byte aligned");
    uint8_t* base = static_cast<uint8_t*>(workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int32_t* offs = static_cast<const int32_t*>(p->expert_offsets);

    // the reference's rule for leaving the mat-vec kernels: more than 8 rows per expert on average
    // (lsg_gguf_moe_ffn_set_matvec_rows moves the threshold)
    if (tc_fused_available(p->type) && T / E > matvec_rows().load(std::memory_order_relaxed)) {
        const int tile_m = tc_fused_grouped_tile_m(T, E);
        const int t_max = (T + tile_m - 1) / tile_m + E;
        int* tile_expert = reinterpret_cast<int*>(base + l.map_off);
        int* tile_mstart = tile_expert + t_max;
        int rc = build_mmq_tile_map(offs, E, tile_m, t_max, tile_expert, tile_mstart, s, T, true);
        if (rc != LSG_OK) return rc;
        return tc_fused_moe_ffn(p->type, T, E, H, I, p->A_base, p->gate_ptrs, p->up_ptrs, p->down_ptrs, offs,
                                p->D_base, p->out_dtype, tile_expert, tile_mstart, t_max, tile_m,
                                base + l.fused_off, l.fused_bytes, s, p->perm, p->perm ? p->top_k : 1);
    }

    lsg_gguf_grouped_gemm_params g = {};
    g.type = p->type; g.strategy = LSG_GGUF_STRATEGY_INT; g.num_experts = E;
    g.N = I; g.K = H; g.expert_offsets = offs; g.out_dtype = LSG_DTYPE_BF16;
    uint8_t* gws = base + l.grouped_off;

    // Few rows per expert (the reference's rule): every projection takes the grouped mat-vec,
    // and at these sizes the launches are the cost.  The routed rows are quantized straight
    // from the token matrix through the permutation (no gathered copy), up reads the Q8_1
    // blocks and the segment list gate's call left in the workspace, and the activation is
    // formed inside the quantizer of the down projection (no bf16 activation buffer): eight
    // launches instead of twelve, same bits.
    if (T / E <= 8 && H % 8 == 0 && I % 8 == 0 && (reinterpret_cast<uintptr_t>(p->A_base) & 15) == 0) {
        int rc = p->perm ? quantize_q8_1_gather(p->A_base, p->perm, p->top_k, gws, T, H, s, true)
                         : quantize_q8_1(p->A_base, gws, T, H, s, true);
        if (rc != LSG_OK) return rc;
        g.A_base = nullptr;
        g.D_base = base + l.g_off; g.B_ptrs = p->gate_ptrs;
        rc = grouped_gemm_matvec(&g, T, gws, l.grouped_bytes, s, true, false);
        if (rc != LSG_OK) return rc;
        g.D_base = base + l.u_off; g.B_ptrs = p->up_ptrs;
        rc = grouped_gemm_matvec(&g, T, gws, l.grouped_bytes, s, true, true);
        if (rc != LSG_OK) return rc;
        rc = quantize_q8_1_silu_mul(base + l.g_off, base + l.u_off, gws, T, I, s, true);
        if (rc != LSG_OK) return rc;
        g.N = H; g.K = I; g.D_base = p->D_base; g.B_ptrs = p->down_ptrs; g.out_dtype = p->out_dtype;
        return grouped_gemm_matvec(&g, T, gws, l.grouped_bytes, s, true, false);
    }

    const void* rows = p->A_base;
    if (p->perm) {
        if (l.gather_bytes == 0)
            return fail(LSG_ERR_UNSUPPORTED,
                        "gguf_moe_ffn: a permutation with this type and batch needs the rows gathered by the caller "
                        "(lsg_moe_permute)");
        int rc = lsg_moe_permute(p->A_base, p->perm, T, p->top_k, H, base + l.gather_off, stream);
        if (rc != LSG_OK) return rc;
        rows = base + l.gather_off;
    }
    g.A_base = rows;
    g.D_base = base + l.g_off; g.B_ptrs = p->gate_ptrs;
    int rc = lsg_gguf_grouped_gemm(&g, T, gws, l.grouped_bytes, LSG_GGUF_FORCE_AUTO, stream);
    if (rc != LSG_OK) return rc;
    g.D_base = base + l.u_off; g.B_ptrs = p->up_ptrs;
    rc = lsg_gguf_grouped_gemm(&g, T, gws, l.grouped_bytes, LSG_GGUF_FORCE_AUTO, stream);
    if (rc != LSG_OK) return rc;
    const long long n_vec = static_cast<long long>(T) * I / 8;
    LSG_CUDA_TRY(launch_kernel(silu_mul_bf16_kernel, dim3(static_cast<unsigned>((n_vec + 255) / 256)), dim3(256), 0, s,
                               true, reinterpret_cast<const uint4*>(base + l.g_off),
                               reinterpret_cast<const uint4*>(base + l.u_off),
                               reinterpret_cast<uint4*>(base + l.act_off), n_vec));
    g.N = H; g.K = I; g.A_base = base + l.act_off; g.D_base = p->D_base; g.B_ptrs = p->down_ptrs;
    g.out_dtype = p->out_dtype;
    return lsg_gguf_grouped_gemm(&g, T, gws, l.grouped_bytes, LSG_GGUF_FORCE_AUTO, stream);
}
