// Host side of the GGUF mmvq path: argument checks, activation quantization,
// per-type dispatch.  Replaces launch_gguf_mmvq of the reference
// (csrc/sm120/gemm/gguf/gguf_mmvq.cu:130-152).
#include "mmvq.cuh"
#include "host.h"

namespace lsg {

namespace {

int dispatch_launch(int type, const MmvqArgs& a, cudaStream_t s, bool pdl) {
    switch (type) {
        case 0: return mmvq_launch_t0(a, s, pdl);
        case 1: return mmvq_launch_t1(a, s, pdl);
        case 2: return mmvq_launch_t2(a, s, pdl);
        case 3: return mmvq_launch_t3(a, s, pdl);
        case 4: return mmvq_launch_t4(a, s, pdl);
        case 5: return mmvq_launch_t5(a, s, pdl);
        case 6: return mmvq_launch_t6(a, s, pdl);
        case 7: return mmvq_launch_t7(a, s, pdl);
    }
    return fail(LSG_ERR_UNSUPPORTED, "gguf_mmvq: unknown type %d", type);
}

int dispatch_max_rows(int type, int K) {
    switch (type) {
        case 0: return mmvq_max_rows_t0(K);
        case 1: return mmvq_max_rows_t1(K);
        case 2: return mmvq_max_rows_t2(K);
        case 3: return mmvq_max_rows_t3(K);
        case 4: return mmvq_max_rows_t4(K);
        case 5: return mmvq_max_rows_t5(K);
        case 6: return mmvq_max_rows_t6(K);
        case 7: return mmvq_max_rows_t7(K);
    }
    return 0;
}

}  // namespace

int check_gemm_params(const char* op, const lsg_gguf_mmvq_params* p) {
    if (!p) return fail(LSG_ERR_INVALID, "%s: null params", op);
    const int qk = gguf_block_values(p->type);
    if (qk == 0) return fail(LSG_ERR_UNSUPPORTED, "%s: unknown GGUF type %d", op, p->type);
    if (p->M < 0 || p->N < 0 || p->K < 0) return fail(LSG_ERR_INVALID, "%s: negative shape", op);
    if (p->K % qk != 0)
        return fail(LSG_ERR_INVALID, "%s: K must be divisible by %d, got K=%d", op, qk, p->K);
    if (p->out_dtype != LSG_DTYPE_BF16 && p->out_dtype != LSG_DTYPE_F32)
        return fail(LSG_ERR_UNSUPPORTED, "%s: out_dtype must be bf16 or f32", op);
    return LSG_OK;
}

// xq: Q8_1 blocks of all M rows.  ldc: output row stride.  Rows are processed
// in batches that fit the shared-memory activation image.
int mmvq_q8_1(int type, int M, int N, int K, const void* W, const void* xq, void* C, int ldc,
              int out_f32, cudaStream_t stream, bool pdl) {
    if (M == 0 || N == 0) return LSG_OK;
    if (K == 0) return fail(LSG_ERR_INVALID, "gguf_mmvq: K must be positive");
    if (!W || !xq || !C) return fail(LSG_ERR_INVALID, "gguf_mmvq: null pointer");
    if (reinterpret_cast<uintptr_t>(W) & 15)
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmvq: packed weight must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(xq) & 3)
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmvq: Q8_1 buffer must be 4-byte aligned");
    const int max_rows = dispatch_max_rows(type, K);
    if (max_rows < 1)
        return fail(LSG_ERR_UNSUPPORTED, "gguf_mmvq: K=%d too large for the shared-memory pipeline", K);
    // Eight rows per register pass; keep batches a multiple of eight when possible.
    int batch = max_rows >= 8 ? (max_rows / 8) * 8 : max_rows;
    if (batch > 32) batch = 32;
    const size_t xq_row = static_cast<size_t>(K / 32) * kQ8_1Bytes;
    const size_t c_elem = out_f32 ? 4 : 2;
    for (int m0 = 0; m0 < M; m0 += batch) {
        MmvqArgs a = {};
        a.W = static_cast<const uint8_t*>(W);
        a.xq = static_cast<const uint8_t*>(xq) + static_cast<size_t>(m0) * xq_row;
        a.C = static_cast<uint8_t*>(C) + static_cast<size_t>(m0) * ldc * c_elem;
        a.status = device_status_word();
        a.M = (M - m0) < batch ? (M - m0) : batch;
        a.N = N;
        a.K = K;
        a.ldc = ldc;
        a.out_f32 = out_f32;
        const int rc = dispatch_launch(type, a, stream, pdl && m0 == 0);
        if (rc != LSG_OK) return rc;
    }
    return LSG_OK;
}

}  // namespace lsg

using namespace lsg;

extern "C" size_t lsg_gguf_mmvq_workspace_bytes(int M, int K) {
    if (M <= 0 || K <= 0) return 0;
    return static_cast<size_t>(M) * (K / 32) * kQ8_1Bytes;
}

extern "C" int lsg_gguf_mmvq_q8_1(const lsg_gguf_mmvq_params* p, const void* xq, void* stream) {
    int rc = check_gemm_params("gguf_mmvq", p);
    if (rc != LSG_OK) return rc;
    return mmvq_q8_1(p->type, p->M, p->N, p->K, p->B, xq, p->C, p->N,
                     p->out_dtype == LSG_DTYPE_F32, static_cast<cudaStream_t>(stream), false);
}

extern "C" int lsg_gguf_mmvq(const lsg_gguf_mmvq_params* p, void* workspace,
                             size_t workspace_bytes, void* stream) {
    int rc = check_gemm_params("gguf_mmvq", p);
    if (rc != LSG_OK) return rc;
    if (p->M == 0 || p->N == 0) return LSG_OK;
    const size_t need = lsg_gguf_mmvq_workspace_bytes(p->M, p->K);
    if (!workspace || workspace_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "gguf_mmvq: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = quantize_q8_1(p->A, workspace, p->M, p->K, s, true);
    if (rc != LSG_OK) return rc;
    return mmvq_q8_1(p->type, p->M, p->N, p->K, p->B, workspace, p->C, p->N,
                     p->out_dtype == LSG_DTYPE_F32, s, true);
}
