// Host side of the GGUF mmvq path: argument checks, activation quantization,
// per-type dispatch.  Replaces launch_gguf_mmvq of the reference
// (csrc/sm120/gemm/gguf/gguf_mmvq.cu:130-152).
#include "mmvq.cuh"
#include "host.h"

#include <stdlib.h>

namespace lsg {

namespace {

// Process-wide launch geometry.  Defaults suit decode on a 148-SM B200; the
// environment (LSG_MMVQ_WARPS / _CTAS / _STAGE_KB / _SHARE) or lsg_mmvq_set_tuning
// override them.
MmvqTune& tuning() {
    static MmvqTune t = [] {
        MmvqTune v{15, 1, 24, 1, 0};
        if (const char* e = getenv("LSG_MMVQ_WARPS")) v.warps = atoi(e);
        if (const char* e = getenv("LSG_MMVQ_CTAS")) v.ctas = atoi(e);
        if (const char* e = getenv("LSG_MMVQ_STAGE_KB")) v.stage_kb = atoi(e);
        if (const char* e = getenv("LSG_MMVQ_SHARE")) v.share = atoi(e);
#ifdef LSG_DEBUG_KNOBS
        if (getenv("LSG_MMVQ_SKIP")) v.skip_math = 1;
#endif
        return v;
    }();
    return t;
}

MmvqTune sane_tuning() {
    MmvqTune v = tuning();
    v.warps = v.warps < 1 ? 1 : (v.warps > 15 ? 15 : v.warps);
    v.ctas = v.ctas < 1 ? 1 : (v.ctas > 8 ? 8 : v.ctas);
    v.share = v.share < 1 ? 1 : (v.share > 8 ? 8 : v.share);
    v.stage_kb = v.stage_kb < 1 ? 1 : (v.stage_kb > 96 ? 96 : v.stage_kb);
    return v;
}

int g_drop_slab = -1;   // failure-path test hook (lsg_test_mmvq_drop_slab)
#ifdef LSG_MMVQ_TRACE
unsigned long long* g_trace = nullptr;
int g_trace_launch = 0, g_trace_slots = 0;
#endif

int dispatch_launch(int type, const MmvqArgs& a_in, cudaStream_t s, bool pdl) {
    const MmvqTune tn = sane_tuning();
    MmvqArgs a = a_in;
    a.wait_limit = wait_limit_cycles();
    a.drop_slab = g_drop_slab;
#ifdef LSG_MMVQ_TRACE
    a.trace = g_trace && g_trace_slots > 0 ? g_trace + static_cast<size_t>(g_trace_launch++ % g_trace_slots) * 1024 * 16 : nullptr;
#endif
    switch (type) {
        case 0: return mmvq_launch_t0(a, tn, s, pdl);
        case 1: return mmvq_launch_t1(a, tn, s, pdl);
        case 2: return mmvq_launch_t2(a, tn, s, pdl);
        case 3: return mmvq_launch_t3(a, tn, s, pdl);
        case 4: return mmvq_launch_t4(a, tn, s, pdl);
        case 5: return mmvq_launch_t5(a, tn, s, pdl);
        case 6: return mmvq_launch_t6(a, tn, s, pdl);
        case 7: return mmvq_launch_t7(a, tn, s, pdl);
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

MmvqTune mmvq_tuning() { return sane_tuning(); }

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
              int out_f32, cudaStream_t stream, bool pdl, const void* A_bf16, int dep_mode) {
    if (M == 0 || N == 0) return LSG_OK;
    if (K == 0) return fail(LSG_ERR_INVALID, "gguf_mmvq: K must be positive");
    if (!W || (!xq && !A_bf16) || !C) return fail(LSG_ERR_INVALID, "gguf_mmvq: null pointer");
    if (reinterpret_cast<uintptr_t>(W) & 15)
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmvq: packed weight must be 16-byte aligned");
    if (!A_bf16 && (reinterpret_cast<uintptr_t>(xq) & 3))
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
        a.xq = xq ? static_cast<const uint8_t*>(xq) + static_cast<size_t>(m0) * xq_row : nullptr;
        a.A = A_bf16 ? static_cast<const __nv_bfloat16*>(A_bf16) + static_cast<size_t>(m0) * K : nullptr;
        a.C = static_cast<uint8_t*>(C) + static_cast<size_t>(m0) * ldc * c_elem;
        a.status = device_status_word();
        a.M = (M - m0) < batch ? (M - m0) : batch;
        a.N = N;
        a.K = K;
        a.ldc = ldc;
        a.out_f32 = out_f32;
        a.dep_mode = (pdl && m0 == 0) ? dep_mode : 0;   // later row batches are fully serialized launches
        const int rc = dispatch_launch(type, a, stream, pdl && m0 == 0);
        if (rc != LSG_OK) return rc;
    }
    return LSG_OK;
}

// The same activations against n <= 4 weight matrices of one type and K, as one launch
// per batch of rows.  Matrix j writes C[j], [M][N[j]] row-major.
int mmvq_q8_1_joined(int type, int M, int K, int n, const void* const* W, void* const* C, const int* N,
                     const void* xq, int out_f32, cudaStream_t stream, bool pdl, const void* A_bf16, int dep_mode = 0,
                     const void* const* A_each = nullptr, const void* const* xq_each = nullptr) {
    if (n < 1 || n > 1 + kMmvqMaxExtra) return fail(LSG_ERR_INVALID, "gguf_mmvq: 1..6 matrices per joined launch");
    if (n == 1) return mmvq_q8_1(type, M, N[0], K, W[0], xq, C[0], N[0], out_f32, stream, pdl, A_bf16, dep_mode);
    if (M == 0) return LSG_OK;
    if (K == 0) return fail(LSG_ERR_INVALID, "gguf_mmvq: K must be positive");
    if (!xq && !A_bf16) return fail(LSG_ERR_INVALID, "gguf_mmvq: null pointer");
    for (int j = 0; j < n; ++j) {
        if (N[j] < 1) return fail(LSG_ERR_INVALID, "gguf_mmvq: joined matrices need N >= 1");
        if (!W[j] || !C[j]) return fail(LSG_ERR_INVALID, "gguf_mmvq: null pointer");
        if (reinterpret_cast<uintptr_t>(W[j]) & 15)
            return fail(LSG_ERR_ALIGNMENT, "gguf_mmvq: packed weight must be 16-byte aligned");
    }
    if (!A_bf16 && (reinterpret_cast<uintptr_t>(xq) & 3))
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmvq: Q8_1 buffer must be 4-byte aligned");
    const int max_rows = dispatch_max_rows(type, K);
    if (max_rows < 1)
        return fail(LSG_ERR_UNSUPPORTED, "gguf_mmvq: K=%d too large for the shared-memory pipeline", K);
    int batch = max_rows >= 8 ? (max_rows / 8) * 8 : max_rows;
    if (batch > 32) batch = 32;
    const size_t xq_row = static_cast<size_t>(K / 32) * kQ8_1Bytes;
    const size_t c_elem = out_f32 ? 4 : 2;
    for (int m0 = 0; m0 < M; m0 += batch) {
        MmvqArgs a = {};
        a.W = static_cast<const uint8_t*>(W[0]);
        a.xq = xq ? static_cast<const uint8_t*>(xq) + static_cast<size_t>(m0) * xq_row : nullptr;
        a.A = A_bf16 ? static_cast<const __nv_bfloat16*>(A_bf16) + static_cast<size_t>(m0) * K : nullptr;
        a.C = static_cast<uint8_t*>(C[0]) + static_cast<size_t>(m0) * N[0] * c_elem;
        a.status = device_status_word();
        a.M = (M - m0) < batch ? (M - m0) : batch;
        a.N = N[0];
        a.K = K;
        a.ldc = N[0];
        a.out_f32 = out_f32;
        a.n_extra = n - 1;
        for (int j = 1; j < n; ++j) {
            a.Wx[j - 1] = static_cast<const uint8_t*>(W[j]);
            a.Cx[j - 1] = static_cast<uint8_t*>(C[j]) + static_cast<size_t>(m0) * N[j] * c_elem;
            a.Nx[j - 1] = N[j];
            if (A_bf16)
                a.Ax[j - 1] = static_cast<const __nv_bfloat16*>(A_each && A_each[j] ? A_each[j] : A_bf16) + static_cast<size_t>(m0) * K;
            else
                a.xqx[j - 1] = static_cast<const uint8_t*>(xq_each && xq_each[j] ? xq_each[j] : xq) + static_cast<size_t>(m0) * xq_row;
        }
        a.dep_mode = (pdl && m0 == 0) ? dep_mode : 0;
        const int rc = dispatch_launch(type, a, stream, pdl && m0 == 0);
        if (rc != LSG_OK) return rc;
    }
    return LSG_OK;
}

bool fused_quant_ok(int M, int K, const void* A) {
    static const long long limit = [] {
        const char* e = getenv("LSG_MMVQ_FUSED_QUANT_MAX");
        return e ? atoll(e) : 32768LL;
    }();
    return A && (reinterpret_cast<uintptr_t>(A) & 15) == 0 && static_cast<long long>(M) * K <= limit;
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
                     p->out_dtype == LSG_DTYPE_F32, static_cast<cudaStream_t>(stream), true);
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
    // Few activation values: every CTA quantizes them itself while its first weights are
    // in flight, which saves a launch and a dependency.  Otherwise quantize once, here.
    if (fused_quant_ok(p->M, p->K, p->A))
        return mmvq_q8_1(p->type, p->M, p->N, p->K, p->B, nullptr, p->C, p->N,
                         p->out_dtype == LSG_DTYPE_F32, s, true, p->A);
    rc = quantize_q8_1(p->A, workspace, p->M, p->K, s, true);
    if (rc != LSG_OK) return rc;
    return mmvq_q8_1(p->type, p->M, p->N, p->K, p->B, workspace, p->C, p->N,
                     p->out_dtype == LSG_DTYPE_F32, s, true);
}

namespace lsg {
namespace {

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

// Device-side alias of a page-locked host buffer, or null when the memory is pageable
// (or not 16-byte aligned, which the vector accesses below need).
void* mapped_alias(const void* host) {
    static const bool off = [] {
        const char* e = getenv("LSG_MMVQ_HOST_DIRECT");
        return e && atoi(e) == 0;
    }();
    if (off || (reinterpret_cast<uintptr_t>(host) & 15)) return nullptr;
    cudaPointerAttributes at = {};
    if (cudaPointerGetAttributes(&at, host) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return at.type == cudaMemoryTypeHost ? at.devicePointer : nullptr;
}

// Result rows from device scratch to the mapped host buffer, 16 bytes per store so that
// the writes cross the bus as full segments.
__global__ void __launch_bounds__(256)
store_to_host_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long bytes) {
    pdl_launch_dependents();
    pdl_wait_prior();
    const long long n16 = bytes >> 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride)
        reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    if (blockIdx.x == 0 && threadIdx.x < (bytes & 15))
        dst[(n16 << 4) + threadIdx.x] = src[(n16 << 4) + threadIdx.x];
}

}  // namespace
}  // namespace lsg

namespace lsg {
namespace {

// Byte ranges of an entry's activations and result.
struct Span {
    uintptr_t b, e;
    bool meets(const Span& o) const { return b < o.e && o.b < e; }
};
Span a_span(const lsg_gguf_mmvq_params& q) {
    const uintptr_t b = reinterpret_cast<uintptr_t>(q.A);
    return {b, b + static_cast<uintptr_t>(q.M) * q.K * 2};
}
Span c_span(const lsg_gguf_mmvq_params& q) {
    const uintptr_t b = reinterpret_cast<uintptr_t>(q.C);
    return {b, b + static_cast<uintptr_t>(q.M) * q.N * (q.out_dtype == LSG_DTYPE_F32 ? 4 : 2)};
}

// True when entry j reads nothing an entry before `limit` writes and writes nothing such an
// entry reads or writes.
bool entry_independent(const lsg_gguf_mmvq_params* p, int j, int limit) {
    const Span a = a_span(p[j]), c = c_span(p[j]);
    for (int k = 0; k < limit; ++k) {
        if (p[k].M == 0 || p[k].N == 0) continue;
        const Span ak = a_span(p[k]), ck = c_span(p[k]);
        if (a.meets(ck) || c.meets(ck) || c.meets(ak)) return false;
    }
    return true;
}

// The same for all entries [i, i + run) against the entries before i.
bool independent_of_earlier(const lsg_gguf_mmvq_params* p, int i, int run) {
    for (int j = i; j < i + run; ++j)
        if (!entry_independent(p, j, i)) return false;
    return true;
}

// LSG_MMVQ_BATCH_OVERLAP=0 keeps every launch of a batch waiting for the one in front of it.
bool batch_overlap_enabled() {
    static const bool on = [] {
        const char* e = getenv("LSG_MMVQ_BATCH_OVERLAP");
        return !e || atoi(e) != 0;
    }();
    return on;
}

// Entries [i, i + run) of a batch that can share one launch: same activations, type, K,
// batch rows and output type, at most four, every N >= 1.
int joinable_run(const lsg_gguf_mmvq_params* p, int i, int n, bool distinct_a = false) {
    int run = 1;
    if (p[i].M < 1 || p[i].N < 1) return 1;
    // with launches that may skip their wait, a launch holds only entries that all depend on
    // earlier entries of the call or all do not: one dependent entry would make the others wait
    const bool free0 = distinct_a && entry_independent(p, i, i);
    while (i + run < n && run < 1 + kMmvqMaxExtra) {
        const lsg_gguf_mmvq_params& a = p[i];
        const lsg_gguf_mmvq_params& b = p[i + run];
        if (b.M != a.M || b.K != a.K || b.type != a.type || b.out_dtype != a.out_dtype || b.N < 1) break;
        if (distinct_a && entry_independent(p, i + run, i) != free0) break;
        if (b.A != a.A) {
            // Activations of its own: the entry may share the launch when both take the
            // quantizer inside the kernel and it shares no buffer with the entries already in
            // the run (they are computed at the same time).
            if (!distinct_a || !fused_quant_ok(a.M, a.K, a.A) || !fused_quant_ok(b.M, b.K, b.A)) break;
            bool apart = true;
            const Span ab = a_span(b), cb = c_span(b);
            for (int k = i; k < i + run && apart; ++k) apart = !ab.meets(c_span(p[k])) && !cb.meets(c_span(p[k])) && !cb.meets(a_span(p[k]));
            if (!apart) break;
        }
        ++run;
    }
    return run;
}

// One launch of a batch call: entries [first, first + count), how it is ordered against the
// launch in front of it (MmvqArgs::dep_mode; -1: the entries are empty, nothing is launched)
// and whether the activations are quantized inside the mat-vec.
struct BatchGroup {
    int first, count, kind;
    bool fused;
};

// Launches that neither read what an earlier entry of the batch writes nor write what an
// earlier entry reads or writes need not wait for the launch in front of them: only the first
// launch waits for the work in front of the batch (and releases the next launch only after
// that wait).  Needs the first launch to be a mat-vec with the quantizer inside and at least
// one later launch of that kind that is independent of the entries before it.
bool batch_is_relaxed(const lsg_gguf_mmvq_params* p, int n) {
    if (!batch_overlap_enabled()) return false;
    bool first = true, first_fused = false;
    for (int i = 0; i < n;) {
        const int run = joinable_run(p, i, n, true);
        if (p[i].M > 0 && p[i].N > 0) {
            const bool fused = fused_quant_ok(p[i].M, p[i].K, p[i].A);
            if (first) first_fused = fused;
            else if (first_fused && fused && independent_of_earlier(p, i, run)) return true;
            first = false;
        }
        i += run;
    }
    return false;
}

// The launch that starts at entry i.
BatchGroup next_batch_group(const lsg_gguf_mmvq_params* p, int n, int i, bool relaxed) {
    BatchGroup g = {i, joinable_run(p, i, n, batch_overlap_enabled()), -1, false};
    const lsg_gguf_mmvq_params& e = p[i];
    if (e.M == 0 || e.N == 0) return g;
    g.fused = fused_quant_ok(e.M, e.K, e.A);
    g.kind = 0;
    if (relaxed) {
        bool launched = false;
        for (int k = 0; k < i && !launched; ++k) launched = p[k].M > 0 && p[k].N > 0;
        if (!launched) g.kind = 1;
        else if (g.fused && independent_of_earlier(p, i, g.count)) g.kind = 2;
    }
    return g;
}

}  // namespace
}  // namespace lsg

extern "C" size_t lsg_gguf_mmvq_batch_workspace_bytes(const lsg_gguf_mmvq_params* p, int n) {
    size_t need = 0;
    for (int i = 0; p && i < n; ++i) {
        const size_t w = lsg_gguf_mmvq_workspace_bytes(p[i].M, p[i].K);
        need = w > need ? w : need;
    }
    return need;
}

extern "C" int lsg_gguf_mmvq_batch(const lsg_gguf_mmvq_params* p, int n, void* workspace,
                                   size_t workspace_bytes, void* stream) {
    if (n == 0) return LSG_OK;
    if (!p || n < 0) return fail(LSG_ERR_INVALID, "gguf_mmvq_batch: null params");
    for (int i = 0; i < n; ++i) {
        const int rc = check_gemm_params("gguf_mmvq_batch", p + i);
        if (rc != LSG_OK) return rc;
    }
    const size_t need = lsg_gguf_mmvq_batch_workspace_bytes(p, n);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(LSG_ERR_WORKSPACE, "gguf_mmvq_batch: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < n;) {
        const BatchGroup g = next_batch_group(p, n, i, batch_is_relaxed(p, n));
        i = g.first + g.count;
        if (g.kind < 0) continue;   // empty entries
        const lsg_gguf_mmvq_params& e = p[g.first];
        const void* W[1 + kMmvqMaxExtra];
        const void* A[1 + kMmvqMaxExtra];
        void* C[1 + kMmvqMaxExtra];
        int N[1 + kMmvqMaxExtra];
        for (int j = 0; j < g.count; ++j) {
            W[j] = p[g.first + j].B;
            A[j] = p[g.first + j].A;
            C[j] = p[g.first + j].C;
            N[j] = p[g.first + j].N;
        }
        const int out_f32 = e.out_dtype == LSG_DTYPE_F32;
        int rc;
        if (g.fused) {
            rc = mmvq_q8_1_joined(e.type, e.M, e.K, g.count, W, C, N, nullptr, out_f32, s, true, e.A, g.kind, A);
        } else {
            rc = quantize_q8_1(e.A, workspace, e.M, e.K, s, true);
            if (rc != LSG_OK) return rc;
            rc = mmvq_q8_1_joined(e.type, e.M, e.K, g.count, W, C, N, workspace, out_f32, s, true, nullptr);
        }
        if (rc != LSG_OK) return rc;
    }
    return LSG_OK;
}

extern "C" int lsg_gguf_mmvq_batch_plan(const lsg_gguf_mmvq_params* p, int n, int* first, int* count, int* kind,
                                        int cap) {
    if (n < 0 || (n > 0 && !p)) return fail(LSG_ERR_INVALID, "gguf_mmvq_batch_plan: null params");
    const bool relaxed = batch_is_relaxed(p, n);
    int groups = 0;
    for (int i = 0; i < n;) {
        const BatchGroup g = next_batch_group(p, n, i, relaxed);
        i = g.first + g.count;
        if (g.kind < 0) continue;
        if (groups < cap) {
            if (first) first[groups] = g.first;
            if (count) count[groups] = g.count;
            if (kind) kind[groups] = g.kind + (g.fused ? 0 : 4);
        }
        ++groups;
    }
    return groups;
}

namespace lsg {
namespace {

constexpr int kMaxHostBatch = 64;

struct HostSlot {
    int first;            // earliest entry of the batch with the same activations
    size_t a_off, q_off;  // staged activations (pageable source) and their Q8_1 image
    size_t c_off;         // result rows when they are not written to the host directly
};

// Workspace layout of a batch; entries with the same A, M and K share one Q8_1 image.
size_t plan_host_batch(const lsg_gguf_mmvq_params* p, int n, HostSlot* slot) {
    size_t off = 0;
    for (int i = 0; i < n; ++i) {
        HostSlot h = {};
        h.first = i;
        for (int j = 0; j < i; ++j)
            if (p[j].A == p[i].A && p[j].M == p[i].M && p[j].K == p[i].K) {
                h.first = slot ? slot[j].first : j;
                break;
            }
        const size_t M = p[i].M > 0 ? p[i].M : 0, N = p[i].N > 0 ? p[i].N : 0, K = p[i].K > 0 ? p[i].K : 0;
        if (h.first == i) {
            h.a_off = off;
            off += align256(M * K * 2);
            h.q_off = off;
            off += align256(M * (K / 32) * kQ8_1Bytes);
        } else if (slot) {
            h.a_off = slot[h.first].a_off;
            h.q_off = slot[h.first].q_off;
        }
        h.c_off = off;
        off += align256(M * N * 4);
        if (slot) slot[i] = h;
    }
    return off;
}

}  // namespace
}  // namespace lsg

extern "C" size_t lsg_gguf_mmvq_host_batch_workspace_bytes(const lsg_gguf_mmvq_params* p, int n) {
    if (!p || n <= 0 || n > kMaxHostBatch) return 0;
    return plan_host_batch(p, n, nullptr);
}

extern "C" size_t lsg_gguf_mmvq_host_workspace_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    lsg_gguf_mmvq_params p = {};
    p.M = M;
    p.N = N;
    p.K = K;
    return plan_host_batch(&p, 1, nullptr);
}

// Page-locked buffers are reached from the kernels themselves: the quantizer reads the
// activations through their device alias and the mat-vec (or, above four batch rows, a
// small kernel with 16-byte stores) writes the result rows, so that a projection is two
// dependent kernels on one engine.  Copies by the DMA engines (the route for pageable
// memory) cost an engine switch before and after the mat-vec, several times the
// mat-vec's own duration at batch 1.
extern "C" int lsg_gguf_mmvq_host_batch(const lsg_gguf_mmvq_params* p, int n, void* workspace,
                                        size_t workspace_bytes, void* stream) {
    if (n == 0) return LSG_OK;
    if (!p || n < 0) return fail(LSG_ERR_INVALID, "gguf_mmvq_host: null params");
    if (n > kMaxHostBatch)
        return fail(LSG_ERR_INVALID, "gguf_mmvq_host: at most %d projections per batch, got %d", kMaxHostBatch, n);
    for (int i = 0; i < n; ++i) {
        const int rc = check_gemm_params("gguf_mmvq_host", p + i);
        if (rc != LSG_OK) return rc;
        if (p[i].M > 0 && p[i].N > 0 && (!p[i].A || !p[i].C))
            return fail(LSG_ERR_INVALID, "gguf_mmvq_host: null host pointer (entry %d)", i);
        if (p[i].M > 0 && p[i].N > 0 && p[i].K == 0)
            return fail(LSG_ERR_INVALID, "gguf_mmvq: K must be positive");
    }
    HostSlot slot[kMaxHostBatch];
    const size_t need = plan_host_batch(p, n, slot);
    if (need == 0) return LSG_OK;
    if (!workspace || workspace_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "gguf_mmvq_host: workspace too small (have %zu, need %zu)",
                    workspace ? workspace_bytes : size_t(0), need);
    if (reinterpret_cast<uintptr_t>(workspace) & 255)
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmvq_host: workspace must be 256-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* base = static_cast<uint8_t*>(workspace);
    // Every input is there when the call is made, so the distinct activations are quantized by
    // ONE launch up front (their reads over PCIe overlap) instead of one quantizer launch in
    // front of each group of projections: a layer of seven projections is five dependent
    // launches instead of eight.  More than eight distinct inputs fall back to one launch each.
    bool quantized_up_front = false;
    {
        const void* xs[8];
        void* qs[8];
        int Ms[8], Ks[8];
        int cnt = 0;
        bool fits = true;
        // not when a projection reads what an earlier one of the batch writes
        for (int j = 1; j < n && fits; ++j) {
            const uintptr_t a0 = reinterpret_cast<uintptr_t>(p[j].A);
            const uintptr_t a1 = a0 + static_cast<size_t>(p[j].M) * p[j].K * 2;
            for (int i = 0; i < j; ++i) {
                const uintptr_t c0 = reinterpret_cast<uintptr_t>(p[i].C);
                const uintptr_t c1 = c0 + static_cast<size_t>(p[i].M) * p[i].N * (p[i].out_dtype == LSG_DTYPE_F32 ? 4 : 2);
                if (a0 < c1 && c0 < a1) fits = false;
            }
        }
        for (int i = 0; i < n && fits; ++i) {
            if (p[i].M == 0 || p[i].N == 0 || slot[i].first != i) continue;
            if (cnt == 8) {
                fits = false;
                break;
            }
            const void* a_src = mapped_alias(p[i].A);
            if (!a_src) {
                const size_t a_bytes = static_cast<size_t>(p[i].M) * p[i].K * 2;
                LSG_CUDA_TRY(cudaMemcpyAsync(base + slot[i].a_off, p[i].A, a_bytes, cudaMemcpyHostToDevice, s));
                a_src = base + slot[i].a_off;
            }
            xs[cnt] = a_src;
            qs[cnt] = base + slot[i].q_off;
            Ms[cnt] = p[i].M;
            Ks[cnt] = p[i].K;
            ++cnt;
        }
        if (fits && cnt > 1) {
            const int rc = quantize_q8_1_batch(cnt, xs, qs, Ms, Ks, s, true);
            if (rc != LSG_OK) return rc;
            quantized_up_front = true;
        }
    }
    // With every input quantized up front, every result written straight to its page-locked
    // buffer and no buffer shared between entries, the projections do not depend on each other:
    // those of one shape share a launch whatever their input, and a launch does not wait for
    // the one in front of it (the first waits for the quantizer and only then releases the next).
    bool apart = quantized_up_front && batch_overlap_enabled();
    for (int i = 0; i < n && apart; ++i) {
        if (p[i].M == 0 || p[i].N == 0) continue;
        if (p[i].M > 4 || !mapped_alias(p[i].C)) apart = false;
        for (int k = 0; k < i && apart; ++k) {
            if (p[k].M == 0 || p[k].N == 0) continue;
            if (c_span(p[i]).meets(c_span(p[k])) || c_span(p[i]).meets(a_span(p[k])) || a_span(p[i]).meets(c_span(p[k])))
                apart = false;
        }
    }
    bool launched = false;
    for (int i = 0; i < n;) {
        const lsg_gguf_mmvq_params& e = p[i];
        int run = joinable_run(p, i, n);
        if (apart && e.M > 0 && e.N > 0) {
            run = 1;
            while (i + run < n && run < 1 + kMmvqMaxExtra && p[i + run].M == e.M && p[i + run].K == e.K &&
                   p[i + run].type == e.type && p[i + run].out_dtype == e.out_dtype && p[i + run].N >= 1)
                ++run;
        }
        if (e.M == 0 || e.N == 0) {
            i += run;
            continue;
        }
        const int out_f32 = e.out_dtype == LSG_DTYPE_F32;
        const size_t a_bytes = static_cast<size_t>(e.M) * e.K * 2;
        uint8_t* q_dev = base + slot[i].q_off;
        int rc;
        if (slot[i].first == i && !quantized_up_front) {
            const void* a_src = mapped_alias(e.A);
            if (!a_src) {
                LSG_CUDA_TRY(cudaMemcpyAsync(base + slot[i].a_off, e.A, a_bytes, cudaMemcpyHostToDevice, s));
                a_src = base + slot[i].a_off;
            }
            rc = quantize_q8_1(a_src, q_dev, e.M, e.K, s, true);
            if (rc != LSG_OK) return rc;
        }
        // The projections of this input that can share a launch; each writes either the
        // host buffer's alias or its rows of the workspace.
        const void* W[1 + kMmvqMaxExtra];
        const void* XQ[1 + kMmvqMaxExtra];
        void* C[1 + kMmvqMaxExtra];
        void* c_map[1 + kMmvqMaxExtra];
        int N[1 + kMmvqMaxExtra];
        for (int j = 0; j < run; ++j) {
            c_map[j] = mapped_alias(p[i + j].C);
            W[j] = p[i + j].B;
            XQ[j] = base + slot[i + j].q_off;
            N[j] = p[i + j].N;
            C[j] = (c_map[j] && e.M <= 4) ? c_map[j] : static_cast<void*>(base + slot[i + j].c_off);
        }
        const int dep_mode = apart ? (launched ? 2 : 1) : 0;
        launched = true;
        rc = mmvq_q8_1_joined(e.type, e.M, e.K, run, W, C, N, q_dev, out_f32, s, true, nullptr, dep_mode, nullptr, XQ);
        if (rc != LSG_OK) return rc;
        for (int j = 0; j < run; ++j) {
            if (C[j] == c_map[j]) continue;
            const size_t c_bytes = static_cast<size_t>(e.M) * N[j] * (out_f32 ? 4 : 2);
            if (c_map[j]) {
                const long long n16 = static_cast<long long>(c_bytes >> 4);
                const unsigned grid = static_cast<unsigned>(n16 < 256 ? 1 : (n16 / 256 > 296 ? 296 : n16 / 256));
                LSG_CUDA_TRY(launch_kernel(store_to_host_kernel, dim3(grid), dim3(256), 0, s, true,
                                           static_cast<const uint8_t*>(C[j]), static_cast<uint8_t*>(c_map[j]),
                                           static_cast<long long>(c_bytes)));
            } else {
                LSG_CUDA_TRY(cudaMemcpyAsync(p[i + j].C, C[j], c_bytes, cudaMemcpyDeviceToHost, s));
            }
        }
        i += run;
    }
    return LSG_OK;
}

extern "C" int lsg_gguf_mmvq_host(const lsg_gguf_mmvq_params* p, void* workspace,
                                  size_t workspace_bytes, void* stream) {
    if (!p) return fail(LSG_ERR_INVALID, "gguf_mmvq_host: null params");
    return lsg_gguf_mmvq_host_batch(p, 1, workspace, workspace_bytes, stream);
}

extern "C" int lsg_test_mmvq_drop_slab(int slab) {
    g_drop_slab = slab < 0 ? -1 : slab;
    return LSG_OK;
}

#ifdef LSG_MMVQ_TRACE
extern "C" __attribute__((visibility("default"))) int lsg_mmvq_set_trace(void* buf, int slots) {
    g_trace = static_cast<unsigned long long*>(buf);
    g_trace_slots = slots;
    g_trace_launch = 0;
    return LSG_OK;
}
#endif

extern "C" int lsg_mmvq_set_tuning(int consumer_warps, int ctas_per_sm, int stage_kib,
                                   int smem_share, int skip_math) {
    MmvqTune& t = tuning();
    if (consumer_warps > 0) t.warps = consumer_warps;
    if (ctas_per_sm > 0) t.ctas = ctas_per_sm;
    if (stage_kib > 0) t.stage_kb = stage_kib;
    if (smem_share > 0) t.share = smem_share;
#ifdef LSG_DEBUG_KNOBS
    if (skip_math >= 0) t.skip_math = skip_math ? 1 : 0;
#else
    if (skip_math > 0)
        return fail(LSG_ERR_UNSUPPORTED, "mmvq_set_tuning: skip_math exists in bench builds (-DLSG_DEBUG_KNOBS) only");
#endif
    return LSG_OK;
}
