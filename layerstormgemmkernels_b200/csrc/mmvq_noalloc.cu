// lsg_gguf_mmvq_noalloc: the GGUF decode mat-vec for callers that may not allocate.
//
// lsg_gguf_mmvq needs a scratch buffer for the Q8_1 image of the activations and leaves
// its allocation to the caller.  Some callers have nowhere to get one from: code running
// under a fixed device-memory plan (everything reserved at start-up, nothing afterwards),
// a plug-in invoked from inside another runtime that owns the allocator, or a latency-
// critical decode loop where a cudaMalloc would serialise the whole device.  For them the
// scratch lives here, in a file-scope device array that every GPU loading this library
// carries until the process exits.
//
// Limits and rules:
//   * the Q8_1 image must fit the array: M * (K/32) * 36 <= LSG_NOALLOC_MAX_Q8_1_BYTES
//     (147,456 bytes: eight rows of K = 16384, or one row of K = 131072); larger
//     problems are rejected with LSG_ERR_WORKSPACE and a message saying so;
//   * the first call on each device looks the array's device address up
//     (cudaGetSymbolAddress) and remembers it; make that first call outside any stream
//     capture;
//   * all calls on a device share the one array, which simply keeps whatever the last call
//     wrote.  Nothing in it has to start at zero - the quantizer overwrites every byte the
//     mat-vec then reads - but two calls whose kernels overlap on the GPU (different
//     streams, no ordering between them) would race on it.  Serialise them, or use
//     lsg_gguf_mmvq with separate workspaces.
//   * no cudaMalloc, cudaFree or other allocating call is made, here or below.
#include "common.cuh"
#include "formats.cuh"
#include "host.h"

namespace lsg {

namespace {

constexpr size_t kNoAllocScratchBytes = 147456;  // == LSG_NOALLOC_MAX_Q8_1_BYTES in lsg.h

static __device__ __align__(256) unsigned char g_noalloc_q8_1_scratch[kNoAllocScratchBytes];

// Device address of the scratch array on the current device.  In host code the array's
// name is only a stand-in; the address a kernel can use has to be asked for, once per
// device, with that device current.
int noalloc_scratch(void** out) {
    static void* cached[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && cached[dev]) {
        *out = cached[dev];
        return LSG_OK;
    }
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_q8_1_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_noalloc_q8_1_scratch)");
    if (!p) return fail(LSG_ERR_CUDA, "gguf_mmvq_noalloc: scratch symbol has no device address");
    if (dev >= 0 && dev < 64) cached[dev] = p;
    *out = p;
    return LSG_OK;
}

}  // namespace

}  // namespace lsg

using namespace lsg;

extern "C" int lsg_gguf_mmvq_noalloc(const lsg_gguf_mmvq_params* p, void* stream) {
    int rc = check_gemm_params("gguf_mmvq_noalloc", p);
    if (rc != LSG_OK) return rc;
    if (p->M == 0 || p->N == 0) return LSG_OK;
    const size_t need = static_cast<size_t>(p->M) * (p->K / 32) * kQ8_1Bytes;
    if (need > kNoAllocScratchBytes)
        return fail(LSG_ERR_WORKSPACE,
                    "gguf_mmvq_noalloc: M=%d, K=%d needs %zu bytes of Q8_1 scratch but the built-in "
                    "array holds %zu; use lsg_gguf_mmvq with a caller-provided workspace",
                    p->M, p->K, need, kNoAllocScratchBytes);
    void* scratch = nullptr;
    rc = noalloc_scratch(&scratch);
    if (rc != LSG_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    rc = quantize_q8_1(p->A, scratch, p->M, p->K, s, true);
    if (rc != LSG_OK) return rc;
    return mmvq_q8_1(p->type, p->M, p->N, p->K, p->B, scratch, p->C, p->N,
                     p->out_dtype == LSG_DTYPE_F32, s, true);
}
