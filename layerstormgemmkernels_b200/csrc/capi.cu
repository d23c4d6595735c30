// C-ABI plumbing: thread-local error text, per-device status word, queries.
#include "common.cuh"
#include "formats.cuh"
#include "host.h"

#include <string.h>

namespace lsg {

namespace {
thread_local char g_err[512] = "";
__device__ unsigned int g_status_word = 0;
long long g_wait_limit = kWaitLimitCycles;
}  // namespace

long long wait_limit_cycles() { return g_wait_limit; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) in %s", static_cast<int>(e),
             cudaGetErrorString(e), what);
    return LSG_ERR_CUDA;
}

unsigned int* device_status_word() {
    static unsigned int* cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev];
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    if (dev >= 0 && dev < 64) cached[dev] = static_cast<unsigned int*>(p);
    return static_cast<unsigned int*>(p);
}

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < 64 && cached[dev]) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
        n = 148;
    if (dev >= 0 && dev < 64) cached[dev] = n;
    return n;
}

}  // namespace lsg

using namespace lsg;

extern "C" const char* lsg_last_error(void) { return g_err; }

extern "C" const char* lsg_version(void) { return "lsg-b200 0.1 (sm_100a)"; }

extern "C" int lsg_device_status(int* code) {
    if (!code) return fail(LSG_ERR_INVALID, "device_status: null pointer");
    LSG_CUDA_TRY(cudaDeviceSynchronize());
    unsigned int v = 0;
    LSG_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_status_word, sizeof(v)));
    if (v != 0) {
        const unsigned int zero = 0;
        LSG_CUDA_TRY(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(zero)));
    }
    *code = static_cast<int>(v);
    return LSG_OK;
}

extern "C" int lsg_set_wait_limit_cycles(long long cycles) {
    if (cycles < 0) return fail(LSG_ERR_INVALID, "set_wait_limit_cycles: negative limit");
    g_wait_limit = cycles == 0 ? kWaitLimitCycles : cycles;
    return LSG_OK;
}

extern "C" int lsg_gguf_block_values(int type) { return gguf_block_values(type); }
extern "C" int lsg_gguf_block_bytes(int type) { return gguf_block_bytes(type); }

extern "C" int lsg_quantize_q8_1(const void* x_bf16, void* q8_1_out, int M, int K, void* stream) {
    return quantize_q8_1(x_bf16, q8_1_out, M, K, static_cast<cudaStream_t>(stream), false);
}
