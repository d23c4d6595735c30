// One translation unit per GGUF type (compiled with -DLSG_MMVQ_TYPE=<id>) so the
// eight decoders build in parallel.  Picks the kernel variant and the pipeline
// geometry for a shape and launches it.
#include "mmvq.cuh"

#ifndef LSG_MMVQ_TYPE
#error "compile with -DLSG_MMVQ_TYPE=<lsg_gguf_type id>"
#endif

namespace lsg {

namespace {

constexpr int T = LSG_MMVQ_TYPE;
constexpr int kConsumerWarps = 15;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kSmemCap = 227 * 1024;
constexpr int kStageTarget = 24 * 1024;

template <int MT, int RW, int L, int XREG>
int launch_variant(const MmvqArgs& a, int grid, size_t smem, cudaStream_t stream, bool pdl) {
    auto kernel = mmvq_kernel<T, MT, RW, L, XREG>;
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemCap));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    LSG_CUDA_TRY(launch_kernel(kernel, dim3(grid), dim3(kThreads), smem, stream, pdl, a));
    return LSG_OK;
}

}  // namespace

// Largest number of activation rows one launch can hold in shared memory.
int MMVQ_FN(max_rows)(int K) {
    constexpr ChunkShape S = Fmt<T>::SHAPE;
    const int per_row = x_row_bytes<S>(K);
    const int row_bytes = (K / Fmt<T>::VALS) * Fmt<T>::BYTES;
    // leave room for two stages of at least one weight row each
    const int ring_min = 2 * (((row_bytes + 47 + 127) / 128) * 128) + 256;
    const int rows = (kSmemCap - ring_min) / per_row;
    return rows < 1 ? 0 : rows;
}

int MMVQ_FN(launch)(MmvqArgs a, cudaStream_t stream, bool pdl) {
    using F = Fmt<T>;
    constexpr ChunkShape S = F::SHAPE;
    constexpr int CHUNK_VALS = (S == kBlock) ? 32 : 64;
    constexpr int XR = (S == kBlock) ? 4 : 2;

    a.row_bytes = (a.K / F::VALS) * F::BYTES;
    const int C = a.K / CHUNK_VALS;
    const int grid = a.N < sm_count() ? a.N : sm_count();
    const int rows_per_cta = (a.N + grid - 1) / grid;

    a.x_bytes = ((a.M * x_row_bytes<S>(a.K) + 127) / 128) * 128;
    int slab_rows = kStageTarget / a.row_bytes;
    if (slab_rows < 1) slab_rows = 1;
    if (slab_rows > rows_per_cta) slab_rows = rows_per_cta;
    int stage_bytes = ((slab_rows * a.row_bytes + 47 + 127) / 128) * 128;
    const int bar_bytes = 2 * kMmvqMaxStages * 8;
    int avail = kSmemCap - a.x_bytes - bar_bytes;
    while (slab_rows > 1 && 2 * stage_bytes > avail) {
        slab_rows = (slab_rows + 1) / 2;
        stage_bytes = ((slab_rows * a.row_bytes + 47 + 127) / 128) * 128;
    }
    if (2 * stage_bytes > avail)
        return fail(LSG_ERR_UNSUPPORTED,
                    "gguf_mmvq: M=%d rows of K=%d do not fit shared memory with a weight ring",
                    a.M, a.K);
    const int n_slabs = (rows_per_cta + slab_rows - 1) / slab_rows;
    int stages = avail / stage_bytes;
    if (stages > kMmvqMaxStages) stages = kMmvqMaxStages;
    if (stages > n_slabs) stages = n_slabs < 2 ? 2 : n_slabs;
    a.slab_rows = slab_rows;
    a.stage_bytes = stage_bytes;
    a.stages = stages;
    const size_t smem = static_cast<size_t>(a.x_bytes) + static_cast<size_t>(stages) * stage_bytes + bar_bytes;

    const bool wide = C >= 24;  // a whole warp per weight row
    if (a.M == 1) {
        if (wide && C <= 32 * XR) return launch_variant<1, 2, 32, XR>(a, grid, smem, stream, pdl);
        if (wide) return launch_variant<1, 2, 32, 0>(a, grid, smem, stream, pdl);
        return launch_variant<1, 2, 8, 0>(a, grid, smem, stream, pdl);
    }
    if (a.M == 2) {
        if (wide) return launch_variant<2, 2, 32, 0>(a, grid, smem, stream, pdl);
        return launch_variant<2, 2, 8, 0>(a, grid, smem, stream, pdl);
    }
    if (a.M <= 4) {
        if (wide) return launch_variant<4, 2, 32, 0>(a, grid, smem, stream, pdl);
        return launch_variant<4, 2, 8, 0>(a, grid, smem, stream, pdl);
    }
    if (wide) return launch_variant<8, 2, 32, 0>(a, grid, smem, stream, pdl);
    return launch_variant<8, 2, 8, 0>(a, grid, smem, stream, pdl);
}

}  // namespace lsg
