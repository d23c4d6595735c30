// One translation unit per GGUF type (compiled with -DLSG_MMVQ_TYPE=<id>) so the
// eight decoders build in parallel.  Picks the kernel variant and the pipeline
// geometry for a shape and launches it.
#include "mmvq_grouped.cuh"


#ifndef LSG_MMVQ_TYPE
#error "compile with -DLSG_MMVQ_TYPE=<lsg_gguf_type id>"
#endif

namespace lsg {

namespace {

constexpr int T = LSG_MMVQ_TYPE;
constexpr int kSmemCap = 227 * 1024;

template <int MT, int RW, int L>
int launch_variant(const MmvqArgs& a, int grid, size_t smem, cudaStream_t stream, bool pdl) {
    auto kernel = mmvq_kernel<T, MT, RW, L>;
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemCap));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    LSG_CUDA_TRY(launch_kernel(kernel, dim3(grid), dim3((a.cons_warps + 1) * 32), smem, stream, pdl, a));
    return LSG_OK;
}

template <int MT, int RW>
int launch_lanes(int lanes, const MmvqArgs& a, int grid, size_t smem, cudaStream_t stream, bool pdl) {
    switch (lanes) {
        case 4: return launch_variant<MT, RW, 4>(a, grid, smem, stream, pdl);
        case 8: return launch_variant<MT, RW, 8>(a, grid, smem, stream, pdl);
        case 16: return launch_variant<MT, RW, 16>(a, grid, smem, stream, pdl);
        default: return launch_variant<MT, RW, 32>(a, grid, smem, stream, pdl);
    }
}

template <int MT>
int launch_rows(int rw, int lanes, const MmvqArgs& a, int grid, size_t smem, cudaStream_t stream,
                bool pdl) {
    // one weight row per lane group is only built for whole-warp groups (long rows)
    if (rw == 1 && lanes == 32) return launch_variant<MT, 1, 32>(a, grid, smem, stream, pdl);
    return launch_lanes<MT, 2>(lanes, a, grid, smem, stream, pdl);
}

}  // namespace

// Largest number of batch rows one launch can hold in shared memory.
int MMVQ_FN(max_rows)(int K) {
    const int per_row = x_row_bytes<T>(K);
    const int row_bytes = (K / Fmt<T>::VALS) * Fmt<T>::BYTES;
    // leave room for two stages of at least one weight row each
    const int ring_min = 2 * (((row_bytes + 47 + 127) / 128) * 128) + 256;
    const int rows = (kSmemCap - ring_min) / per_row;
    return rows < 1 ? 0 : rows;
}

int MMVQ_FN(launch)(MmvqArgs a, const MmvqTune& tn_in, cudaStream_t stream, bool pdl) {
    using F = Fmt<T>;
    a.row_bytes = (a.K / F::VALS) * F::BYTES;
    // Small matrices (a CTA's share of the weights is at most 40 KB, e.g. a 1024 x 4096 Q4_K
    // k or v projection launched alone): eleven
    // consumer warps and half the shared memory, so that two consecutive launches of a
    // stream are resident together and the second one's prologue and weight prefetch overlap
    // the first one's tail.
    MmvqTune tn = tn_in;
    // Joined launches: geometry follows the rows of all matrices together.
    const int n_prob = 1 + a.n_extra;
    int n_rows[1 + kMmvqMaxExtra] = {a.N};
    int n_total = a.N;
    for (int j = 0; j < a.n_extra; ++j) {
        n_rows[1 + j] = a.Nx[j];
        n_total += a.Nx[j];
    }
    int ctas_of[1 + kMmvqMaxExtra] = {};
    {
        static const int small_kb = [] {
            const char* e = getenv("LSG_MMVQ_SMALL_KB");
            return e ? atoi(e) : 40;   // 0 switches this off
        }();
        const long long per_cta = static_cast<long long>(n_total) * a.row_bytes / (sm_count() > 0 ? sm_count() : 1);
        if (small_kb > 0 && per_cta <= static_cast<long long>(small_kb) * 1024 && tn.share == 1 && tn.ctas == 1) {
            tn.warps = tn.warps > 11 ? 11 : tn.warps;
            tn.share = 2;
        }
    }
    // Launches of a batch that do not wait for each other (dep_mode 1, 2), one batch row,
    // quantizer inside: half the shared memory and few enough warps for two CTAs' registers, so
    // that the next launch's CTA is resident beside this one's - it builds its activation image
    // and fills its ring while this one streams, and keeps the memory system busy through this
    // one's tail.  Measured on the decoder layer (two launches per layer): 25.2 -> 22.6 us with
    // six consumer warps for Q4_K, 35.8 -> 33.6 us with seven for Q6_K.  With launches that wait
    // for each other, with more batch rows (the arithmetic needs the warps) and with results
    // written to host memory the full-size CTA is faster.
    if (a.dep_mode != 0 && a.M == 1 && a.A != nullptr && tn.share == 1 && tn.ctas == 1) {
        const int w = (T == LSG_GGUF_Q4_K) ? 6 : 7;
        tn.warps = tn.warps > w ? w : tn.warps;
        tn.share = 2;
    }
    const int U = a.K / Mmvq<T>::UV;
    a.cons_warps = tn.warps;
    a.debug_skip = tn.skip_math;
    a.x_bytes = ((a.M * x_row_bytes<T>(a.K) + 127) / 128) * 128;
    const int bar_bytes = 2 * kMmvqMaxStages * 8 + 16 + kMmvqMaxStages * 4;

    // lanes per weight row: the smallest power of two covering the units of a row
    int lanes = 4;
    while (lanes < 32 && lanes < U) lanes *= 2;

    // Several CTAs per SM when the activation image leaves room for their rings:
    // their prologues, tails and pipeline fills then overlap each other and, under
    // programmatic dependent launch, the neighbouring kernels in the stream.
    int grid = 0, rw = 2, stages = 0;
    size_t smem = 0;
    // `share` = how many CTAs (of this and of neighbouring launches) split an SM's
    // shared memory; `ctas` = how many of them belong to one launch.
    for (int share = tn.share > tn.ctas ? tn.share : tn.ctas; share >= 1; --share) {
        const int ctas = tn.ctas < share ? tn.ctas : share;
        const int smem_cap = kSmemCap / share - (share > 1 ? 1024 : 0);  // 1 KB per-CTA reserve
        const int slots = sm_count() * ctas;
        grid = n_total < slots ? n_total : slots;
        int rows_per_cta = (n_total + grid - 1) / grid;
        if (n_prob > 1) {
            // CTAs in proportion to the rows; what rounding leaves over goes, one at a
            // time, to the matrix with the most rows per CTA.
            int used = 0;
            for (int j = 0; j < n_prob; ++j) {
                int g = static_cast<int>(static_cast<long long>(grid) * n_rows[j] / n_total);
                ctas_of[j] = g < 1 ? 1 : g;
                used += ctas_of[j];
            }
            while (used != grid) {
                int pick = 0;
                double worst = used < grid ? -1.0 : 1e30;
                for (int j = 0; j < n_prob; ++j) {
                    const double load = static_cast<double>(n_rows[j]) / ctas_of[j];
                    if (used < grid ? load > worst : (ctas_of[j] > 1 && load < worst)) {
                        worst = load;
                        pick = j;
                    }
                }
                ctas_of[pick] += used < grid ? 1 : -1;
                used += used < grid ? 1 : -1;
            }
            rows_per_cta = 0;
            for (int j = 0; j < n_prob; ++j) {
                const int r = (n_rows[j] + ctas_of[j] - 1) / ctas_of[j];
                rows_per_cta = r > rows_per_cta ? r : rows_per_cta;
            }
        }
        // Long rows: one row per lane group, so that the rows resident in the ring
        // are enough to occupy every consumer warp.
        rw = (lanes == 32 && a.row_bytes * 2 * tn.warps > (smem_cap * 3) / 4) ? 1 : 2;
        // Few rows per CTA (small matrices): one row per lane group doubles the number of row
        // groups, so that they cover the consumer warps instead of leaving most of them idle.
        // (One row per group is only built for whole-warp groups; for narrower groups the
        // slab must be planned with the two rows per group the kernel really takes, or a
        // third of its row groups come out empty.)
        if (lanes == 32 && rows_per_cta < 2 * tn.warps) rw = 1;
        int slab_rows = tn.stage_kb * 1024 / a.row_bytes;
        // whole row groups per slab, so that no lane group idles on a ragged slab end
        const int rpp = (32 / lanes) * rw;
        if (slab_rows > rpp) slab_rows -= slab_rows % rpp;
        if (slab_rows < 1) slab_rows = 1;
        if (slab_rows > rows_per_cta) slab_rows = rows_per_cta;
        int stage_bytes = ((slab_rows * a.row_bytes + 47 + 127) / 128) * 128;
        const int avail = smem_cap - a.x_bytes - bar_bytes;
        while (slab_rows > 1 && 2 * stage_bytes > avail) {
            slab_rows = (slab_rows + 1) / 2;
            stage_bytes = ((slab_rows * a.row_bytes + 47 + 127) / 128) * 128;
        }
        if (2 * stage_bytes > avail) {
            if (share > 1) continue;
            return fail(LSG_ERR_UNSUPPORTED,
                        "gguf_mmvq: M=%d rows of K=%d do not fit shared memory with a weight ring",
                        a.M, a.K);
        }
        const int n_slabs = (rows_per_cta + slab_rows - 1) / slab_rows;
        stages = avail / stage_bytes;
        if (stages > kMmvqMaxStages) stages = kMmvqMaxStages;
        if (stages > n_slabs) stages = n_slabs < 2 ? 2 : n_slabs;
        a.slab_rows = slab_rows;
        a.stage_bytes = stage_bytes;
        a.stages = stages;
        smem = static_cast<size_t>(a.x_bytes) + static_cast<size_t>(stages) * stage_bytes + bar_bytes;
        break;
    }

    if (n_prob > 1) {
        a.rows_q = n_rows[0] / ctas_of[0];
        a.rows_r = n_rows[0] % ctas_of[0];
        int first = ctas_of[0];
        for (int j = 0; j < a.n_extra; ++j) {
            a.cta0x[j] = first;
            a.rows_qx[j] = n_rows[1 + j] / ctas_of[1 + j];
            a.rows_rx[j] = n_rows[1 + j] % ctas_of[1 + j];
            first += ctas_of[1 + j];
        }
    }
    finish_args(a, grid, (32 / lanes) * rw);
    if (a.M == 1) return launch_rows<1>(rw, lanes, a, grid, smem, stream, pdl);
    if (a.M == 2) return launch_rows<2>(rw, lanes, a, grid, smem, stream, pdl);
    if (a.M <= 4) return launch_rows<4>(rw, lanes, a, grid, smem, stream, pdl);
    return launch_rows<8>(rw, lanes, a, grid, smem, stream, pdl);
}

namespace {

template <int RW, int L>
int launch_grouped_variant(const GroupedArgs& a, int grid, size_t smem, cudaStream_t stream, bool pdl) {
    auto kernel = mmvq_grouped_kernel<T, RW, L>;
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kSmemCap));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    LSG_CUDA_TRY(launch_kernel(kernel, dim3(grid), dim3((a.cons_warps + 1) * 32), smem, stream, pdl, a));
    return LSG_OK;
}

constexpr int kGroupedCtlBytes = 2 * kMmvqMaxStages * 8 + 16 + kMmvqMaxStages * 4 + 3 * kGroupedMaxSlabs * 4;
constexpr int kGroupedImageBudget = 64 * 1024;  // activation image of one segment

}  // namespace

// Rows of one segment: as many batch rows as fit the image budget (at least 1, at most 64).
int MMVQ_FN(grouped_max_rows)(int K, const MmvqTune&) {
    int rows = kGroupedImageBudget / x_row_bytes<T>(K);
    if (rows > 64) rows = 64;
    if (rows >= 8) rows &= ~7;
    return rows < 1 ? 1 : rows;
}

int MMVQ_FN(grouped_launch)(GroupedArgs a, const MmvqTune& tn, int max_segments, cudaStream_t stream,
                            bool pdl) {
    using F = Fmt<T>;
    a.row_bytes = (a.K / F::VALS) * F::BYTES;
    a.cons_warps = tn.warps;
    const int U = a.K / Mmvq<T>::UV;
    int lanes = 4;
    while (lanes < 32 && lanes < U) lanes *= 2;
    const int max_rows = MMVQ_FN(grouped_max_rows)(a.K, tn);
    a.x_bytes = ((max_rows * x_row_bytes<T>(a.K) + 127) / 128) * 128;
    const int avail = kSmemCap - a.x_bytes - kGroupedCtlBytes - 128;
    int slab_rows = tn.stage_kb * 1024 / a.row_bytes;
    if (slab_rows < 1) slab_rows = 1;
    if (slab_rows > a.N) slab_rows = a.N;
    int stage_bytes = ((slab_rows * a.row_bytes + 47 + 127) / 128) * 128;
    while (slab_rows > 1 && 2 * stage_bytes > avail) {
        slab_rows = (slab_rows + 1) / 2;
        stage_bytes = ((slab_rows * a.row_bytes + 47 + 127) / 128) * 128;
    }
    if (2 * stage_bytes > avail)
        return fail(LSG_ERR_UNSUPPORTED, "gguf_grouped_gemm: K=%d does not fit the shared-memory ring", a.K);
    int stages = avail / stage_bytes;
    if (stages > kMmvqMaxStages) stages = kMmvqMaxStages;
    a.slab_rows = slab_rows;
    a.stage_bytes = stage_bytes;
    a.stages = stages;
    // Enough CTAs that no CTA's slab table can overflow even if every segment is live.
    const long long v_max = static_cast<long long>(max_segments) * a.N;
    long long grid = sm_count();
    const long long per_cta_cap = static_cast<long long>(kGroupedMaxSlabs / 4) * slab_rows;
    if (v_max / grid > per_cta_cap) grid = (v_max + per_cta_cap - 1) / per_cta_cap;
    // each segment boundary inside a range adds a slab: bound that too
    const long long seg_cap = static_cast<long long>(kGroupedMaxSlabs / 4) * a.N;
    if (v_max / grid > seg_cap) grid = (v_max + seg_cap - 1) / seg_cap;
    if (grid > 0x7fffffffLL) return fail(LSG_ERR_UNSUPPORTED, "gguf_grouped_gemm: problem too large");
    const size_t smem = static_cast<size_t>(a.x_bytes) + static_cast<size_t>(stages) * stage_bytes +
                        kGroupedCtlBytes;
    switch (lanes) {
        case 4: return launch_grouped_variant<2, 4>(a, static_cast<int>(grid), smem, stream, pdl);
        case 8: return launch_grouped_variant<2, 8>(a, static_cast<int>(grid), smem, stream, pdl);
        case 16: return launch_grouped_variant<2, 16>(a, static_cast<int>(grid), smem, stream, pdl);
        default: return launch_grouped_variant<2, 32>(a, static_cast<int>(grid), smem, stream, pdl);
    }
}

}  // namespace lsg
