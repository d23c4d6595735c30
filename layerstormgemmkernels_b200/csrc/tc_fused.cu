// Tensor-core GGUF GEMM with the weight dequantization fused into the operand pipeline.
//
// Same contract as the prepared-operand path (tc_gemm.cu): C[m, n] = sum_k x16[m,k] * w16[n,k]
// with w16 the fp16 of the dequantized weight and x16 the fp16 of the activation's Q8_1
// round trip, i.e. the reference's integer result (csrc/sm120/gemm/gguf/mmq_mma/
// mmq_kernel_32aligned.cuh:34-169, gguf_mmvq.cu:66-187) up to one fp16 rounding per operand.
// The difference is where w16 comes from: here the packed GGUF blocks are read straight from
// global memory by eight decoder warps, dequantized in registers and stored into TENSOR
// MEMORY (tcgen05.st), from where tcgen05.mma takes them as its A operand.  No fp16 copy of
// the weights exists in HBM (they cost their packed 4.5-8.5 bits per value of traffic) nor in
// shared memory: the shared-memory port, which limits a tcgen05 GEMM with both operands in
// shared memory (128 x 256 x 64 tile: 48 KB read + 48 KB written per 512 tensor cycles at
// 128 B/clk), only carries the token tile.
//
// The roles are swapped with respect to the usual GEMM: the WEIGHT rows are the M = 128 side
// of tcgen05.mma and the token rows the N side (32..256).  A decode batch of a few tokens then
// still fills the 128 tensor-memory lanes, and one kernel serves 2-token decode, expert-routed
// MoE batches and 4096-token prefill.
//
//   warps 0-3   epilogue: tcgen05.ld (lane = weight row, column = token), stores transposed
//               into C (32 lanes = 32 consecutive output columns of one token)
//   warp 4      TMA producer: one (64 x NT) box of x16 per stage into shared memory
//   warp 5      MMA issuer: 4 x tcgen05.mma.cta_group::1.kind::f16 (M128, N = NT, K16) per
//               stage, A from tensor memory, B through a shared-memory descriptor
//   warps 6-13  weight decoders: warp w owns the 32 tensor-memory lanes (= weight rows) of its
//               quadrant w % 4 and one half of every 64-value K block; per K block a thread
//               writes its 32 fp16 values as 16 packed columns of its lane
// Tensor memory (512 columns): the accumulators in columns 0..255 (two of NT <= 128 columns,
// alternating so the epilogue overlaps the next tile, or one of 256), the weight ring in
// columns 256..511 (8 stages x 32 columns).  Expert batches whose experts hold a little more
// than 256 rows take token tiles of 320 or 384 rows instead (one accumulator in columns 0..nt-1,
// two MMAs per K step, the ring in the columns after it): a second, nearly empty 256-row tile
// would repeat the whole weight decoding for a handful of rows.  A stage is "full" after nine arrivals (eight
// decoder warps + the TMA transaction); tcgen05.commit releases it.  All waits are
// time-limited; a time-out ends every role and is reported in the status word.
//
// Small token counts with few weight rows would leave most SMs idle, so the K range of an
// output tile can be split over several CTAs.  Each split stores its fp32 partial tile; per
// 32-row slice the warp that arrives last at the slice's counter adds the partials in split
// order (deterministic) and writes C.  The counters are zeroed by the activation-preparation
// kernel of the same call.
#include "common.cuh"
#include "formats.cuh"
#include "host.h"
#include "tcgen05.cuh"

namespace lsg {

using namespace tc;

namespace {

constexpr int WM = 128;                  // weight rows per tile
constexpr int kDecWarps = 8;
constexpr int kFusedThreads = (6 + kDecWarps) * 32;
constexpr int kMaxStages = 8;               // weight ring in tensor memory: 8 x 32 columns
constexpr int kTmemCols = 512;
constexpr int kAColBase = 256;              // first column of the weight ring
constexpr int kAColsPerStage = BK / 2;      // 64 fp16 of a row = 32 packed columns
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kRawSlotBytes = kDecThreads * 16;     // 16 packed bytes per decoder thread and K block (Q4_K)
constexpr int kHdrRingBytes = 4 * kDecThreads * 16; // block headers of four consecutive 256-value blocks, per thread
constexpr int kTabTiles = 340;                      // grouped calls: tile table copied to shared memory (expert, first row, end row)
constexpr int kTabBytes = kTabTiles * 12 + 16;

struct FusedArgs {
    const uint8_t* W;             // dense: packed rows
    const void* const* B_ptrs;    // grouped: per-expert packed matrices
    const void* const* B_ptrs2;   // optional second set (same shape): weight tiles from split_wt on come
    int split_wt;                 //   from it and their outputs land col2_off columns further right
    int col2_off;
    long long row_bytes;
    void* C;
    int ldc;
    int out_dtype;
    int K, N, M;
    int nt;                       // token rows per tile: 32, 64, 128, 256, 320 or 384
    int tile_rows;                // dense: rows per token tile (M shared evenly among its tiles, <= nt)
    int box_rows;                 // rows of one TMA box of the token tile (nt, or 64 above 256)
    int a_col_base;               // first tensor-memory column of the weight ring (256, or nt above 256)
    int n_wtiles;                 // ceil(N / 128)
    int t_tiles;                  // dense: ceil(M / nt); grouped: capacity of the tile map
    const int* tile_expert;
    const int* tile_mstart;
    const int32_t* expert_offsets;
    int stages;
    int raw_depth;                // K blocks of packed weights in flight per decoder (0: none)
    int raw_bytes;                // shared memory of that ring
    int ksplit;                   // CTAs per output tile along K
    int kb_per_split;             // K blocks per split
    float* partial;               // [items][ksplit][128][nt] fp32, only with ksplit > 1
    unsigned int* counters;       // [tiles][4 epilogue warps], zero on entry
    const float* row_scale;       // optional per-token output scale (the unquantized-activation route)
    void* const* C_ptrs;          // optional: n_out output matrices (this GPU's and its peers'); every
    int n_out;                    //   element is stored into each of them (GEMM + all-gather)
    int col_off;                  // column offset of this call's N columns inside the output rows
    unsigned int* status;
#ifdef LSG_TCF_EXP
    int dbg;
#endif
#ifdef LSG_TCF_TRACE
    unsigned long long* trace;   // [grid][16] cycle sums per role
#endif
};
// Knock-out switches for timing experiments, only in builds with -DLSG_TCF_EXP (the shipped
// library has none): environment variable LSG_TCF_EXP = sum of 1 (no epilogue stores), 2 (no
// token-tile loads), 4 (no weight decoding), 8 (no epilogue at all).  Results are garbage then.
#ifdef LSG_TCF_EXP
#define TCF_DBG(a, bit) (((a).dbg & (bit)) != 0)
#else
#define TCF_DBG(a, bit) false
#endif

// Where the roles spend their time, only in builds with -DLSG_TCF_TRACE: cycles summed per CTA
// into trace[blockIdx.x * 16 + slot] by one lane of each role.  Slots: 0 MMA waits for a full
// stage, 1 MMA waits for a free accumulator, 2 MMA role total, 3 decoder (warp 6) waits for a
// free stage, 4 decoder total, 5 TMA waits for a free stage, 6 TMA total, 7 epilogue (warp 0)
// waits for the accumulator, 8 epilogue total, 9 items, 10 K blocks.
#ifdef LSG_TCF_TRACE
#define TCF_T0() const long long tcf_t0 = clock64(); long long tcf_w0 = 0, tcf_w1 = 0, tcf_n0 = 0, tcf_n1 = 0
#define TCF_ADD(slot, expr)                                                                                  \
    do {                                                                                                     \
        if (a.trace) a.trace[blockIdx.x * 16 + (slot)] += static_cast<unsigned long long>(expr);           \
    } while (0)
// every lane times the statement and sums in a register (no divergence, no memory traffic inside
// the loops); one lane adds the sums to the trace when its role ends
#define TCF_TIMED(which, stmt)                                                                               \
    do {                                                                                                     \
        const long long tcf_a = clock64();                                                                   \
        stmt;                                                                                                \
        tcf_w##which += clock64() - tcf_a;                                                                   \
    } while (0)
#define TCF_COUNT(which, n) tcf_n##which += (n)
#else
#define TCF_T0()
#define TCF_ADD(slot, expr)
#define TCF_TIMED(which, stmt) stmt
#define TCF_COUNT(which, n)
#endif

// Eight 32-bit columns of this thread's tensor-memory lane (the warp's lane quadrant).
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
                 "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D[tmem] (+)= A[tmem] * B[smem]: A is M x 16 fp16, row m in lane m, two values per column.
__device__ __forceinline__ void tc_mma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// ---------------------------------------------------------------------------
// Weight decoders.  load() fetches what thread (row, half h) needs for K block kb into
// registers; emit() turns it into 32 fp16 values (four 16-byte chunks, K order).
// ---------------------------------------------------------------------------
template <int T>
struct DecGeneric {
    // Generic decoder: no register staging, the packed bytes are read while decoding.
    struct Regs {
        const uint8_t* blk;
        int c;
    };
    __device__ static __forceinline__ Regs load(const uint8_t* row, int kb, int h, int K) {
        using F = Fmt<T>;
        Regs r;
        const int k0 = kb * BK + 32 * h;
        if (row == nullptr || k0 >= K) {
            r.blk = nullptr;
            r.c = 0;
        } else if (F::VALS == 256) {
            r.blk = row + static_cast<long long>(k0 >> 8) * F::BYTES;
            r.c = (k0 >> 5) & 7;
        } else {
            r.blk = row + static_cast<long long>(k0 >> 5) * F::BYTES;
            r.c = 0;
        }
        return r;
    }
    __device__ static __forceinline__ void emit(const Regs& r, int, uint4 (&out)[4]) {
        if (r.blk == nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) out[j] = make_uint4(0, 0, 0, 0);
            return;
        }
        float v[32];
        dequant_chunk32<T>(r.blk, r.c, v);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            out[j] = make_uint4(pack_h2(v[8 * j], v[8 * j + 1]), pack_h2(v[8 * j + 2], v[8 * j + 3]),
                                pack_h2(v[8 * j + 4], v[8 * j + 5]), pack_h2(v[8 * j + 6], v[8 * j + 7]));
    }
};

// Work item -> tile coordinates.  Items are ordered weight tile fastest, then K split, then
// token tile, so CTAs running together share a token tile (and, grouped, an expert).
struct Item {
    int tt, wt, ks;
    int expert;       // -1 dense
    int mstart, mend;
    bool live;
};

__device__ __forceinline__ Item decode_item(const FusedArgs& a, int w, const int* tab) {
    Item it;
    it.wt = w % a.n_wtiles;
    const int rest = w / a.n_wtiles;
    it.ks = rest % a.ksplit;
    it.tt = rest / a.ksplit;
    it.expert = -1;
    it.mstart = it.tt * a.tile_rows;
    it.mend = min(a.M, it.mstart + a.tile_rows);
    it.live = true;
    if (a.tile_expert) {
        if (tab) {   // the CTA's copy of the tile map: no dependent global loads per item
            it.expert = tab[3 * it.tt];
            it.mstart = tab[3 * it.tt + 1];
            it.mend = tab[3 * it.tt + 2];
            it.live = it.expert >= 0;
            return it;
        }
        const int e = a.tile_expert[it.tt];
        it.expert = e;
        it.live = e >= 0;
        if (it.live) {
            // never past the rows the caller holds, whatever the offsets say
            it.mstart = min(a.tile_mstart[it.tt], a.M);
            it.mend = min(a.expert_offsets[e + 1], a.M);
            // balanced tile maps: the expert's tiles share its rows evenly
            const int m = it.mend - min(a.expert_offsets[e], a.M);
            it.mend = min(it.mend, it.mstart + balanced_tile_rows(m, a.nt));
        }
    }
    return it;
}

// Ring position shared by the roles: stage index and how often the ring has wrapped.
struct Ring {
    int s;
    uint32_t lap;
    int n;
    __device__ __forceinline__ void advance() {
        if (++s == n) {
            s = 0;
            ++lap;
        }
    }
};

// What a decoder thread needs to publish a K block: barriers, its tensor-memory lane base
// (lane quadrant of the warp) and the status word.
struct DecCtx {
    uint64_t* full;
    uint64_t* empty;
    uint32_t tmem_a;        // tensor-memory address of column kAColBase in this warp's lane quadrant
    unsigned int* status;
    uint32_t hint;
#ifdef LSG_TCF_TRACE
    mutable long long waited;          // cycles this thread waited for a free stage
#endif
};

// Waits until the stage is free, stores 2 x 8 packed columns of this thread's lane (column
// offsets c0 and c1 inside the stage), and arrives on the stage's "full" barrier.
__device__ __forceinline__ bool publish_stage(const DecCtx& c, Ring& ring, const uint32_t* lo, uint32_t c0,
                                              const uint32_t* hi, uint32_t c1) {
#ifdef LSG_TCF_TRACE
    const long long tw = clock64();
#endif
    if (ring.lap > 0 &&
        !__all_sync(0xffffffffu, mbar_wait_bounded(&c.empty[ring.s], (ring.lap - 1) & 1, c.status, kDevWaitEmpty, c.hint)))
        return false;
#ifdef LSG_TCF_TRACE
    c.waited += clock64() - tw;
#endif
    tc_fence_after();  // the MMAs that last read this stage are ordered before the stores
    const uint32_t col = c.tmem_a + static_cast<uint32_t>(ring.s * kAColsPerStage);
    tmem_st8(col + c0, lo);
    tmem_st8(col + c1, hi);
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (elect_one()) mbar_arrive(&c.full[ring.s]);
    ring.advance();
    return true;
}

// One item's K range for one decoder thread: row `row`, half `h` (32 consecutive values) of
// every 64-value K block, any type, any alignment.  Three register sets rotate by name (the
// loop body is written out three times): copying a set whose loads are still in flight would
// wait for them and collapse the lookahead.  Lookahead loads past the end re-read the last
// block instead of being skipped, so no load is conditional.  Returns false after a time-out.
template <class D>
__device__ __forceinline__ bool decode_rows(const DecCtx& c, Ring& ring, const uint8_t* row, int kb0, int kb1,
                                            int h, int K) {
    const int last = kb1 - 1;
    typename D::Regs b0 = D::load(row, kb0, h, K);
    typename D::Regs b1 = D::load(row, min(kb0 + 1, last), h, K);
    typename D::Regs b2;
    auto step = [&](const typename D::Regs& cur, int kb) -> bool {
        uint4 out[4];
        D::emit(cur, (kb & 3) * 2 + h, out);
        const uint32_t o[16] = {out[0].x, out[0].y, out[0].z, out[0].w, out[1].x, out[1].y, out[1].z, out[1].w,
                                out[2].x, out[2].y, out[2].z, out[2].w, out[3].x, out[3].y, out[3].z, out[3].w};
        return publish_stage(c, ring, o, 16u * h, o + 8, 16u * h + 8u);
    };
    for (int kb = kb0; kb < kb1; kb += 3) {
        b2 = D::load(row, min(kb + 2, last), h, K);
        if (!step(b0, kb)) return false;
        if (kb + 1 >= kb1) break;
        b0 = D::load(row, min(kb + 3, last), h, K);
        if (!step(b1, kb + 1)) return false;
        if (kb + 2 >= kb1) break;
        b1 = D::load(row, min(kb + 4, last), h, K);
        if (!step(b2, kb + 2)) return false;
    }
    return true;
}

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Q4_K rows through a private shared-memory ring: every decoder thread copies the 16 bytes
// of nibbles it decodes per K block (and the 16-byte block header once per four K blocks)
// with cp.async, DEPTH K blocks ahead of where it decodes, so the lookahead costs no
// registers and the ring needs no synchronisation between threads.
//
// A 144-byte block is {fp16 d, fp16 dmin, 12 bytes of 6-bit scales/mins, 128 bytes of
// nibbles} (csrc/formats/q4k_format.h:112-133); K block p of the block is nibble pair p: the
// low nibbles of qs[32p..32p+31] are values 64p..64p+31 (sub-block 2p), the high nibbles
// values 64p+32..64p+63 (sub-block 2p+1).  Thread half hb owns bytes 16hb..16hb+15 of the
// pair: values 64p+16hb+(0..15) from the low nibbles and 64p+32+16hb+(0..15) from the high
// ones, i.e. packed columns 8hb..8hb+7 and 16+8hb..16+8hb+7 of the stage.  The value is
// d*sc*q - dmin*mn with the 6-bit sc, mn of the sub-block (csrc/formats/kquant_common.h:36-46);
// d*sc and dmin*mn are formed as fp16 products (one rounding of an exact product, the same
// number fp32 arithmetic followed by a conversion gives) and the value by one fp16 fma.
//
// Requires 16-byte aligned rows and a K range that starts and ends on a 256-value block.
// Returns false after a wait timed out.
template <int DEPTH>
__device__ __forceinline__ bool decode_rows_q4k(const DecCtx& c, Ring& ring, const uint8_t* row, int kb0, int kb1,
                                                int hb, uint8_t* raw, int dec_tid) {
    const uint32_t q_ring = smem_u32(raw) + static_cast<uint32_t>(dec_tid * 16);                          // + slot * kRawSlotBytes
    const uint32_t h_ring = smem_u32(raw) + DEPTH * kRawSlotBytes + static_cast<uint32_t>(dec_tid * 16);  // + (blk & 3) * kRawSlotBytes
    const uint8_t* src = row + static_cast<long long>(kb0 >> 2) * 144;  // block of the next copy
    int issue_kb = kb0;
    auto issue = [&](int slot) {
        if (issue_kb < kb1) {
            const int p = issue_kb & 3;
            cp_async16(q_ring + slot * kRawSlotBytes, src + 16 + p * 32 + 16 * hb);
            if (p == 0) cp_async16(h_ring + ((issue_kb >> 2) & 3) * kRawSlotBytes, src);
            if (p == 3) src += 144;
        }
        ++issue_kb;
        cp_async_commit();  // one group per K block, empty past the end, so the count below is fixed
    };
#pragma unroll
    for (int i = 0; i < DEPTH; ++i) issue(i);

    const __half2 k1024 = __float2half2_rn(1024.0f);
    int slot = 0;
    // The nibbles of K block kb are read from the ring one iteration ahead of their use, so
    // the shared-memory latency hides behind the arithmetic of block kb - 1; the wait for a
    // free stage comes after the arithmetic, right before the stores.
    cp_async_wait<DEPTH - 1>();
    uint4 q = lds128(q_ring);
    for (int kb = kb0; kb < kb1; kb += 4) {
        // ---- once per 256-value block: all eight (scale, min) pairs ----
        // (the header arrived with the group of the block's first K block, already waited for)
        const uint4 hdr = lds128(h_ring + ((kb >> 2) & 3) * kRawSlotBytes);
        // bytes of sc[0..3], sc[4..7], mn[0..3], mn[4..7]
        const uint32_t scw[2] = {hdr.y & 0x3F3F3F3Fu, (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u)};
        const uint32_t mnw[2] = {hdr.z & 0x3F3F3F3Fu, ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u)};
        // (d, -dmin) as a half2
        const uint32_t dd = hdr.x ^ 0x80000000u;
        const __half2 d_ndmin = *reinterpret_cast<const __half2*>(&dd);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            // the next K block's copies have landed (its group is the oldest but one): fetch
            // its nibbles now; past the end this re-reads a finished slot and is not used
            const int nslot = (slot + 1 == DEPTH) ? 0 : slot + 1;
            cp_async_wait<DEPTH - 2>();
            q = lds128(q_ring + nslot * kRawSlotBytes);
            // sub-blocks 2p (low nibbles) and 2p+1 (high): half2 (sc, mn) -> (d*sc, -dmin*mn)
            const uint32_t pl = __byte_perm(scw[p >> 1], mnw[p >> 1], (p & 1) ? 0x0062 : 0x0040);
            const uint32_t ph = __byte_perm(scw[p >> 1], mnw[p >> 1], (p & 1) ? 0x0073 : 0x0051);
            uint32_t sl = __byte_perm(pl, 0x64646464u, 0x4140), sh = __byte_perm(ph, 0x64646464u, 0x4140);
            const __half2 sml = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&sl), k1024), d_ndmin);
            const __half2 smh = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&sh), k1024), d_ndmin);
            const __half2 ds_l = __low2half2(sml), nms_l = __high2half2(sml);
            const __half2 ds_h = __low2half2(smh), nms_h = __high2half2(smh);
            uint32_t lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t nl = w[i] & 0x0F0F0F0Fu, nh = (w[i] >> 4) & 0x0F0F0F0Fu;
                // bytes -> fp16 1024 + q by placing each under the exponent byte 0x64
                uint32_t a0 = __byte_perm(nl, 0x64646464u, 0x4140), a1 = __byte_perm(nl, 0x64646464u, 0x4342);
                uint32_t b0 = __byte_perm(nh, 0x64646464u, 0x4140), b1 = __byte_perm(nh, 0x64646464u, 0x4342);
                const __half2 x0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&a0), k1024), ds_l, nms_l);
                const __half2 x1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&a1), k1024), ds_l, nms_l);
                const __half2 y0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&b0), k1024), ds_h, nms_h);
                const __half2 y1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&b1), k1024), ds_h, nms_h);
                lo[2 * i] = *reinterpret_cast<const uint32_t*>(&x0);
                lo[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&x1);
                hi[2 * i] = *reinterpret_cast<const uint32_t*>(&y0);
                hi[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&y1);
            }
            if (!publish_stage(c, ring, lo, 8u * hb, hi, 16u + 8u * hb)) return false;
            issue(slot);
            slot = nslot;
        }
    }
    cp_async_wait<0>();
    return true;
}

template <int T>
__global__ void __launch_bounds__(kFusedThreads, 1)
tc_fused_kernel(const __grid_constant__ CUtensorMap tmX, const FusedArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int stage_bytes = a.nt * 128;              // one (64 x NT) fp16 token tile
    uint8_t* raw = smem + a.stages * stage_bytes;   // packed-weight ring of the staged decoders
    int* tab_mem = reinterpret_cast<int*>(raw + a.raw_bytes);   // kTabBytes
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + a.raw_bytes + kTabBytes);
    uint64_t* empty = full + kMaxStages;
    uint64_t* acc_full = empty + kMaxStages;  // [2]
    uint64_t* acc_empty = acc_full + 2;       // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nacc = a.nt > 128 ? 1 : 2;   // accumulators in columns 0..255

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&full[s], kDecWarps + 1);
            mbar_init(&empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 5) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    pdl_wait_prior();  // x16, the tile map and the zeroed counters come from earlier kernels

    // Grouped calls: every role looks every item's tile up, and three dependent global loads per
    // look-up sit in front of each item's first copy, decode and MMA.  The tile map is small, so
    // the CTA resolves it once into shared memory.
    const int* tab = nullptr;
    if (a.tile_expert && a.t_tiles <= kTabTiles) {
        for (int t = threadIdx.x; t < a.t_tiles; t += kFusedThreads) {
            const int e = a.tile_expert[t];
            int ms = 0, me = 0;
            if (e >= 0) {
                ms = min(a.tile_mstart[t], a.M);
                me = min(a.expert_offsets[e + 1], a.M);
                const int m = me - min(a.expert_offsets[e], a.M);
                me = min(me, ms + balanced_tile_rows(m, a.nt));
            }
            tab_mem[3 * t] = e;
            tab_mem[3 * t + 1] = ms;
            tab_mem[3 * t + 2] = me;
        }
        __syncthreads();
        tab = tab_mem;
    }

    const int kblocks_all = (a.K + BK - 1) / BK;
    const int total = a.t_tiles * a.ksplit * a.n_wtiles;
    const uint32_t hint = 2000u;  // suspend-time hint of the barrier waits, ns

    if (warp == 4) {
        // ------------------------------ TMA producer (x16 tiles) ------------------
        // The whole warp walks the loop, one elected lane issues the copies (see the MMA issuer).
        {
            TCF_T0();
            Ring ring = {0, 0u, a.stages};
            bool ok = true;
            for (int w = blockIdx.x; w < total && ok && !*abort_flag; w += gridDim.x) {
                const Item im = decode_item(a, w, tab);
                if (!im.live) continue;
                const int kb0 = im.ks * a.kb_per_split;
                const int kb1 = min(kblocks_all, kb0 + a.kb_per_split);
                const int live_rows = min(a.nt, im.mend - im.mstart);
                const int live_boxes = max(1, (live_rows + a.box_rows - 1) / a.box_rows);
                for (int kb = kb0; kb < kb1; ++kb) {
                    TCF_TIMED(0, if (ring.lap > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty[ring.s], (ring.lap - 1) & 1, a.status, kDevWaitEmpty, hint)));
                    if (!ok) break;
                    if (elect_one()) {
                        if (TCF_DBG(a, 2)) {
                            mbar_arrive(&full[ring.s]);
                        } else {
                            // only the boxes that hold live token rows: the rest of the stage is never read,
                            // and every byte copied takes shared-memory bandwidth from the MMA's operand reads
                            mbar_arrive_expect_tx(&full[ring.s], static_cast<uint32_t>(live_boxes * a.box_rows * 128));
                            for (int r0 = 0; r0 < live_boxes * a.box_rows; r0 += a.box_rows)
                                tma_load_2d(smem + ring.s * stage_bytes + r0 * 128, &tmX, kb * BK, im.mstart + r0, &full[ring.s]);
                        }
                    }
                    __syncwarp();
                    ring.advance();
                }
            }
            if (!ok) *abort_flag = 1;
            if (lane == 0) { TCF_ADD(5, tcf_w0); TCF_ADD(6, clock64() - tcf_t0); }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer --------------------------------
        // The whole warp walks the loop so that descriptors and addresses stay warp-uniform
        // values; one elected lane issues the tensor-core instructions.
        TCF_T0();
        Ring ring = {0, 0u, a.stages};
        int tile_i = 0, ab = 0;
        uint32_t acc_lap = 0;  // how often the accumulator set has been cycled through
        bool ok = true;
        for (int w = blockIdx.x; w < total && ok && !*abort_flag; w += gridDim.x) {
            const Item im = decode_item(a, w, tab);
            if (!im.live) continue;
            const int kb0 = im.ks * a.kb_per_split;
            const int kb1 = min(kblocks_all, kb0 + a.kb_per_split);
            TCF_TIMED(1, if (acc_lap > 0) ok = __all_sync(0xffffffffu, mbar_wait_bounded(&acc_empty[ab], (acc_lap - 1) & 1, a.status, kDevWaitTmem, hint)));
            if (!ok) break;
            TCF_COUNT(0, 1); TCF_COUNT(1, kb1 - kb0);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + ab * a.nt;
            // N of the instruction follows the token rows that are really in the tile (a multiple
            // of 16): the ragged last tile of an expert costs tensor time for its rows only
            const int live = min(a.nt, im.mend - im.mstart);
            const int live16 = max(16, (live + 15) & ~15);
            // more than 256 rows take two instructions per K step; split evenly (a short second
            // instruction would cost its issue time, not its tensor time)
            const int n1 = live16 <= 256 ? live16 : ((live16 >> 1) + 15) & ~15, n2 = live16 - n1;
            const uint32_t idesc = idesc_f16(WM, n1);
            const uint32_t idesc2 = idesc_f16(WM, max(16, n2));
            for (int kb = kb0; kb < kb1; ++kb) {
                TCF_TIMED(0, ok = __all_sync(0xffffffffu, mbar_wait_bounded(&full[ring.s], ring.lap & 1, a.status, kDevWaitFull, hint)));
                if (!ok) break;
                tc_fence_after();
                const uint64_t xdesc = smem_desc_sw128(smem_u32(smem + ring.s * stage_bytes));
                const uint64_t xdesc2 = smem_desc_sw128(smem_u32(smem + ring.s * stage_bytes + n1 * 128));
                const uint32_t a_tmem = tmem_base + a.a_col_base + ring.s * kAColsPerStage;
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        tc_mma_f16_ta(d_tmem, a_tmem + 8 * k, xdesc + 2 * k, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
                        if (n2 > 0)
                            tc_mma_f16_ta(d_tmem + n1, a_tmem + 8 * k, xdesc2 + 2 * k, idesc2, (kb != kb0 || k != 0) ? 1u : 0u);
                    }
                    tc_commit(&empty[ring.s]);
                }
                __syncwarp();
                ring.advance();
            }
            if (!ok) break;
            if (elect_one()) tc_commit(&acc_full[ab]);
            __syncwarp();
            ++tile_i;
            if (++ab == nacc) {
                ab = 0;
                ++acc_lap;
            }
        }
        if (!ok) *abort_flag = 1;
        if (lane == 0) { TCF_ADD(0, tcf_w0); TCF_ADD(1, tcf_w1); TCF_ADD(9, tcf_n0); TCF_ADD(10, tcf_n1); TCF_ADD(2, clock64() - tcf_t0); }
    } else if (warp >= 6) {
        // ------------------------------ weight decoders ---------------------------
        // warp -> lane quadrant (a warp may only touch tensor-memory lanes 32 * (warp % 4) ..),
        // and which half of each K block it decodes
        const int quad = warp & 3;
        const int half = (warp - 6) >> 2;
        const int r = quad * 32 + lane;          // weight row inside the tile
        const int dec_tid = threadIdx.x - 6 * 32;
        DecCtx ctx;
        ctx.full = full;
        ctx.empty = empty;
        ctx.tmem_a = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + a.a_col_base;
        ctx.status = a.status;
        ctx.hint = hint;
#ifdef LSG_TCF_TRACE
        ctx.waited = 0;
#endif
        TCF_T0();
        Ring ring = {0, 0u, a.stages};
        for (int w = blockIdx.x; w < total && !*abort_flag; w += gridDim.x) {
            const Item im = decode_item(a, w, tab);
            if (!im.live) continue;
            const int kb0 = im.ks * a.kb_per_split;
            const int kb1 = min(kblocks_all, kb0 + a.kb_per_split);
            const bool second = a.B_ptrs2 != nullptr && im.wt >= a.split_wt;
            const uint8_t* base = a.B_ptrs ? static_cast<const uint8_t*>((second ? a.B_ptrs2 : a.B_ptrs)[im.expert])
                                           : a.W;
            const int n = min((second ? im.wt - a.split_wt : im.wt) * WM + r, a.N - 1);
            const uint8_t* row = base ? base + static_cast<long long>(n) * a.row_bytes : nullptr;
            // The staged decoder copies 16-byte pieces; a matrix that is not 16-byte aligned goes
            // through the byte-wise generic decoder instead.  The choice is uniform over the CTA.
            bool ok;
            const bool aligned16 =
                ((reinterpret_cast<uintptr_t>(base) | static_cast<uintptr_t>(a.row_bytes)) & 15) == 0;
            if (TCF_DBG(a, 4)) {
                ok = true;
                for (int kb = kb0; kb < kb1 && ok; ++kb) {
                    if (ring.lap > 0)
                        ok = __all_sync(0xffffffffu, mbar_wait_bounded(&empty[ring.s], (ring.lap - 1) & 1, a.status,
                                                                       kDevWaitEmpty, hint));
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full[ring.s]);
                    ring.advance();
                }
            } else if (T == LSG_GGUF_Q4_K && a.raw_depth > 0 && row != nullptr && aligned16) {
                if (a.raw_depth == 8)
                    ok = decode_rows_q4k<8>(ctx, ring, row, kb0, kb1, half, raw, dec_tid);
                else
                    ok = decode_rows_q4k<4>(ctx, ring, row, kb0, kb1, half, raw, dec_tid);
            } else {
                ok = decode_rows<DecGeneric<T>>(ctx, ring, row, kb0, kb1, half, a.K);
            }
            if (!ok) {
                *abort_flag = 1;
                break;
            }
        }
#ifdef LSG_TCF_TRACE
        if (warp == 6 && lane == 0) { TCF_ADD(3, ctx.waited); TCF_ADD(4, clock64() - tcf_t0); }
#endif
    } else {
        // ------------------------------ epilogue (warps 0-3) ----------------------
        TCF_T0();
        int tile_i = 0, ab = 0;
        uint32_t acc_lap = 0;
        for (int w = blockIdx.x; w < total && !*abort_flag; w += gridDim.x) {
            const Item im = decode_item(a, w, tab);
            if (!im.live) continue;
            bool landed = false;
            TCF_TIMED(0, landed = __all_sync(0xffffffffu, mbar_wait_bounded(&acc_full[ab], acc_lap & 1, a.status, kDevWaitMma, hint)));
            if (!landed) {
                *abort_flag = 1;
                break;
            }
            tc_fence_after();
            const bool second = a.B_ptrs2 != nullptr && im.wt >= a.split_wt;
            const int n_local = (second ? im.wt - a.split_wt : im.wt) * WM + warp * 32 + lane;
            const bool n_ok = n_local < a.N;
            const int n = n_local + (second ? a.col2_off : 0) + a.col_off;   // this thread's output column
            const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + ab * a.nt;

            if (a.ksplit == 1) {
#pragma unroll 1
                for (int c = 0; c < a.nt; c += 32) {
                    if (im.mstart + c >= im.mend) break;  // warp-uniform: no token rows left in this tile
                    if (TCF_DBG(a, 8)) break;
                    uint32_t v[32];
                    tmem_ld32(t_lane + c, v);
                    if (n_ok && a.n_out == 0 && !a.row_scale && a.out_dtype == LSG_DTYPE_BF16 && !TCF_DBG(a, 1)) {
                        // the common case on its own: one conversion and one 2-byte store per token row
                        const int rows = min(32, im.mend - (im.mstart + c));
                        uint16_t* dst = static_cast<uint16_t*>(a.C) + static_cast<size_t>(im.mstart + c) * a.ldc + n;
                        if (rows == 32) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                dst[static_cast<size_t>(i) * a.ldc] = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(v[i])));
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (i < rows)
                                    dst[static_cast<size_t>(i) * a.ldc] = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(v[i])));
                        }
                    } else if (n_ok && !TCF_DBG(a, 1)) {
                        const int rows = min(32, im.mend - (im.mstart + c));
                        if (a.row_scale) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (i < rows)
                                    v[i] = __float_as_uint(__uint_as_float(v[i]) * __ldg(a.row_scale + im.mstart + c + i));
                        }
                        const size_t o = static_cast<size_t>(im.mstart + c) * a.ldc + n;
                        const int n_out = a.n_out > 0 ? a.n_out : 1;
                        for (int po = 0; po < n_out; ++po) {
                            void* Cb = a.n_out > 0 ? a.C_ptrs[po] : a.C;
                            if (a.out_dtype == LSG_DTYPE_F32) {
                                float* dst = static_cast<float*>(Cb) + o;
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (i < rows) dst[static_cast<size_t>(i) * a.ldc] = __uint_as_float(v[i]);
                            } else {
                                uint16_t* dst = static_cast<uint16_t*>(Cb) + o;
                                const bool f16 = a.out_dtype == LSG_DTYPE_F16;
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    if (i < rows) {
                                        const float x = __uint_as_float(v[i]);
                                        dst[static_cast<size_t>(i) * a.ldc] =
                                            f16 ? __half_as_ushort(__float2half_rn(x))
                                                : __bfloat16_as_ushort(__float2bfloat16_rn(x));
                                    }
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
            } else {
                // Split K: park this split's fp32 tile [token][128 weight rows]; per 32-row
                // slice of the tile, the warp that arrives last at the slice's counter adds
                // the splits in order and writes C.  Each epilogue warp works alone, so no
                // CTA-wide barrier sits inside a loop that a time-out may leave.
                const int tile_id = im.tt * a.n_wtiles + im.wt;
                const size_t tile_elems = static_cast<size_t>(WM) * a.nt;
                float* mine = a.partial + (static_cast<size_t>(tile_id) * a.ksplit + im.ks) * tile_elems;
                const int live_rows = min(a.nt, im.mend - im.mstart);
#pragma unroll 1
                for (int c = 0; c < live_rows; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(t_lane + c, v);
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        mine[static_cast<size_t>(c + i) * WM + warp * 32 + lane] = __uint_as_float(v[i]);
                }
                tc_fence_before();
                __threadfence();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
                unsigned int prev = 0;
                if (lane == 0) prev = atomicAdd(&a.counters[tile_id * 4 + warp], 1u);
                prev = __shfl_sync(0xffffffffu, prev, 0);
                if (prev == static_cast<unsigned int>(a.ksplit - 1)) {
                    __threadfence();
                    const float* tile0 = a.partial + static_cast<size_t>(tile_id) * a.ksplit * tile_elems;
                    if (n_ok) {
                        // 32 token rows at a time: the loads of one split are independent and all
                        // in flight together; the splits are added in order.
                        for (int i0 = 0; i0 < live_rows; i0 += 32) {
                            float acc[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
                            const float* col = tile0 + static_cast<size_t>(i0) * WM + warp * 32 + lane;
                            for (int sp = 0; sp < a.ksplit; ++sp) {
                                float v[32];
#pragma unroll
                                for (int i = 0; i < 32; ++i)
                                    v[i] = (i0 + i < live_rows) ? __ldcg(col + sp * tile_elems + static_cast<size_t>(i) * WM)
                                                                : 0.0f;
#pragma unroll
                                for (int i = 0; i < 32; ++i) acc[i] += v[i];
                            }
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                if (i0 + i < live_rows) {
                                    if (a.row_scale) acc[i] *= __ldg(a.row_scale + im.mstart + i0 + i);
                                    const size_t o = static_cast<size_t>(im.mstart + i0 + i) * a.ldc + n;
                                    const int n_out = a.n_out > 0 ? a.n_out : 1;
                                    for (int po = 0; po < n_out; ++po) {
                                        void* Cb = a.n_out > 0 ? a.C_ptrs[po] : a.C;
                                        if (a.out_dtype == LSG_DTYPE_F32)
                                            static_cast<float*>(Cb)[o] = acc[i];
                                        else if (a.out_dtype == LSG_DTYPE_F16)
                                            static_cast<uint16_t*>(Cb)[o] = __half_as_ushort(__float2half_rn(acc[i]));
                                        else
                                            static_cast<uint16_t*>(Cb)[o] = __bfloat16_as_ushort(__float2bfloat16_rn(acc[i]));
                                    }
                                }
                            }
                        }
                    }
                }
            }
            ++tile_i;
            if (++ab == nacc) {
                ab = 0;
                ++acc_lap;
            }
        }
        if (warp == 0 && lane == 0) { TCF_ADD(7, tcf_w0); TCF_ADD(8, clock64() - tcf_t0); }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Activation preparation: bf16 -> fp16 of the Q8_1 round trip (d_h * rn(x / d), the values
// the integer kernels multiply by), plus zeroing of the split-K tile counters.
//
// SWIGLU = false: x[rows, K].  With a permutation the rows are gathered on the way in: row i
// of the output is token perm[i] / top_k of x (the permute pass of a MoE layer folded in).
// SWIGLU = true: x = gu[rows, 2K] holds gate | up; per element
//   act = bf16( silu(g) * u )  with silu(g) = g / (1 + exp(-g)) in fp32
// (what a caller computing the activation in fp32 and storing bf16 gets), then the round trip.
//
// Four lanes per 32-value block, eight values (one 16-byte vector) each.  The thread block is
// (vectors of a row, rows); every thread handles RB rows, so RB (2 RB with SwiGLU) independent
// loads are in flight per thread and no index needs a division.  Grouped callers may hold
// fewer rows than the buffer they pass: the row count then lives on the device (live_rows).
// ---------------------------------------------------------------------------
template <int RB, bool SWIGLU>
__global__ void __launch_bounds__(256)
x_prep_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ out, int rows, int vpr,
              unsigned int* __restrict__ counters, int n_counters, const int32_t* __restrict__ live_rows,
              const int32_t* __restrict__ perm, int top_k, const int32_t* __restrict__ first_row) {
    const unsigned lanes = __activemask();   // a block of K/8 x rows threads may end in a partial warp
    pdl_launch_dependents();
    pdl_wait_prior();
    const int tx = threadIdx.x, ty = threadIdx.y;
    if (counters) {
        const int nthreads = blockDim.x * blockDim.y;
        const long long stride = static_cast<long long>(gridDim.x) * gridDim.y * nthreads;
        for (long long i = (static_cast<long long>(blockIdx.y) * gridDim.x + blockIdx.x) * nthreads + ty * blockDim.x + tx;
             i < n_counters; i += stride)
            counters[i] = 0;
    }
    const int live = live_rows ? min(rows, __ldg(live_rows)) : rows;
    if (static_cast<int>(blockIdx.x * (blockDim.y * RB)) >= live) return;   // the whole block lies past the live rows
    // ... or before the first row any expert of this call owns (a call on a group of experts)
    if (first_row && static_cast<int>((blockIdx.x + 1) * (blockDim.y * RB)) <= __ldg(first_row)) return;
    const int v = blockIdx.y * blockDim.x + tx;
    const int rbase = blockIdx.x * (blockDim.y * RB) + ty;
    const int ld_in = SWIGLU ? 2 * vpr : vpr;
    const uint4* xin = reinterpret_cast<const uint4*>(x);
    uint4 g[RB], u[RB];
    bool ok[RB];
#pragma unroll
    for (int j = 0; j < RB; ++j) {
        const int r = rbase + j * blockDim.y;
        ok[j] = v < vpr && r < live;
        g[j] = make_uint4(0, 0, 0, 0);
        u[j] = make_uint4(0, 0, 0, 0);
        if (ok[j]) {
            const int sr = perm ? __ldg(perm + r) / top_k : r;
            const uint4* src = xin + static_cast<size_t>(sr) * ld_in + v;
            g[j] = __ldg(src);
            if (SWIGLU) u[j] = __ldg(src + vpr);
        }
    }
#pragma unroll
    for (int j = 0; j < RB; ++j) {
        const uint32_t gw[4] = {g[j].x, g[j].y, g[j].z, g[j].w}, uw[4] = {u[j].x, u[j].y, u[j].z, u[j].w};
        float val[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const float a = __uint_as_float(hh ? (gw[i] & 0xFFFF0000u) : (gw[i] << 16));
                if (SWIGLU) {
                    const float b = __uint_as_float(hh ? (uw[i] & 0xFFFF0000u) : (uw[i] << 16));
                    val[2 * i + hh] = __bfloat162float(__float2bfloat16_rn((a / (1.0f + expf(-a))) * b));
                } else {
                    val[2 * i + hh] = a;
                }
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(val[i]));
        amax = fmaxf(amax, __shfl_xor_sync(lanes, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(lanes, amax, 2));
        const float d = amax / 127.0f;
        const float rcp = (amax == 0.0f) ? 0.0f : 1.0f / d;
        const float dh = __half2float(__float2half(d));
        uint32_t pk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float r2[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                // same integer as rn(fl(x / d)): the product with the reciprocal only differs
                // next to a half-integer, and there the true quotient decides
                r2[hh] = dh * q8_round_f(val[2 * i + hh], d, rcp);
            }
            pk[i] = pack_h2(r2[0], r2[1]);
        }
        if (ok[j]) {
            const int r = rbase + j * blockDim.y;
            reinterpret_cast<uint4*>(out)[static_cast<size_t>(r) * vpr + v] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
}

// rows x K values (K a multiple of 32).  The block is (min(K/8, 256) vectors, 256 / that rows).
template <bool SWIGLU>
int launch_x_prep(const __nv_bfloat16* x, __half* out, long long rows, int K, unsigned int* counters, int n_counters,
                  const int32_t* live_rows, const int32_t* perm, int top_k, cudaStream_t s,
                  const int32_t* first_row = nullptr) {
    if (rows <= 0 || rows > 0x7fffffffll) return rows == 0 ? LSG_OK : fail(LSG_ERR_UNSUPPORTED, "activation preparation: too many rows");
    const int vpr = K / 8;
    const int bx = vpr < 256 ? vpr : 256;
    const int by = 256 / bx > 0 ? 256 / bx : 1;
    const int gy = (vpr + bx - 1) / bx;
    // four rows per thread once there are enough rows to fill the GPU that way
    const bool rb4 = rows >= 4ll * by * 2 * sm_count();
    const int rows_per_block = by * (rb4 ? 4 : 1);
    const unsigned gx = static_cast<unsigned>((rows + rows_per_block - 1) / rows_per_block);
    if (rb4)
        LSG_CUDA_TRY(launch_kernel(x_prep_kernel<4, SWIGLU>, dim3(gx, gy), dim3(bx, by), 0, s, true, x, out,
                                   static_cast<int>(rows), vpr, counters, n_counters, live_rows, perm, top_k, first_row));
    else
        LSG_CUDA_TRY(launch_kernel(x_prep_kernel<1, SWIGLU>, dim3(gx, gy), dim3(bx, by), 0, s, true, x, out,
                                   static_cast<int>(rows), vpr, counters, n_counters, live_rows, perm, top_k, first_row));
    return LSG_OK;
}

// bf16 activation rows -> fp16 scaled by a power of two per row: the row's largest magnitude
// lands in [2^14, 2^15), out[m,k] = x[m,k] * 2^-e_m exactly, scale[m] = 2^e_m for the epilogue.
// One warp per row.  Rows of zeros (or with no finite value) keep scale 1.
__global__ void __launch_bounds__(256)
x_rows_to_f16_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ out, float* __restrict__ scale, int M,
                     int K, unsigned int* __restrict__ counters, int n_counters) {
    pdl_launch_dependents();
    pdl_wait_prior();
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n_counters; i += gridDim.x * 256) counters[i] = 0;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K);
    const int nvec = K / 8;
    uint32_t amax_bits = 0;  // largest |x| as bf16 bits in the upper half (monotonic in magnitude)
    for (int i = lane; i < nvec; i += 32) {
        const uint4 v = __ldg(src + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            amax_bits = max(amax_bits, (w[j] << 16) & 0x7FFF0000u);
            amax_bits = max(amax_bits, w[j] & 0x7FFF0000u);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, o));
    // exponent of the largest finite magnitude; shift it to 14
    int ex = static_cast<int>(amax_bits >> 23);        // biased fp32 exponent, 0..255
    int shift = (ex == 0 || ex == 255) ? 0 : (ex - 127) - 14;
    // keep both factors normal fp32 numbers
    shift = max(-100, min(100, shift));
    const float down = __uint_as_float(static_cast<uint32_t>(127 - shift) << 23);  // 2^-shift
    const float up = __uint_as_float(static_cast<uint32_t>(127 + shift) << 23);    // 2^shift
    if (lane == 0) scale[row] = up;
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * K);
    for (int i = lane; i < nvec; i += 32) {
        const uint4 v = __ldg(src + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            o[j] = pack_h2(__uint_as_float(w[j] << 16) * down, __uint_as_float(w[j] & 0xFFFF0000u) * down);
        dst[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

#ifdef LSG_TCF_TRACE
unsigned long long* g_tcf_trace = nullptr;   // [launch slot][148][16]
int g_tcf_trace_slots = 0, g_tcf_trace_launch = 0;
#endif

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

bool staged_decoder(int type) { return type == LSG_GGUF_Q4_K; }

struct Plan {
    int nt, box_rows, a_col_base, stages, raw_depth, raw_bytes, t_tiles, n_wtiles, ksplit, kb_per_split;
    size_t x_bytes, partial_bytes, counter_bytes;
    size_t total() const { return x_bytes + partial_bytes + counter_bytes; }
};

int pick_nt(long long rows_per_problem) {
    static const int force = [] {
        const char* e = getenv("LSG_TC_FUSED_DENSE_NT");
        return e ? atoi(e) : 0;
    }();
    if (force == 32 || force == 64 || force == 128 || force == 256 || force == 320 || force == 384) return force;
    if (rows_per_problem <= 32) return 32;
    if (rows_per_problem <= 64) return 64;
    if (rows_per_problem <= 128) return 128;
    // Every token tile repeats the decoding of the weights, so above 256 rows the height that
    // needs the fewest tiles wins; at equal count the lower one (more stages in shared memory).
    // Measured on 14336 x 4096 Q4_K: M = 4096 0.474 ms with 256-row tiles, 0.399 ms with 384.
    int best = 256;
    long long best_tiles = (rows_per_problem + 255) / 256;
    for (int nt : {320, 384}) {
        const long long tiles = (rows_per_problem + nt - 1) / nt;
        if (tiles < best_tiles) {
            best = nt;
            best_tiles = tiles;
        }
    }
    return best;
}

// rows: token rows of the whole call; t_tiles: dense tile count or the tile map's capacity.
Plan make_plan(long long rows, int nt, int t_tiles, int N, int K, bool allow_split, bool staged) {
    Plan p = {};
    p.nt = nt;
    const int stage_bytes = nt * 128;
    // packed-weight ring of the staged decoders, 8 K blocks deep
    p.raw_depth = staged ? 8 : 0;
    p.raw_bytes = staged ? p.raw_depth * kRawSlotBytes + kHdrRingBytes : 0;
    p.stages = (224 * 1024 - p.raw_bytes - kTabBytes) / stage_bytes;
    p.box_rows = nt > 256 ? 64 : nt;   // taller tiles: boxes of 64 rows, of which only those with live rows are copied
    p.a_col_base = nt > 256 ? nt : kAColBase;
    const int ring_stages = (kTmemCols - p.a_col_base) / kAColsPerStage;
    if (p.stages > ring_stages) p.stages = ring_stages;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    p.t_tiles = t_tiles;
    p.n_wtiles = (N + WM - 1) / WM;
    const int kblocks = (K + BK - 1) / BK;
    p.ksplit = 1;
    if (allow_split) {
        // split K until every SM has an item, keeping at least 8 K blocks per split
        const int items = p.t_tiles * p.n_wtiles;
        const int sms = sm_count();
        int want = (sms + items - 1) / items;
        const int cap = kblocks / 8 > 0 ? kblocks / 8 : 1;
        if (want > cap) want = cap;
        // the last arrival adds ksplit partial tiles; keep that short next to the main loop
        const int most = nt <= 32 ? 16 : (nt <= 64 ? 4 : (nt <= 128 ? 2 : 1));
        if (want > most) want = most;
        if (want > 1) p.ksplit = want;
    }
    p.kb_per_split = (kblocks + p.ksplit - 1) / p.ksplit;
    p.kb_per_split = (p.kb_per_split + 3) & ~3;  // splits cover whole 256-value blocks
    p.ksplit = (kblocks + p.kb_per_split - 1) / p.kb_per_split;  // no empty splits
    p.x_bytes = align256(static_cast<size_t>(rows) * K * 2);
    if (p.ksplit > 1) {
        p.partial_bytes = align256(static_cast<size_t>(p.t_tiles) * p.n_wtiles * p.ksplit * WM * nt * 4);
        p.counter_bytes = align256(static_cast<size_t>(p.t_tiles) * p.n_wtiles * 4 * 4);
    }
    return p;
}

template <int T>
int launch_fused_t(const CUtensorMap& tmX, const FusedArgs& a, cudaStream_t s) {
    static bool configured[64] = {};
    int dev = 0;
    LSG_CUDA_TRY(cudaGetDevice(&dev));
    const int smem = a.stages * a.nt * 128 + a.raw_bytes + kTabBytes + 1024 + 512;
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        LSG_CUDA_TRY(cudaFuncSetAttribute(tc_fused_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          227 * 1024));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const long long items = static_cast<long long>(a.t_tiles) * a.ksplit * a.n_wtiles;
    int grid = sm_count();
    if (grid > items) grid = static_cast<int>(items);
    if (grid < 1) grid = 1;
#ifdef LSG_TCF_TRACE
    FusedArgs at = a;
    at.trace = g_tcf_trace && g_tcf_trace_slots > 0
                   ? g_tcf_trace + static_cast<size_t>(g_tcf_trace_launch++ % g_tcf_trace_slots) * 148 * 16
                   : nullptr;
    LSG_CUDA_TRY(launch_kernel(tc_fused_kernel<T>, dim3(grid), dim3(kFusedThreads), smem, s, true, tmX, at));
#else
    LSG_CUDA_TRY(launch_kernel(tc_fused_kernel<T>, dim3(grid), dim3(kFusedThreads), smem, s, true, tmX, a));
#endif
    return LSG_OK;
}

int launch_fused(int type, const CUtensorMap& tmX, const FusedArgs& a, cudaStream_t s) {
    switch (type) {
        case 0: return launch_fused_t<0>(tmX, a, s);
        case 1: return launch_fused_t<1>(tmX, a, s);
        case 2: return launch_fused_t<2>(tmX, a, s);
        case 3: return launch_fused_t<3>(tmX, a, s);
        case 4: return launch_fused_t<4>(tmX, a, s);
        case 5: return launch_fused_t<5>(tmX, a, s);
        case 6: return launch_fused_t<6>(tmX, a, s);
        case 7: return launch_fused_t<7>(tmX, a, s);
    }
    return fail(LSG_ERR_UNSUPPORTED, "gguf fused mmq: unknown type %d", type);
}

int g_mode_override = -1;

int env_mode() {
    static int mode = [] {
        const char* e = getenv("LSG_TC_FUSED");
        return e ? atoi(e) : 1;
    }();
    return g_mode_override >= 0 ? g_mode_override : mode;
}

}  // namespace

// 0: never; 1: types with a register-staged decoder; 2: every type (generic decoder).
bool tc_fused_available(int type) {
    const int mode = env_mode();
    if (mode <= 0) return false;
    if (type == LSG_GGUF_Q4_K) return true;
    return mode >= 2;
}

bool tc_fused_forced() { return env_mode() >= 2; }

size_t tc_fused_dense_scratch_bytes(int M, int N, int K) {
    const int nt = pick_nt(M);
    return make_plan(M, nt, (M + nt - 1) / nt, N, K, true, false).total();
}

// Token rows per tile of a grouped call, from the average rows per expert.  Routed batches
// scatter around their mean (a few standard deviations of a multinomial), so the tile is
// chosen with a fifth of headroom: an expert that holds a few rows more than its tile pays
// the whole weight decoding a second time for those few rows.  Averages beyond 320 rows take
// 256-row tiles (several per expert).
int tc_fused_grouped_tile_m(long long T, int E) {
    static const int force = [] {
        const char* e = getenv("LSG_TC_FUSED_TILE_M");
        return e ? atoi(e) : 0;
    }();
    if (force == 64 || force == 128 || force == 256 || force == 320 || force == 384) return force;
    const long long avg = E > 0 ? (T + E - 1) / E : T;
    // Tiles are balanced per expert (routing.cu), so the tile height only caps how many rows
    // share one pass over an expert's weights; the 5/6 margin keeps most experts of a routed
    // batch in one tile of the chosen height.
    if (avg * 6 <= 64 * 5) return 64;      // the workspace reserves a tile map for tiles of 64 rows or more
    if (avg * 6 <= 128 * 5) return 128;
    if (avg * 6 <= 256 * 5) return 256;
    // above 256 rows the accumulator is single and the stages are large: 320-row tiles keep four
    // stages in shared memory (384-row tiles three), so 384 only where it saves a second tile
    if (avg * 6 <= 320 * 5) return 320;
    if (avg * 6 <= 384 * 5) return 384;
    return 320;
}

size_t tc_fused_grouped_scratch_bytes(long long T, int E, int N, int K) {
    const int nt = tc_fused_grouped_tile_m(T, E);
    return make_plan(T, nt, static_cast<int>((T + nt - 1) / nt) + E, N, K, false, false).total();
}

// Dense: C[M, N] (ldc) = x . W^T with W packed GGUF rows.
int tc_fused_dense(int type, int M, int N, int K, const void* A_bf16, const void* W, void* C, int ldc,
                   int out_dtype, void* ws, size_t ws_bytes, cudaStream_t s, const MmqOutputs* outs) {
    if (M == 0 || N == 0) return LSG_OK;
    if (K % 32 != 0) return fail(LSG_ERR_UNSUPPORTED, "gguf fused mmq: K must be a multiple of 32");
    const int nt = pick_nt(M);
    const Plan p = make_plan(M, nt, (M + nt - 1) / nt, N, K, true, staged_decoder(type));
    if (!ws || ws_bytes < p.total())
        return fail(LSG_ERR_WORKSPACE, "gguf_mmq: workspace too small (have %zu, need %zu)",
                    ws ? ws_bytes : size_t(0), p.total());
    if (reinterpret_cast<uintptr_t>(ws) & 255)
        return fail(LSG_ERR_ALIGNMENT, "gguf_mmq: workspace must be 256-byte aligned");
    uint8_t* wsb = static_cast<uint8_t*>(ws);
    __half* x16 = reinterpret_cast<__half*>(wsb);
    float* partial = reinterpret_cast<float*>(wsb + p.x_bytes);
    unsigned int* counters = reinterpret_cast<unsigned int*>(wsb + p.x_bytes + p.partial_bytes);
    const int n_counters = p.ksplit > 1 ? p.t_tiles * p.n_wtiles * 4 : 0;
    int rc = launch_x_prep<false>(static_cast<const __nv_bfloat16*>(A_bf16), x16, M, K,
                                  n_counters ? counters : static_cast<unsigned int*>(nullptr), n_counters, nullptr,
                                  nullptr, 1, s);
    if (rc != LSG_OK) return rc;
    CUtensorMap tmX;
    rc = make_map(&tmX, x16, M, K, p.box_rows);
    if (rc != LSG_OK) return rc;
    FusedArgs a = {};
    a.W = static_cast<const uint8_t*>(W);
    a.row_bytes = static_cast<long long>(K / gguf_block_values(type)) * gguf_block_bytes(type);
    a.C = C; a.ldc = ldc; a.out_dtype = out_dtype;
    if (outs) {
        a.C_ptrs = outs->C_ptrs; a.n_out = outs->n_out; a.col_off = outs->col_off;
    }
    a.K = K; a.N = N; a.M = M;
    a.nt = nt; a.tile_rows = balanced_tile_rows(M, nt); a.box_rows = p.box_rows; a.a_col_base = p.a_col_base; a.n_wtiles = p.n_wtiles; a.t_tiles = p.t_tiles; a.stages = p.stages; a.raw_depth = p.raw_depth; a.raw_bytes = p.raw_bytes;
    a.ksplit = p.ksplit; a.kb_per_split = p.kb_per_split;
    a.partial = partial; a.counters = counters;
    a.status = device_status_word();
#ifdef LSG_TCF_EXP
    a.dbg = getenv("LSG_TCF_EXP") ? atoi(getenv("LSG_TCF_EXP")) : 0;
#endif
    return launch_fused(type, tmX, a, s);
}

// Unquantized-activation variant: C[M, N] = A_bf16 . dequant(W)^T.  The tensor core multiplies
// fp16 by fp16, so each activation row is brought into fp16 range by a power of two of its own
// (exact: a bf16 value has 8 significant bits, fp16 holds 11) and the output row is scaled
// back in the epilogue.  Only elements more than 2^28 below their row's largest magnitude lose
// bits, which is below what fp32 accumulation resolves.
size_t tc_fused_bf16_scratch_bytes(int M, int N, int K) {
    const int nt = pick_nt(M);
    return make_plan(M, nt, (M + nt - 1) / nt, N, K, true, false).total() + align256(static_cast<size_t>(M) * 4);
}

int tc_fused_dense_bf16(int type, int M, int N, int K, const void* A_bf16, const void* W, void* C, int ldc,
                        int out_dtype, void* ws, size_t ws_bytes, cudaStream_t s) {
    if (M == 0 || N == 0) return LSG_OK;
    if (K % 32 != 0) return fail(LSG_ERR_UNSUPPORTED, "gguf_gemm_bf16: K must be a multiple of 32");
    if (reinterpret_cast<uintptr_t>(A_bf16) & 15)
        return fail(LSG_ERR_ALIGNMENT, "gguf_gemm_bf16: activations must be 16-byte aligned");
    const int nt = pick_nt(M);
    const Plan p = make_plan(M, nt, (M + nt - 1) / nt, N, K, true, staged_decoder(type));
    const size_t need = p.total() + align256(static_cast<size_t>(M) * 4);
    if (!ws || ws_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "gguf_gemm_bf16: workspace too small (have %zu, need %zu)",
                    ws ? ws_bytes : size_t(0), need);
    if (reinterpret_cast<uintptr_t>(ws) & 255)
        return fail(LSG_ERR_ALIGNMENT, "gguf_gemm_bf16: workspace must be 256-byte aligned");
    uint8_t* wsb = static_cast<uint8_t*>(ws);
    __half* x16 = reinterpret_cast<__half*>(wsb);
    float* partial = reinterpret_cast<float*>(wsb + p.x_bytes);
    unsigned int* counters = reinterpret_cast<unsigned int*>(wsb + p.x_bytes + p.partial_bytes);
    float* row_scale = reinterpret_cast<float*>(wsb + p.total());
    const int n_counters = p.ksplit > 1 ? p.t_tiles * p.n_wtiles * 4 : 0;
    // one warp per activation row; the first CTAs also zero the split-K counters
    LSG_CUDA_TRY(launch_kernel(x_rows_to_f16_kernel, dim3(static_cast<unsigned>((M + 7) / 8)), dim3(256), 0, s, true,
                               static_cast<const __nv_bfloat16*>(A_bf16), x16, row_scale, M, K,
                               n_counters ? counters : static_cast<unsigned int*>(nullptr), n_counters));
    CUtensorMap tmX;
    int rc = make_map(&tmX, x16, M, K, p.box_rows);
    if (rc != LSG_OK) return rc;
    FusedArgs a = {};
    a.W = static_cast<const uint8_t*>(W);
    a.row_bytes = static_cast<long long>(K / gguf_block_values(type)) * gguf_block_bytes(type);
    a.C = C; a.ldc = ldc; a.out_dtype = out_dtype;
    a.K = K; a.N = N; a.M = M;
    a.nt = nt; a.tile_rows = balanced_tile_rows(M, nt); a.box_rows = p.box_rows; a.a_col_base = p.a_col_base; a.n_wtiles = p.n_wtiles; a.t_tiles = p.t_tiles; a.stages = p.stages;
    a.raw_depth = p.raw_depth; a.raw_bytes = p.raw_bytes;
    a.ksplit = p.ksplit; a.kb_per_split = p.kb_per_split;
    a.partial = partial; a.counters = counters;
    a.row_scale = row_scale;
    a.status = device_status_word();
#ifdef LSG_TCF_EXP
    a.dbg = getenv("LSG_TCF_EXP") ? atoi(getenv("LSG_TCF_EXP")) : 0;
#endif
    return launch_fused(type, tmX, a, s);
}

// Grouped: token rows of expert e are expert_offsets[e]..[e+1] of A; the tile map (tile_m =
// tc_fused_grouped_tile_m) routes token tiles to experts on the device.
int tc_fused_grouped(int type, int T, int E, int N, int K, const void* A_bf16, const void* const* B_ptrs,
                     const int32_t* expert_offsets, void* D, int out_dtype, const int* tile_expert,
                     const int* tile_mstart, int t_max, int tile_m, void* scratch, size_t scratch_bytes,
                     cudaStream_t s) {
    if (T == 0 || N == 0) return LSG_OK;
    if (K % 32 != 0) return fail(LSG_ERR_UNSUPPORTED, "gguf fused grouped mmq: K must be a multiple of 32");
    const Plan p = make_plan(T, tile_m, t_max, N, K, false, staged_decoder(type));
    if (!scratch || scratch_bytes < p.total())
        return fail(LSG_ERR_WORKSPACE, "gguf grouped mmq: scratch too small (have %zu, need %zu)",
                    scratch ? scratch_bytes : size_t(0), p.total());
    __half* x16 = static_cast<__half*>(scratch);
    int rc = launch_x_prep<false>(static_cast<const __nv_bfloat16*>(A_bf16), x16, T, K, nullptr, 0, expert_offsets + E,
                                  nullptr, 1, s);
    if (rc != LSG_OK) return rc;
    CUtensorMap tmX;
    rc = make_map(&tmX, x16, T, K, p.box_rows);
    if (rc != LSG_OK) return rc;
    FusedArgs a = {};
    a.B_ptrs = B_ptrs;
    a.row_bytes = static_cast<long long>(K / gguf_block_values(type)) * gguf_block_bytes(type);
    a.C = D; a.ldc = N; a.out_dtype = out_dtype;
    a.K = K; a.N = N; a.M = T;
    a.nt = tile_m; a.tile_rows = tile_m; a.box_rows = p.box_rows; a.a_col_base = p.a_col_base; a.n_wtiles = p.n_wtiles; a.t_tiles = t_max; a.stages = p.stages; a.raw_depth = p.raw_depth; a.raw_bytes = p.raw_bytes;
    a.ksplit = 1; a.kb_per_split = p.kb_per_split;
    a.tile_expert = tile_expert; a.tile_mstart = tile_mstart; a.expert_offsets = expert_offsets;
    a.status = device_status_word();
#ifdef LSG_TCF_EXP
    a.dbg = getenv("LSG_TCF_EXP") ? atoi(getenv("LSG_TCF_EXP")) : 0;
#endif
    return launch_fused(type, tmX, a, s);
}

// Expert feed-forward block on rows grouped by expert: D = down( silu(gate(x)) * up(x) ).
// One activation preparation, one launch for gate and up together (weight tiles of both
// matrices side by side, outputs gate | up in a bf16 scratch), SwiGLU fused with the second
// preparation, one launch for down.  The same numbers as three grouped GEMMs with the
// activation computed in fp32 and stored as bf16 in between.
size_t tc_fused_moe_ffn_scratch_bytes(long long T, int H, int I) {
    return align256(static_cast<size_t>(T) * H * 2) + align256(static_cast<size_t>(T) * 2 * I * 2) +
           align256(static_cast<size_t>(T) * I * 2);
}

int tc_fused_moe_ffn(int type, int T, int E, int H, int I, const void* A_bf16, const void* const* gate_ptrs,
                     const void* const* up_ptrs, const void* const* down_ptrs, const int32_t* expert_offsets,
                     void* D, int out_dtype, const int* tile_expert, const int* tile_mstart, int t_max, int tile_m,
                     void* scratch, size_t scratch_bytes, cudaStream_t s, const int32_t* perm, int top_k) {
    if (T == 0) return LSG_OK;
    const size_t need = tc_fused_moe_ffn_scratch_bytes(T, H, I);
    if (!scratch || scratch_bytes < need)
        return fail(LSG_ERR_WORKSPACE, "gguf_moe_ffn: scratch too small (have %zu, need %zu)",
                    scratch ? scratch_bytes : size_t(0), need);
    uint8_t* base = static_cast<uint8_t*>(scratch);
    __half* x16 = reinterpret_cast<__half*>(base);
    __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(base + align256(static_cast<size_t>(T) * H * 2));
    __half* act16 = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(gu) + align256(static_cast<size_t>(T) * 2 * I * 2));
    const bool staged = staged_decoder(type);
    const int qk = gguf_block_values(type), qb = gguf_block_bytes(type);

    // gate | up
    int rc = launch_x_prep<false>(static_cast<const __nv_bfloat16*>(A_bf16), x16, T, H, nullptr, 0, expert_offsets + E,
                                  perm, top_k, s, expert_offsets);
    if (rc != LSG_OK) return rc;
    CUtensorMap tmX;
    Plan p = make_plan(T, tile_m, t_max, I, H, false, staged);
    rc = make_map(&tmX, x16, T, H, p.box_rows);
    if (rc != LSG_OK) return rc;
    FusedArgs a = {};
    a.B_ptrs = gate_ptrs; a.B_ptrs2 = up_ptrs; a.split_wt = p.n_wtiles; a.col2_off = I;
    a.row_bytes = static_cast<long long>(H / qk) * qb;
    a.C = gu; a.ldc = 2 * I; a.out_dtype = LSG_DTYPE_BF16;
    a.K = H; a.N = I; a.M = T;
    a.nt = tile_m; a.tile_rows = tile_m; a.box_rows = p.box_rows; a.a_col_base = p.a_col_base; a.n_wtiles = 2 * p.n_wtiles; a.t_tiles = t_max; a.stages = p.stages;
    a.raw_depth = p.raw_depth; a.raw_bytes = p.raw_bytes;
    a.ksplit = 1; a.kb_per_split = p.kb_per_split;
    a.tile_expert = tile_expert; a.tile_mstart = tile_mstart; a.expert_offsets = expert_offsets;
    a.status = device_status_word();
#ifdef LSG_TCF_EXP
    a.dbg = getenv("LSG_TCF_EXP") ? atoi(getenv("LSG_TCF_EXP")) : 0;
#endif
    rc = launch_fused(type, tmX, a, s);
    if (rc != LSG_OK) return rc;

    // SwiGLU + preparation, then down
    rc = launch_x_prep<true>(gu, act16, T, I, nullptr, 0, expert_offsets + E, nullptr, 1, s, expert_offsets);
    if (rc != LSG_OK) return rc;
    CUtensorMap tmA;
    p = make_plan(T, tile_m, t_max, H, I, false, staged);
    rc = make_map(&tmA, act16, T, I, p.box_rows);
    if (rc != LSG_OK) return rc;
    FusedArgs b = {};
    b.B_ptrs = down_ptrs;
    b.row_bytes = static_cast<long long>(I / qk) * qb;
    b.C = D; b.ldc = H; b.out_dtype = out_dtype;
    b.K = I; b.N = H; b.M = T;
    b.nt = tile_m; b.tile_rows = tile_m; b.box_rows = p.box_rows; b.a_col_base = p.a_col_base; b.n_wtiles = p.n_wtiles; b.t_tiles = t_max; b.stages = p.stages;
    b.raw_depth = p.raw_depth; b.raw_bytes = p.raw_bytes;
    b.ksplit = 1; b.kb_per_split = p.kb_per_split;
    b.tile_expert = tile_expert; b.tile_mstart = tile_mstart; b.expert_offsets = expert_offsets;
    b.status = device_status_word();
#ifdef LSG_TCF_EXP
    b.dbg = getenv("LSG_TCF_EXP") ? atoi(getenv("LSG_TCF_EXP")) : 0;
#endif
    return launch_fused(type, tmA, b, s);
}

}  // namespace lsg

extern "C" int lsg_mmq_set_weight_path(int mode) {
    if (mode > 2) return lsg::fail(LSG_ERR_INVALID, "mmq_set_weight_path: mode must be 0, 1, 2 or negative");
    lsg::g_mode_override = mode < 0 ? -1 : mode;
    return LSG_OK;
}

#ifdef LSG_TCF_TRACE
// Trace builds only: buf holds slots x 148 x 16 zeroed 64-bit counters; launch k sums into slot k % slots.
extern "C" __attribute__((visibility("default"))) int lsg_tc_fused_set_trace(void* buf, int slots) {
    lsg::g_tcf_trace = static_cast<unsigned long long*>(buf);
    lsg::g_tcf_trace_slots = slots;
    lsg::g_tcf_trace_launch = 0;
    return LSG_OK;
}
#endif
