// GGUF block formats for sm_100a: byte layouts (the wire format, identical to
// ggml's and to the reference's csrc/formats/*.h) and two decoders per type:
//
//   * dequant_block<T>(): a whole block to fp32 from global memory, following the
//     value order and arithmetic of the reference's dequant_*_block functions
//     (q4k_format.h:112-133, q6k_format.h:60-80, q5k_format.h:58-86,
//     q2k_format.h:59-78, q3k_format.h:60-95, q8_0_format.h:51-58,
//     mxfp4_format.h:111-120).  Used by the lossless-activation golden GEMM.
//
//   * Mmvq<T>: the integer mat-vec decoder.  It reads a "chunk" of a weight row
//     that has been staged in shared memory and dots it with Q8_1 activations.
//     The math is the reference's  w = A*Q + B  decomposition
//     (gguf_int_policy.h:62-230) regrouped per 16- or 32-value group, so that
//     scales are decoded once per group and the B*sum(q) term uses activation
//     sums computed once per call instead of one dp4a per four values.
//
// Chunk shapes (what one thread consumes at a time):
//   kPair  (Q4_K, Q5_K)       64 consecutive values = two whole Q8_1 blocks
//   kQuad  (Q6_K, Q2_K, Q3_K) 4 groups of 16 values, 32 apart, each in a
//                             different Q8_1 block (the formats interleave
//                             four 32-value "quads" in the same bytes)
//   kBlock (Q8_0, Q4_0, MXFP4) one 32-value block
#pragma once

#include "common.cuh"

namespace lsg {

constexpr int kQ8_1Bytes = 36;

// ---------------------------------------------------------------------------
// Type traits
// ---------------------------------------------------------------------------
enum ChunkShape { kPair = 0, kQuad = 1, kBlock = 2 };

template <int T> struct Fmt;
template <> struct Fmt<LSG_GGUF_Q2_K> { static constexpr int VALS = 256, BYTES = 84;  static constexpr ChunkShape SHAPE = kQuad; };
template <> struct Fmt<LSG_GGUF_Q3_K> { static constexpr int VALS = 256, BYTES = 110; static constexpr ChunkShape SHAPE = kQuad; };
template <> struct Fmt<LSG_GGUF_Q4_K> { static constexpr int VALS = 256, BYTES = 144; static constexpr ChunkShape SHAPE = kPair; };
template <> struct Fmt<LSG_GGUF_Q5_K> { static constexpr int VALS = 256, BYTES = 176; static constexpr ChunkShape SHAPE = kPair; };
template <> struct Fmt<LSG_GGUF_Q6_K> { static constexpr int VALS = 256, BYTES = 210; static constexpr ChunkShape SHAPE = kQuad; };
template <> struct Fmt<LSG_GGUF_Q8_0> { static constexpr int VALS = 32,  BYTES = 34;  static constexpr ChunkShape SHAPE = kBlock; };
template <> struct Fmt<LSG_GGUF_MXFP4>{ static constexpr int VALS = 32,  BYTES = 17;  static constexpr ChunkShape SHAPE = kBlock; };
template <> struct Fmt<LSG_GGUF_Q4_0> { static constexpr int VALS = 32,  BYTES = 18;  static constexpr ChunkShape SHAPE = kBlock; };

inline int gguf_block_values(int type) {
    switch (type) {
        case LSG_GGUF_Q2_K: case LSG_GGUF_Q3_K: case LSG_GGUF_Q4_K:
        case LSG_GGUF_Q5_K: case LSG_GGUF_Q6_K: return 256;
        case LSG_GGUF_Q8_0: case LSG_GGUF_MXFP4: case LSG_GGUF_Q4_0: return 32;
        default: return 0;
    }
}
inline int gguf_block_bytes(int type) {
    switch (type) {
        case LSG_GGUF_Q2_K: return 84;
        case LSG_GGUF_Q3_K: return 110;
        case LSG_GGUF_Q4_K: return 144;
        case LSG_GGUF_Q5_K: return 176;
        case LSG_GGUF_Q6_K: return 210;
        case LSG_GGUF_Q8_0: return 34;
        case LSG_GGUF_MXFP4: return 17;
        case LSG_GGUF_Q4_0: return 18;
        default: return 0;
    }
}

#if defined(__CUDACC__)

// ---------------------------------------------------------------------------
// Scalar helpers shared by both decoders
// ---------------------------------------------------------------------------
__device__ __forceinline__ float half_at(const uint8_t* p) {
    return fp16_bits_to_float(static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8));
}

// 6-bit (scale, min) pair j of the 12-byte Q4_K/Q5_K scale field
// (reference: get_scale_min_k4, csrc/formats/kquant_common.h:36-46).
__device__ __forceinline__ void k4_scale_min(int j, const uint8_t* s, int& sc, int& mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// 6-bit Q3_K scale `is` (0..15) of the 12-byte scale field, before the -32 bias.
__device__ __forceinline__ int q3k_scale6(int is, const uint8_t* s) {
    const int lowbyte = s[is & 7];
    const int low4 = (is < 8) ? (lowbyte & 0x0F) : (lowbyte >> 4);
    const int hi2 = (s[8 + (is & 3)] >> (2 * (is >> 2))) & 3;
    return low4 | (hi2 << 4);
}

// E8M0 exponent byte -> half of 2^(e-127), i.e. 2^(e-128), denormal-aware
// (reference: e8m0_to_fp32_half, csrc/formats/mxfp4_format.h:96-104).
__device__ __forceinline__ float e8m0_half_scale(uint32_t e) {
    const uint32_t bits = (e < 2) ? (0x00200000u << e) : ((e - 1u) << 23);
    return __uint_as_float(bits);
}

// e2m1 code -> 2x its real value, an exact small integer (ggml kvalues_mxfp4).
__device__ __forceinline__ int mxfp4_code_value(int code) {
    const int mag_tab = 0x0C080604;  // codes 4..7 -> 4,6,8,12
    const int m = code & 7;
    const int mag = (m < 4) ? m : ((mag_tab >> (8 * (m - 4))) & 0xFF);
    return (code & 8) ? -mag : mag;
}

// ---------------------------------------------------------------------------
// Whole-block dequant to fp32 (golden path; byte loads, no alignment needs)
// ---------------------------------------------------------------------------
template <int T>
__device__ inline void dequant_block(const uint8_t* __restrict__ b, float* __restrict__ out);

template <>
__device__ inline void dequant_block<LSG_GGUF_Q4_K>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t* sc = b + 4;
    const uint8_t* qs = b + 16;
    for (int pair = 0; pair < 4; ++pair) {
        int s0, m0, s1, m1;
        k4_scale_min(2 * pair, sc, s0, m0);
        k4_scale_min(2 * pair + 1, sc, s1, m1);
        const float d0 = d * s0, mm0 = dmin * m0, d1 = d * s1, mm1 = dmin * m1;
        for (int l = 0; l < 32; ++l) {
            const int q = qs[pair * 32 + l];
            out[pair * 64 + l] = d0 * (q & 0xF) - mm0;
            out[pair * 64 + 32 + l] = d1 * (q >> 4) - mm1;
        }
    }
}

template <>
__device__ inline void dequant_block<LSG_GGUF_Q5_K>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t* sc = b + 4;
    const uint8_t* qh = b + 16;
    const uint8_t* qs = b + 48;
    for (int pair = 0; pair < 4; ++pair) {
        int s0, m0, s1, m1;
        k4_scale_min(2 * pair, sc, s0, m0);
        k4_scale_min(2 * pair + 1, sc, s1, m1);
        const float d0 = d * s0, mm0 = dmin * m0, d1 = d * s1, mm1 = dmin * m1;
        for (int l = 0; l < 32; ++l) {
            const int q = qs[pair * 32 + l];
            const int h = qh[l];
            out[pair * 64 + l] = d0 * ((q & 0xF) + (((h >> (2 * pair)) & 1) << 4)) - mm0;
            out[pair * 64 + 32 + l] = d1 * ((q >> 4) + (((h >> (2 * pair + 1)) & 1) << 4)) - mm1;
        }
    }
}

template <>
__device__ inline void dequant_block<LSG_GGUF_Q6_K>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const uint8_t* ql = b;
    const uint8_t* qh = b + 128;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
    const float d = half_at(b + 208);
    for (int ip = 0; ip < 2; ++ip) {
        for (int il = 0; il < 32; ++il) {
            const int is = 8 * ip + il / 16;
            const int h = qh[32 * ip + il];
            const int a = ql[64 * ip + il], c = ql[64 * ip + il + 32];
            float* y = out + 128 * ip + il;
            y[0]  = d * sc[is + 0] * (static_cast<int>((a & 0xF) | (((h >> 0) & 3) << 4)) - 32);
            y[32] = d * sc[is + 2] * (static_cast<int>((c & 0xF) | (((h >> 2) & 3) << 4)) - 32);
            y[64] = d * sc[is + 4] * (static_cast<int>((a >> 4) | (((h >> 4) & 3) << 4)) - 32);
            y[96] = d * sc[is + 6] * (static_cast<int>((c >> 4) | (((h >> 6) & 3) << 4)) - 32);
        }
    }
}

template <>
__device__ inline void dequant_block<LSG_GGUF_Q2_K>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const uint8_t* sc = b;
    const uint8_t* qs = b + 16;
    const float d = half_at(b + 80), dmin = half_at(b + 82);
    for (int n = 0; n < 2; ++n) {
        for (int l = 0; l < 32; ++l) {
            const int is = 8 * n + l / 16;
            const int q = qs[32 * n + l];
            float* y = out + 128 * n + l;
            for (int quad = 0; quad < 4; ++quad) {
                const int s = sc[is + 2 * quad];
                y[32 * quad] = d * (s & 0xF) * ((q >> (2 * quad)) & 3) - dmin * (s >> 4);
            }
        }
    }
}

template <>
__device__ inline void dequant_block<LSG_GGUF_Q3_K>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const uint8_t* hm = b;
    const uint8_t* qs = b + 32;
    const uint8_t* sc = b + 96;
    const float d = half_at(b + 108);
    for (int n = 0; n < 2; ++n) {
        for (int j = 0; j < 4; ++j) {
            for (int l = 0; l < 32; ++l) {
                const int is = 8 * n + 2 * j + l / 16;
                const float dl = d * (q3k_scale6(is, sc) - 32);
                const int q2 = (qs[32 * n + l] >> (2 * j)) & 3;
                const int hb = (hm[l] >> (4 * n + j)) & 1;
                out[128 * n + 32 * j + l] = dl * (q2 - (hb ? 0 : 4));
            }
        }
    }
}

template <>
__device__ inline void dequant_block<LSG_GGUF_Q8_0>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const float d = half_at(b);
    const int8_t* qs = reinterpret_cast<const int8_t*>(b + 2);
    for (int l = 0; l < 32; ++l) out[l] = d * static_cast<float>(qs[l]);
}

template <>
__device__ inline void dequant_block<LSG_GGUF_Q4_0>(const uint8_t* __restrict__ b,
                                                   float* __restrict__ out) {
    const float d = half_at(b);
    const uint8_t* qs = b + 2;
    for (int l = 0; l < 16; ++l) {
        out[l] = d * static_cast<float>((qs[l] & 0xF) - 8);
        out[l + 16] = d * static_cast<float>((qs[l] >> 4) - 8);
    }
}

template <>
__device__ inline void dequant_block<LSG_GGUF_MXFP4>(const uint8_t* __restrict__ b,
                                                    float* __restrict__ out) {
    const float d = e8m0_half_scale(b[0]);
    const uint8_t* qs = b + 1;
    for (int l = 0; l < 16; ++l) {
        out[l] = static_cast<float>(mxfp4_code_value(qs[l] & 0xF)) * d;
        out[l + 16] = static_cast<float>(mxfp4_code_value(qs[l] >> 4)) * d;
    }
}

// ---------------------------------------------------------------------------
// Shared-memory loads by 32-bit shared address
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds8(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// N consecutive little-endian words starting at ANY byte address: N+1 aligned
// word loads and N funnel shifts.  Blocks of 17/18/34/110/210 bytes start on
// 1- or 2-byte boundaries, so their fields are never word aligned in general.
// The extra word read stays inside the staged slab (slabs are padded).
template <int N>
__device__ __forceinline__ void lds_words_unaligned(uint32_t addr, uint32_t (&w)[N]) {
    const uint32_t base = addr & ~3u;
    const uint32_t sh = (addr & 3u) * 8u;
    uint32_t prev = lds32(base);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = lds32(base + 4u * (i + 1));
        w[i] = __funnelshift_r(prev, next, sh);
        prev = next;
    }
}

// ---------------------------------------------------------------------------
// Activation chunk as seen by one thread
// ---------------------------------------------------------------------------
// qs : the chunk's int8 values, 4 per word, in the order the weight decoder
//      produces them.
// d  : the fp32 Q8_1 scale of each group.
// s  : d * (sum of the group's int8 values), for the min / offset terms.
// kPair: 2 groups of 32 (8 words each).  kQuad: 4 groups of 16 (4 words each).
// kBlock: 1 group of 32 in qs[0..7]; d[0]; s[0].
template <ChunkShape S> struct XChunk;
template <> struct XChunk<kPair>  { int qs[16]; float d[2]; float s[2]; };
template <> struct XChunk<kQuad>  { int qs[16]; float d[4]; float s[4]; };
template <> struct XChunk<kBlock> { int qs[8];  float d[1]; float s[1]; };

// ---------------------------------------------------------------------------
// Integer mat-vec decoders.  W<T> holds one chunk of one weight row, unpacked
// once; dot(w, x) returns the chunk's contribution  sum_k w_k * x_k  with
// x_k ~ d * q_k.
// ---------------------------------------------------------------------------
template <int T> struct Mmvq;

// ---- Q4_K: 144 B = {fp16 d, fp16 dmin, 12 B 6-bit scales/mins, 128 B nibbles}
template <> struct Mmvq<LSG_GGUF_Q4_K> {
    static constexpr int CHUNKS_PER_BLOCK = 4;
    struct W {
        uint32_t lo[8];   // low nibbles, sub-block 2p   (values 0..15)
        uint32_t hi[8];   // high nibbles IN PLACE (value*16), sub-block 2p+1
        float a0, a1;     // d*sc(2p), d*sc(2p+1)/16
        float b0, b1;     // dmin*m(2p), dmin*m(2p+1)
    };
    // row: shared address of the row's first block; c: chunk index in the row.
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + (c >> 2) * 144;
        const int p = c & 3;
        const uint4 hdr = lds128(blk);
        const uint4 q0 = lds128(blk + 16 + p * 32);
        const uint4 q1 = lds128(blk + 32 + p * 32);
        const float d = fp16_bits_to_float(hdr.x), dmin = fp16_bits_to_float(hdr.x >> 16);
        // scale bytes 2h,2h+1 | 4+2h,5+2h | 8+2h,9+2h with h = p & 1
        const int sh = (p & 1) * 16;
        const uint32_t a16 = (hdr.y >> sh) & 0xFFFFu;
        const uint32_t b16 = (hdr.z >> sh) & 0xFFFFu;
        const uint32_t c16 = (hdr.w >> sh) & 0xFFFFu;
        uint32_t sc2, mn2;
        if (p < 2) {
            sc2 = a16 & 0x3F3Fu;
            mn2 = b16 & 0x3F3Fu;
        } else {
            sc2 = (c16 & 0x0F0Fu) | ((a16 >> 2) & 0x3030u);
            mn2 = ((c16 >> 4) & 0x0F0Fu) | ((b16 >> 2) & 0x3030u);
        }
        w.a0 = d * static_cast<float>(sc2 & 0xFFu);
        w.a1 = d * static_cast<float>(sc2 >> 8) * 0.0625f;
        w.b0 = dmin * static_cast<float>(mn2 & 0xFFu);
        w.b1 = dmin * static_cast<float>(mn2 >> 8);
        const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            w.lo[i] = q[i] & 0x0F0F0F0Fu;
            w.hi[i] = q[i] & 0xF0F0F0F0u;
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kPair>& x) {
        int d0 = 0, d1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            d0 = dp4a_us(w.lo[i], x.qs[i], d0);
            d1 = dp4a_us(w.hi[i], x.qs[8 + i], d1);
        }
        return x.d[0] * (w.a0 * static_cast<float>(d0)) - w.b0 * x.s[0] +
               x.d[1] * (w.a1 * static_cast<float>(d1)) - w.b1 * x.s[1];
    }
};

// ---- Q5_K: 176 B = {d, dmin, 12 B scales, 32 B high bits, 128 B nibbles}
template <> struct Mmvq<LSG_GGUF_Q5_K> {
    static constexpr int CHUNKS_PER_BLOCK = 4;
    struct W {
        uint32_t lo[8], hi[8];  // 5-bit values 0..31 of sub-blocks 2p, 2p+1
        float a0, a1, b0, b1;
    };
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + (c >> 2) * 176;
        const int p = c & 3;
        const uint4 hdr = lds128(blk);
        const uint4 h0 = lds128(blk + 16), h1 = lds128(blk + 32);
        const uint4 q0 = lds128(blk + 48 + p * 32), q1 = lds128(blk + 64 + p * 32);
        const float d = fp16_bits_to_float(hdr.x), dmin = fp16_bits_to_float(hdr.x >> 16);
        const int sh = (p & 1) * 16;
        const uint32_t a16 = (hdr.y >> sh) & 0xFFFFu;
        const uint32_t b16 = (hdr.z >> sh) & 0xFFFFu;
        const uint32_t c16 = (hdr.w >> sh) & 0xFFFFu;
        uint32_t sc2, mn2;
        if (p < 2) {
            sc2 = a16 & 0x3F3Fu;
            mn2 = b16 & 0x3F3Fu;
        } else {
            sc2 = (c16 & 0x0F0Fu) | ((a16 >> 2) & 0x3030u);
            mn2 = ((c16 >> 4) & 0x0F0Fu) | ((b16 >> 2) & 0x3030u);
        }
        w.a0 = d * static_cast<float>(sc2 & 0xFFu);
        w.a1 = d * static_cast<float>(sc2 >> 8);
        w.b0 = dmin * static_cast<float>(mn2 & 0xFFu);
        w.b1 = dmin * static_cast<float>(mn2 >> 8);
        const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const uint32_t h[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            w.lo[i] = (q[i] & 0x0F0F0F0Fu) | (((h[i] >> (2 * p)) & 0x01010101u) << 4);
            w.hi[i] = ((q[i] >> 4) & 0x0F0F0F0Fu) | (((h[i] >> (2 * p + 1)) & 0x01010101u) << 4);
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kPair>& x) {
        int d0 = 0, d1 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            d0 = dp4a_us(w.lo[i], x.qs[i], d0);
            d1 = dp4a_us(w.hi[i], x.qs[8 + i], d1);
        }
        return x.d[0] * (w.a0 * static_cast<float>(d0)) - w.b0 * x.s[0] +
               x.d[1] * (w.a1 * static_cast<float>(d1)) - w.b1 * x.s[1];
    }
};

// ---- Q6_K: 210 B = {128 B low nibbles, 64 B high 2 bits, 16 int8 scales, fp16 d}
// chunk (ip, h): l in [16h,16h+16) of half ip; quad q gives values
// 128ip + 32q + l, scale index 8ip + 2q + h.
template <> struct Mmvq<LSG_GGUF_Q6_K> {
    static constexpr int CHUNKS_PER_BLOCK = 4;
    struct W {
        uint32_t v[4][4];  // [quad][word] 6-bit values 0..63 (offset 32 not removed)
        float a[4];        // d * scale(quad)
    };
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + (c >> 2) * 210;
        const int ip = (c >> 1) & 1, h = c & 1;
        uint32_t la[4], lb[4], qh[4];
        lds_words_unaligned<4>(blk + 64 * ip + 16 * h, la);
        lds_words_unaligned<4>(blk + 64 * ip + 32 + 16 * h, lb);
        lds_words_unaligned<4>(blk + 128 + 32 * ip + 16 * h, qh);
        const float d = fp16_bits_to_float(lds16(blk + 208));
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int sc = static_cast<int>(static_cast<int8_t>(lds8(blk + 192 + 8 * ip + 2 * q + h)));
            w.a[q] = d * static_cast<float>(sc);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w.v[0][i] = (la[i] & 0x0F0F0F0Fu) | ((qh[i] << 4) & 0x30303030u);
            w.v[1][i] = (lb[i] & 0x0F0F0F0Fu) | ((qh[i] << 2) & 0x30303030u);
            w.v[2][i] = ((la[i] >> 4) & 0x0F0F0F0Fu) | (qh[i] & 0x30303030u);
            w.v[3][i] = ((lb[i] >> 4) & 0x0F0F0F0Fu) | ((qh[i] >> 2) & 0x30303030u);
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kQuad>& x) {
        float r = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int dt = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) dt = dp4a_us(w.v[q][i], x.qs[4 * q + i], dt);
            r += w.a[q] * (x.d[q] * static_cast<float>(dt) - 32.0f * x.s[q]);
        }
        return r;
    }
};

// ---- Q2_K: 84 B = {16 B (scale|min<<4), 64 B 2-bit quants, fp16 d, fp16 dmin}
template <> struct Mmvq<LSG_GGUF_Q2_K> {
    static constexpr int CHUNKS_PER_BLOCK = 4;
    struct W {
        uint32_t v[4][4];
        float a[4], b[4];  // d*scale, dmin*min
    };
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + (c >> 2) * 84;
        const int n = (c >> 1) & 1, h = c & 1;
        uint32_t qs[4];
        lds_words_unaligned<4>(blk + 16 + 32 * n + 16 * h, qs);
        const uint32_t dm = lds16(blk + 80) | (lds16(blk + 82) << 16);
        const float d = fp16_bits_to_float(dm), dmin = fp16_bits_to_float(dm >> 16);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t s = lds8(blk + 8 * n + 2 * q + h);
            w.a[q] = d * static_cast<float>(s & 0xFu);
            w.b[q] = dmin * static_cast<float>(s >> 4);
#pragma unroll
            for (int i = 0; i < 4; ++i) w.v[q][i] = (qs[i] >> (2 * q)) & 0x03030303u;
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kQuad>& x) {
        float r = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int dt = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) dt = dp4a_us(w.v[q][i], x.qs[4 * q + i], dt);
            r += x.d[q] * (w.a[q] * static_cast<float>(dt)) - w.b[q] * x.s[q];
        }
        return r;
    }
};

// ---- Q3_K: 110 B = {32 B high-bit mask, 64 B low 2 bits, 12 B 6-bit scales, fp16 d}
template <> struct Mmvq<LSG_GGUF_Q3_K> {
    static constexpr int CHUNKS_PER_BLOCK = 4;
    struct W {
        uint32_t v[4][4];  // 3-bit values 0..7 (offset 4 not removed)
        float a[4];        // d * (scale6 - 32)
    };
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + (c >> 2) * 110;
        const int n = (c >> 1) & 1, h = c & 1;
        uint32_t qs[4], hm[4], sw[3];
        lds_words_unaligned<4>(blk + 32 + 32 * n + 16 * h, qs);
        lds_words_unaligned<4>(blk + 16 * h, hm);
        lds_words_unaligned<3>(blk + 96, sw);
        const float d = fp16_bits_to_float(lds16(blk + 108));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // scale index is = 8n + 2j + h: low nibble source byte (2j+h), high
            // 2 bits from byte 8 + ((2j+h)&3) at bit 2*(2n + (j>>1)).
            const int lb = 2 * j + h;                       // 0..7
            const uint32_t lowbyte = (((lb < 4) ? sw[0] : sw[1]) >> (8 * (lb & 3))) & 0xFFu;
            const uint32_t low4 = (lowbyte >> (4 * n)) & 0xFu;
            const uint32_t hb = (sw[2] >> (8 * (lb & 3))) & 0xFFu;
            const uint32_t hi2 = (hb >> (2 * (2 * n + (j >> 1)))) & 3u;
            w.a[j] = d * static_cast<float>(static_cast<int>(low4 | (hi2 << 4)) - 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t q2 = (qs[i] >> (2 * j)) & 0x03030303u;
                const uint32_t hs = (hm[i] >> (4 * n + j)) & 0x01010101u;
                w.v[j][i] = q2 | (hs << 2);
            }
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kQuad>& x) {
        float r = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            int dt = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) dt = dp4a_us(w.v[q][i], x.qs[4 * q + i], dt);
            r += w.a[q] * (x.d[q] * static_cast<float>(dt) - 4.0f * x.s[q]);
        }
        return r;
    }
};

// ---- Q8_0: 34 B = {fp16 d, 32 int8}
template <> struct Mmvq<LSG_GGUF_Q8_0> {
    static constexpr int CHUNKS_PER_BLOCK = 1;
    struct W { uint32_t v[8]; float a; };
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + c * 34;
        lds_words_unaligned<8>(blk + 2, w.v);
        w.a = fp16_bits_to_float(lds16(blk));
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kBlock>& x) {
        int dt = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) dt = dp4a_ss(static_cast<int>(w.v[i]), x.qs[i], dt);
        return x.d[0] * (w.a * static_cast<float>(dt));
    }
};

// ---- Q4_0: 18 B = {fp16 d, 16 B nibbles}; low nibble = value j, high = j+16;
// w = d * (q - 8).  Not in the reference; the rule is ggml's.
template <> struct Mmvq<LSG_GGUF_Q4_0> {
    static constexpr int CHUNKS_PER_BLOCK = 1;
    struct W { uint32_t lo[4], hi[4]; float a; };
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + c * 18;
        uint32_t q[4];
        lds_words_unaligned<4>(blk + 2, q);
        w.a = fp16_bits_to_float(lds16(blk));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w.lo[i] = q[i] & 0x0F0F0F0Fu;
            w.hi[i] = q[i] & 0xF0F0F0F0u;  // value * 16
        }
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kBlock>& x) {
        int d0 = 0, d1 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            d0 = dp4a_us(w.lo[i], x.qs[i], d0);
            d1 = dp4a_us(w.hi[i], x.qs[4 + i], d1);
        }
        const int dt = d0 + (d1 >> 4);  // d1 is an exact multiple of 16
        return w.a * (x.d[0] * static_cast<float>(dt) - 8.0f * x.s[0]);
    }
};

// ---- MXFP4: 17 B = {E8M0 exponent, 16 B e2m1 codes}; low nibble = value j,
// high = j+16; value = table[code] * 2^(e-128), table holding 2x the e2m1 value.
template <> struct Mmvq<LSG_GGUF_MXFP4> {
    static constexpr int CHUNKS_PER_BLOCK = 1;
    struct W { uint32_t lo[4], hi[4]; float a; };
    // Eight 4-bit codes -> eight signed bytes through three byte permutes per
    // half: magnitudes come from a 8-entry table selected by the low 3 bits,
    // negated entries from a second table, and bit 3 picks between them.
    __device__ static __forceinline__ void lookup8(uint32_t codes, uint32_t& even, uint32_t& odd) {
        const uint32_t pos_lo = 0x03020100u, pos_hi = 0x0C080604u;
        const uint32_t neg_lo = 0xFDFEFF00u, neg_hi = 0xF4F8FAFCu;
        const uint32_t mag_sel = codes & 0x77777777u;
        const uint32_t sgn_sel = 0x32103210u | ((codes & 0x88888888u) >> 1);
        uint32_t half[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint32_t p = __byte_perm(pos_lo, pos_hi, mag_sel >> (16 * k));
            const uint32_t n = __byte_perm(neg_lo, neg_hi, mag_sel >> (16 * k));
            half[k] = __byte_perm(p, n, sgn_sel >> (16 * k));
        }
        even = __byte_perm(half[0], half[1], 0x6420);  // codes 0,2,4,6 = low nibbles
        odd = __byte_perm(half[0], half[1], 0x7531);   // codes 1,3,5,7 = high nibbles
    }
    __device__ static __forceinline__ void load(uint32_t row, int c, W& w) {
        const uint32_t blk = row + c * 17;
        uint32_t q[4];
        lds_words_unaligned<4>(blk + 1, q);
        w.a = e8m0_half_scale(lds8(blk));
#pragma unroll
        for (int i = 0; i < 4; ++i) lookup8(q[i], w.lo[i], w.hi[i]);
    }
    __device__ static __forceinline__ float dot(const W& w, const XChunk<kBlock>& x) {
        int dt = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            dt = dp4a_ss(static_cast<int>(w.lo[i]), x.qs[i], dt);
            dt = dp4a_ss(static_cast<int>(w.hi[i]), x.qs[4 + i], dt);
        }
        return x.d[0] * (w.a * static_cast<float>(dt));
    }
};

#endif  // __CUDACC__

}  // namespace lsg
