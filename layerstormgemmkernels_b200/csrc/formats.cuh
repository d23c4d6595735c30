// GGUF block formats for sm_100a: byte layouts (the wire format, identical to
// ggml's and to the reference's csrc/formats/*.h), type traits, scalar helpers,
// shared-memory load helpers, and dequant_block<T>(): a whole block to fp32 from
// global memory, following the value order and arithmetic of the reference's
// dequant_*_block functions (q4k_format.h:112-133, q6k_format.h:60-80,
// q5k_format.h:58-86, q2k_format.h:59-78, q3k_format.h:60-95, q8_0_format.h:51-58,
// mxfp4_format.h:111-120).  The integer mat-vec decoders live in mmvq_decode.cuh.
#pragma once

#include "common.cuh"

namespace lsg {

constexpr int kQ8_1Bytes = 36;

// ---------------------------------------------------------------------------
// Type traits
// ---------------------------------------------------------------------------

template <int T> struct Fmt;
template <> struct Fmt<LSG_GGUF_Q2_K> { static constexpr int VALS = 256, BYTES = 84; };
template <> struct Fmt<LSG_GGUF_Q3_K> { static constexpr int VALS = 256, BYTES = 110; };
template <> struct Fmt<LSG_GGUF_Q4_K> { static constexpr int VALS = 256, BYTES = 144; };
template <> struct Fmt<LSG_GGUF_Q5_K> { static constexpr int VALS = 256, BYTES = 176; };
template <> struct Fmt<LSG_GGUF_Q6_K> { static constexpr int VALS = 256, BYTES = 210; };
template <> struct Fmt<LSG_GGUF_Q8_0> { static constexpr int VALS = 32,  BYTES = 34; };
template <> struct Fmt<LSG_GGUF_MXFP4>{ static constexpr int VALS = 32,  BYTES = 17; };
template <> struct Fmt<LSG_GGUF_Q4_0> { static constexpr int VALS = 32,  BYTES = 18; };

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
// 32 consecutive values (chunk c of a block) to fp32: the same arithmetic as
// dequant_block, one chunk at a time, for kernels that spread a block over 8 threads.
// ---------------------------------------------------------------------------
template <int T>
__device__ inline void dequant_chunk32(const uint8_t* __restrict__ b, int c, float* __restrict__ out) {
    if (T == LSG_GGUF_Q4_K || T == LSG_GGUF_Q5_K) {
        const float d = half_at(b), dmin = half_at(b + 2);
        int sc, mn;
        k4_scale_min(c, b + 4, sc, mn);
        const float ds = d * sc, ms = dmin * mn;
        const int pair = c >> 1, hi = c & 1;
        const uint8_t* qs = b + (T == LSG_GGUF_Q4_K ? 16 : 48) + pair * 32;
        for (int l = 0; l < 32; ++l) {
            int q = hi ? (qs[l] >> 4) : (qs[l] & 0xF);
            if (T == LSG_GGUF_Q5_K) q += ((b[16 + l] >> c) & 1) << 4;
            out[l] = ds * q - ms;
        }
    } else if (T == LSG_GGUF_Q6_K) {
        const int ip = c >> 2, quad = c & 3;
        const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
        const float d = half_at(b + 208);
        for (int l = 0; l < 32; ++l) {
            const int ql = b[64 * ip + (quad & 1) * 32 + l];
            const int nib = (quad >= 2) ? (ql >> 4) : (ql & 0xF);
            const int h = (b[128 + 32 * ip + l] >> (2 * quad)) & 3;
            out[l] = d * sc[8 * ip + 2 * quad + l / 16] * (static_cast<int>(nib | (h << 4)) - 32);
        }
    } else if (T == LSG_GGUF_Q2_K) {
        const int n = c >> 2, quad = c & 3;
        const float d = half_at(b + 80), dmin = half_at(b + 82);
        for (int l = 0; l < 32; ++l) {
            const int s = b[8 * n + 2 * quad + l / 16];
            const int q = (b[16 + 32 * n + l] >> (2 * quad)) & 3;
            out[l] = d * (s & 0xF) * q - dmin * (s >> 4);
        }
    } else if (T == LSG_GGUF_Q3_K) {
        const int n = c >> 2, j = c & 3;
        const float d = half_at(b + 108);
        for (int l = 0; l < 32; ++l) {
            const float dl = d * (q3k_scale6(8 * n + 2 * j + l / 16, b + 96) - 32);
            const int q2 = (b[32 + 32 * n + l] >> (2 * j)) & 3;
            const int hb = (b[l] >> (4 * n + j)) & 1;
            out[l] = dl * (q2 - (hb ? 0 : 4));
        }
    } else {
        dequant_block<T>(b, out);  // 32-value blocks: the chunk is the block
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

#endif  // __CUDACC__

}  // namespace lsg
