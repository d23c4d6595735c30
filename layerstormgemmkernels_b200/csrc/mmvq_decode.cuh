// Integer mat-vec decoders for the GGUF types, sm_100a.
//
// The math is the reference's  w = A*Q + B  decomposition against Q8_1
// activations (csrc/sm120/gemm/gguf/gguf_int_policy.h:62-230 and
// gguf_mmvq_impl.cuh:43-70), regrouped so that one lane consumes a whole "unit"
// of a weight row - a 256-value super-block (Q4_K, Q5_K), half a super-block
// (Q6_K, Q2_K, Q3_K) or a 32-value block (Q8_0, Q4_0, MXFP4):
//
//   * the block header (scales, mins) is decoded once per unit with word-wide
//     bit tricks instead of once per four values;
//   * the B*sum(q) terms use per-group activation sums prepared once per CTA
//     in the activation image, not one dp4a per four values;
//   * 4-bit high nibbles are dotted in place (value*16) and the 1/16 is folded
//     into the scale; 6-, 3- and 2-bit values are dotted unsigned and their
//     offsets (-32, -4) are applied through the same sums;
//   * RW weight rows share every activation load.
//
// Activation image (one per batch row, built by build_x_image):
//   [qs planes][d][s]
//   qs : 16-byte pieces; piece j of unit u lives at (j*U + u)*16, so the lanes
//        of a warp, which hold consecutive units, read consecutive 16-byte
//        slots (no bank conflicts);
//   d  : fp32 Q8_1 scale per 32 values; four per float4, float4 h of unit u at
//        d_off + (h*U + u)*16 (for 32-value units: one float per unit);
//   s  : per-group sums, same plane layout - fp32 d*sum(q) per 32 (Q4_K, Q5_K,
//        Q4_0) or per 16 (Q2_K), int32 sum(q) per 16 (Q6_K, Q3_K).
#pragma once

#include "common.cuh"
#include "formats.cuh"

namespace lsg {

#if defined(__CUDACC__)

enum SumKind { kSumNone = 0, kSumF32Per32 = 1, kSumF32Per16 = 2, kSumI32Per16 = 3 };

struct XView {
    uint32_t base;   // shared address of the image of the tile's first batch row
    uint32_t rowb;   // bytes per row image
    uint32_t d_off;  // byte offset of the d planes inside a row image
    uint32_t s_off;  // byte offset of the s planes
    int U;           // units per weight row
    int mlast;       // last valid batch row of the tile (rows beyond re-read it)
};

template <int T> struct Mmvq;

__device__ __forceinline__ int sext8(uint32_t w, int k) {
    return static_cast<int>(static_cast<int8_t>((w >> (8 * k)) & 0xFFu));
}
__device__ __forceinline__ int zext8(uint32_t w, int k) {
    return static_cast<int>((w >> (8 * k)) & 0xFFu);
}
__device__ __forceinline__ void unpack4(const uint4& v, uint32_t* dst) {
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
__device__ __forceinline__ void unpack4f(const uint4& v, float* dst) {
    dst[0] = __uint_as_float(v.x); dst[1] = __uint_as_float(v.y);
    dst[2] = __uint_as_float(v.z); dst[3] = __uint_as_float(v.w);
}

// 6-bit scales and mins of a Q4_K / Q5_K header as four byte-packed words:
// sc[0] = scales 0..3, sc[1] = scales 4..7, mn[0] = mins 0..3, mn[1] = mins 4..7.
// w0..w2 are the three words of the 12-byte field (get_scale_min_k4 for all j at once).
__device__ __forceinline__ void k4_unpack_all(uint32_t w0, uint32_t w1, uint32_t w2,
                                              uint32_t (&sc)[2], uint32_t (&mn)[2]) {
    sc[0] = w0 & 0x3F3F3F3Fu;
    mn[0] = w1 & 0x3F3F3F3Fu;
    sc[1] = (w2 & 0x0F0F0F0Fu) | ((w0 >> 2) & 0x30303030u);
    mn[1] = ((w2 >> 4) & 0x0F0F0F0Fu) | ((w1 >> 2) & 0x30303030u);
}

// ===========================================================================
// Q4_K: 144 B = {fp16 d, fp16 dmin, 12 B 6-bit scales/mins, 128 B nibbles}
// ===========================================================================
template <> struct Mmvq<LSG_GGUF_Q4_K> {
    static constexpr int UV = 256;
    static constexpr int NS = 8;
    static constexpr SumKind SUM = kSumF32Per32;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        uint32_t blk[RW], sc[RW][2], mn[RW][2];
        float d[RW], dmin[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            blk[r] = row[r] + u * 144;
            const uint4 h = lds128(blk[r]);
            d[r] = fp16_bits_to_float(h.x);
            dmin[r] = fp16_bits_to_float(h.x >> 16);
            k4_unpack_all(h.y, h.z, h.w, sc[r], mn[r]);
        }
        float s1[RW * MT], s2[RW * MT];
#pragma unroll
        for (int i = 0; i < RW * MT; ++i) { s1[i] = 0.0f; s2[i] = 0.0f; }

#pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint32_t lo[RW][8], hi[RW][8];
            int sc_lo[RW], sc_hi[RW];
            float m_lo[RW], m_hi[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                uint32_t q[8];
                unpack4(lds128(blk[r] + 16 + 32 * p), q);
                unpack4(lds128(blk[r] + 32 + 32 * p), q + 4);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    lo[r][i] = q[i] & 0x0F0F0F0Fu;
                    hi[r][i] = q[i] & 0xF0F0F0F0u;  // value * 16, dotted in place
                }
                sc_lo[r] = zext8(sc[r][p >> 1], 2 * (p & 1));
                sc_hi[r] = zext8(sc[r][p >> 1], 2 * (p & 1) + 1);
                m_lo[r] = static_cast<float>(zext8(mn[r][p >> 1], 2 * (p & 1)));
                m_hi[r] = static_cast<float>(zext8(mn[r][p >> 1], 2 * (p & 1) + 1));
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
                uint32_t x[16];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    unpack4(lds128(xrow + ((4 * p + j) * xv.U + u) * 16), x + 4 * j);
                const uint32_t off = ((p >> 1) * xv.U + u) * 16 + (p & 1) * 8;
                const uint2 dx = lds64(xrow + xv.d_off + off);
                const uint2 sx = lds64(xrow + xv.s_off + off);
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    int d0 = 0, d1 = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        d0 = dp4a_us(lo[r][i], static_cast<int>(x[i]), d0);
                        d1 = dp4a_us(hi[r][i], static_cast<int>(x[8 + i]), d1);
                    }
                    s1[r * MT + m] += __uint_as_float(dx.x) * static_cast<float>(d0 * sc_lo[r]) +
                                      __uint_as_float(dx.y) * (static_cast<float>(d1 * sc_hi[r]) * 0.0625f);
                    s2[r * MT + m] += m_lo[r] * __uint_as_float(sx.x) + m_hi[r] * __uint_as_float(sx.y);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m)
                acc[r * MT + m] += d[r] * s1[r * MT + m] - dmin[r] * s2[r * MT + m];
    }
};

// ===========================================================================
// Q5_K: 176 B = {d, dmin, 12 B scales, 32 B fifth bits, 128 B nibbles}
// ===========================================================================
template <> struct Mmvq<LSG_GGUF_Q5_K> {
    static constexpr int UV = 256;
    static constexpr int NS = 8;
    static constexpr SumKind SUM = kSumF32Per32;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        uint32_t blk[RW], sc[RW][2], mn[RW][2], qh[RW][8];
        float d[RW], dmin[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            blk[r] = row[r] + u * 176;
            const uint4 h = lds128(blk[r]);
            d[r] = fp16_bits_to_float(h.x);
            dmin[r] = fp16_bits_to_float(h.x >> 16);
            k4_unpack_all(h.y, h.z, h.w, sc[r], mn[r]);
            unpack4(lds128(blk[r] + 16), qh[r]);
            unpack4(lds128(blk[r] + 32), qh[r] + 4);
        }
        float s1[RW * MT], s2[RW * MT];
#pragma unroll
        for (int i = 0; i < RW * MT; ++i) { s1[i] = 0.0f; s2[i] = 0.0f; }

#pragma unroll
        for (int p = 0; p < 4; ++p) {
            uint32_t lo[RW][8], hi[RW][8];
            int sc_lo[RW], sc_hi[RW];
            float m_lo[RW], m_hi[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                uint32_t q[8];
                unpack4(lds128(blk[r] + 48 + 32 * p), q);
                unpack4(lds128(blk[r] + 64 + 32 * p), q + 4);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    lo[r][i] = (q[i] & 0x0F0F0F0Fu) | (((qh[r][i] >> (2 * p)) & 0x01010101u) << 4);
                    hi[r][i] = ((q[i] >> 4) & 0x0F0F0F0Fu) |
                               (((qh[r][i] >> (2 * p + 1)) & 0x01010101u) << 4);
                }
                sc_lo[r] = zext8(sc[r][p >> 1], 2 * (p & 1));
                sc_hi[r] = zext8(sc[r][p >> 1], 2 * (p & 1) + 1);
                m_lo[r] = static_cast<float>(zext8(mn[r][p >> 1], 2 * (p & 1)));
                m_hi[r] = static_cast<float>(zext8(mn[r][p >> 1], 2 * (p & 1) + 1));
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
                uint32_t x[16];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    unpack4(lds128(xrow + ((4 * p + j) * xv.U + u) * 16), x + 4 * j);
                const uint32_t off = ((p >> 1) * xv.U + u) * 16 + (p & 1) * 8;
                const uint2 dx = lds64(xrow + xv.d_off + off);
                const uint2 sx = lds64(xrow + xv.s_off + off);
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    int d0 = 0, d1 = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        d0 = dp4a_us(lo[r][i], static_cast<int>(x[i]), d0);
                        d1 = dp4a_us(hi[r][i], static_cast<int>(x[8 + i]), d1);
                    }
                    s1[r * MT + m] += __uint_as_float(dx.x) * static_cast<float>(d0 * sc_lo[r]) +
                                      __uint_as_float(dx.y) * static_cast<float>(d1 * sc_hi[r]);
                    s2[r * MT + m] += m_lo[r] * __uint_as_float(sx.x) + m_hi[r] * __uint_as_float(sx.y);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m)
                acc[r * MT + m] += d[r] * s1[r * MT + m] - dmin[r] * s2[r * MT + m];
    }
};

// ===========================================================================
// Q6_K: 210 B = {128 B low nibbles, 64 B high 2 bits, 16 int8 scales, fp16 d}
// unit = one 128-value half ip; value (quad q, l) sits at 32q + l of the unit,
// low bits in ql[64ip + 32(q&1) + l] nibble (q>>1), high bits qh[32ip + l] >> 2q,
// scale index 8ip + 2q + l/16.
// ===========================================================================
template <> struct Mmvq<LSG_GGUF_Q6_K> {
    static constexpr int UV = 128;
    static constexpr int NS = 8;
    static constexpr SumKind SUM = kSumI32Per16;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        const int ip = u & 1;
        uint32_t blk[RW], scw[RW][2];
        float d[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            blk[r] = row[r] + (u >> 1) * 210;
            d[r] = fp16_bits_to_float(lds16(blk[r] + 208));
            lds_words_unaligned<2>(blk[r] + 192 + 8 * ip, scw[r]);
        }
        float s1[RW * MT];
#pragma unroll
        for (int i = 0; i < RW * MT; ++i) s1[i] = 0.0f;

#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
            uint32_t v[RW][4][4];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                uint32_t la[4], lb[4], qh[4];
                lds_words_unaligned<4>(blk[r] + 64 * ip + 16 * hs, la);
                lds_words_unaligned<4>(blk[r] + 64 * ip + 32 + 16 * hs, lb);
                lds_words_unaligned<4>(blk[r] + 128 + 32 * ip + 16 * hs, qh);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    v[r][0][i] = (la[i] & 0x0F0F0F0Fu) | ((qh[i] << 4) & 0x30303030u);
                    v[r][1][i] = (lb[i] & 0x0F0F0F0Fu) | ((qh[i] << 2) & 0x30303030u);
                    v[r][2][i] = ((la[i] >> 4) & 0x0F0F0F0Fu) | (qh[i] & 0x30303030u);
                    v[r][3][i] = ((lb[i] >> 4) & 0x0F0F0F0Fu) | ((qh[i] >> 2) & 0x30303030u);
                }
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
                float dx[4];
                uint32_t is0[4], is1[4];
                unpack4f(lds128(xrow + xv.d_off + u * 16), dx);
                unpack4(lds128(xrow + xv.s_off + u * 16), is0);             // sums 0..3
                unpack4(lds128(xrow + xv.s_off + (xv.U + u) * 16), is1);    // sums 4..7
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t x[4];
                    unpack4(lds128(xrow + ((2 * q + hs) * xv.U + u) * 16), x);
                    const int e = 2 * q + hs;  // 16-value group of the unit
                    const int isum = static_cast<int>(e < 4 ? is0[e & 3] : is1[e & 3]);
#pragma unroll
                    for (int r = 0; r < RW; ++r) {
                        int dt = 0;
#pragma unroll
                        for (int i = 0; i < 4; ++i) dt = dp4a_us(v[r][q][i], static_cast<int>(x[i]), dt);
                        const int sc = sext8(scw[r][e >> 2], e & 3);
                        s1[r * MT + m] += dx[q] * static_cast<float>((dt - 32 * isum) * sc);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r * MT + m] += d[r] * s1[r * MT + m];
    }
};

// ===========================================================================
// Q2_K: 84 B = {16 B (scale | min<<4), 64 B 2-bit quants, fp16 d, fp16 dmin}
// unit = half n; value (quad q, l) = (qs[32n + l] >> 2q) & 3, scale byte 8n + 2q + l/16.
// ===========================================================================
template <> struct Mmvq<LSG_GGUF_Q2_K> {
    static constexpr int UV = 128;
    static constexpr int NS = 8;
    static constexpr SumKind SUM = kSumF32Per16;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        const int n = u & 1;
        uint32_t blk[RW], scw[RW][2];
        float d[RW], dmin[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            blk[r] = row[r] + (u >> 1) * 84;
            const uint32_t dm = lds32(blk[r] + 80);  // 84-byte blocks keep 4-byte alignment
            d[r] = fp16_bits_to_float(dm);
            dmin[r] = fp16_bits_to_float(dm >> 16);
            scw[r][0] = lds32(blk[r] + 8 * n);
            scw[r][1] = lds32(blk[r] + 8 * n + 4);
        }
        float s1[RW * MT], s2[RW * MT];
#pragma unroll
        for (int i = 0; i < RW * MT; ++i) { s1[i] = 0.0f; s2[i] = 0.0f; }

#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
            uint32_t w[RW][4];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
#pragma unroll
                for (int i = 0; i < 4; ++i) w[r][i] = lds32(blk[r] + 16 + 32 * n + 16 * hs + 4 * i);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
                float dx[4], fs0[4], fs1[4];
                unpack4f(lds128(xrow + xv.d_off + u * 16), dx);
                unpack4f(lds128(xrow + xv.s_off + u * 16), fs0);
                unpack4f(lds128(xrow + xv.s_off + (xv.U + u) * 16), fs1);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t x[4];
                    unpack4(lds128(xrow + ((2 * q + hs) * xv.U + u) * 16), x);
                    const int e = 2 * q + hs;
                    const float fsum = e < 4 ? fs0[e & 3] : fs1[e & 3];
#pragma unroll
                    for (int r = 0; r < RW; ++r) {
                        int dt = 0;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            dt = dp4a_us((w[r][i] >> (2 * q)) & 0x03030303u, static_cast<int>(x[i]), dt);
                        const int sb = zext8(scw[r][e >> 2], e & 3);
                        s1[r * MT + m] += dx[q] * static_cast<float>(dt * (sb & 0xF));
                        s2[r * MT + m] += static_cast<float>(sb >> 4) * fsum;
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m)
                acc[r * MT + m] += d[r] * s1[r * MT + m] - dmin[r] * s2[r * MT + m];
    }
};

// ===========================================================================
// Q3_K: 110 B = {32 B high-bit mask, 64 B low 2 bits, 12 B 6-bit scales, fp16 d}
// unit = half n; value (j, l) = ((qs[32n + l] >> 2j) & 3) - (hmask[l] bit (4n+j) ? 0 : 4),
// scale index 8n + 2j + l/16, scale = 6-bit value - 32.
// ===========================================================================
template <> struct Mmvq<LSG_GGUF_Q3_K> {
    static constexpr int UV = 128;
    static constexpr int NS = 8;
    static constexpr SumKind SUM = kSumI32Per16;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        const int n = u & 1;
        uint32_t blk[RW];
        int sc[RW][8];  // scale of group e = 2j + hs
        float d[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            blk[r] = row[r] + (u >> 1) * 110;
            d[r] = fp16_bits_to_float(lds16(blk[r] + 108));
            uint32_t sw[3];
            lds_words_unaligned<3>(blk[r] + 96, sw);
            // scale index is = 8n + e: low nibble from byte e (low half for n = 0, high
            // half for n = 1), top 2 bits from byte 8 + (e & 3) at bit 2*(2n + (e >> 2)).
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t lowbyte = (sw[e >> 2] >> (8 * (e & 3))) & 0xFFu;
                const uint32_t low4 = (lowbyte >> (4 * n)) & 0xFu;
                const uint32_t hb = (sw[2] >> (8 * (e & 3))) & 0xFFu;
                const uint32_t hi2 = (hb >> (2 * (2 * n + (e >> 2)))) & 3u;
                sc[r][e] = static_cast<int>(low4 | (hi2 << 4)) - 32;
            }
        }
        float s1[RW * MT];
#pragma unroll
        for (int i = 0; i < RW * MT; ++i) s1[i] = 0.0f;

#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
            uint32_t wq[RW][4], wh[RW][4];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                lds_words_unaligned<4>(blk[r] + 32 + 32 * n + 16 * hs, wq[r]);
                lds_words_unaligned<4>(blk[r] + 16 * hs, wh[r]);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
                float dx[4];
                uint32_t is0[4], is1[4];
                unpack4f(lds128(xrow + xv.d_off + u * 16), dx);
                unpack4(lds128(xrow + xv.s_off + u * 16), is0);
                unpack4(lds128(xrow + xv.s_off + (xv.U + u) * 16), is1);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t x[4];
                    unpack4(lds128(xrow + ((2 * j + hs) * xv.U + u) * 16), x);
                    const int e = 2 * j + hs;
                    const int isum = static_cast<int>(e < 4 ? is0[e & 3] : is1[e & 3]);
#pragma unroll
                    for (int r = 0; r < RW; ++r) {
                        int dt = 0;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const uint32_t q2 = (wq[r][i] >> (2 * j)) & 0x03030303u;
                            const uint32_t hb = (wh[r][i] >> (4 * n + j)) & 0x01010101u;
                            dt = dp4a_us(q2 | (hb << 2), static_cast<int>(x[i]), dt);
                        }
                        s1[r * MT + m] += dx[j] * static_cast<float>((dt - 4 * isum) * sc[r][e]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r)
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[r * MT + m] += d[r] * s1[r * MT + m];
    }
};

// ===========================================================================
// 32-value blocks: Q8_0 (34 B), Q4_0 (18 B), MXFP4 (17 B)
// ===========================================================================
template <> struct Mmvq<LSG_GGUF_Q8_0> {
    static constexpr int UV = 32;
    static constexpr int NS = 0;
    static constexpr SumKind SUM = kSumNone;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        uint32_t w[RW][8];
        float d[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const uint32_t blk = row[r] + u * 34;
            d[r] = fp16_bits_to_float(lds16(blk));
            lds_words_unaligned<8>(blk + 2, w[r]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
            uint32_t x[8];
            unpack4(lds128(xrow + u * 16), x);
            unpack4(lds128(xrow + (xv.U + u) * 16), x + 4);
            const float dx = __uint_as_float(lds32(xrow + xv.d_off + u * 4));
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int dt = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) dt = dp4a_ss(static_cast<int>(w[r][i]), static_cast<int>(x[i]), dt);
                acc[r * MT + m] += (d[r] * dx) * static_cast<float>(dt);
            }
        }
    }
};

// Q4_0: {fp16 d, 16 B nibbles}; low nibble = value j, high nibble = value j+16;
// w = d * (q - 8).  Not in the reference; the block rule is ggml's.
template <> struct Mmvq<LSG_GGUF_Q4_0> {
    static constexpr int UV = 32;
    static constexpr int NS = 1;
    static constexpr SumKind SUM = kSumF32Per32;

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        uint32_t lo[RW][4], hi[RW][4];
        float d[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const uint32_t blk = row[r] + u * 18;
            d[r] = fp16_bits_to_float(lds16(blk));
            uint32_t q[4];
            lds_words_unaligned<4>(blk + 2, q);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                lo[r][i] = q[i] & 0x0F0F0F0Fu;
                hi[r][i] = q[i] & 0xF0F0F0F0u;
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
            uint32_t x[8];
            unpack4(lds128(xrow + u * 16), x);
            unpack4(lds128(xrow + (xv.U + u) * 16), x + 4);
            const float dx = __uint_as_float(lds32(xrow + xv.d_off + u * 4));
            const float sx = __uint_as_float(lds32(xrow + xv.s_off + u * 4));
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int d0 = 0, d1 = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    d0 = dp4a_us(lo[r][i], static_cast<int>(x[i]), d0);
                    d1 = dp4a_us(hi[r][i], static_cast<int>(x[4 + i]), d1);
                }
                const int dt = d0 + (d1 >> 4);  // d1 is an exact multiple of 16
                acc[r * MT + m] += d[r] * (dx * static_cast<float>(dt) - 8.0f * sx);
            }
        }
    }
};

// MXFP4: {E8M0 exponent, 16 B e2m1 codes}; low nibble = value j, high = j+16;
// value = table[code] * 2^(e-128) with the table holding twice the e2m1 value.
template <> struct Mmvq<LSG_GGUF_MXFP4> {
    static constexpr int UV = 32;
    static constexpr int NS = 0;
    static constexpr SumKind SUM = kSumNone;

    // Eight 4-bit codes -> eight signed bytes with three byte permutes per half:
    // magnitudes from an 8-entry table selected by the low 3 bits, negated entries
    // from a second table, bit 3 choosing between the two.
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

    template <int RW, int MT>
    __device__ static __forceinline__ void unit_dot(const uint32_t (&row)[RW], int u,
                                                    const XView& xv, float (&acc)[RW * MT]) {
        uint32_t lo[RW][4], hi[RW][4];
        float d[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const uint32_t blk = row[r] + u * 17;
            d[r] = e8m0_half_scale(lds8(blk));
            uint32_t q[4];
            lds_words_unaligned<4>(blk + 1, q);
#pragma unroll
            for (int i = 0; i < 4; ++i) lookup8(q[i], lo[r][i], hi[r][i]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const uint32_t xrow = xv.base + min(m, xv.mlast) * xv.rowb;
            uint32_t x[8];
            unpack4(lds128(xrow + u * 16), x);
            unpack4(lds128(xrow + (xv.U + u) * 16), x + 4);
            const float dx = __uint_as_float(lds32(xrow + xv.d_off + u * 4));
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                int dt = 0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    dt = dp4a_ss(static_cast<int>(lo[r][i]), static_cast<int>(x[i]), dt);
                    dt = dp4a_ss(static_cast<int>(hi[r][i]), static_cast<int>(x[4 + i]), dt);
                }
                acc[r * MT + m] += (d[r] * dx) * static_cast<float>(dt);
            }
        }
    }
};

#endif  // __CUDACC__

}  // namespace lsg
