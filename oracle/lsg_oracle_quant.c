/*
 * CPU oracle, part 2: FP8 and NVFP4 activation quantizers.  TEST INFRASTRUCTURE ONLY.
 * Each function cites the reference file:line it follows.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

static float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* fp32 -> fp8 e4m3 (1-4-3, bias 7, max 448, no infinities), round to nearest even,
 * saturating to +-448; NaN -> 0x7F.  What cvt.rn.satfinite.e4m3x2.f32 does, which is what
 * the reference's __nv_fp8_e4m3(float) constructor issues. */
ORACLE_API uint8_t oracle_f32_to_e4m3(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint8_t sign = (uint8_t)((x >> 24) & 0x80u);
    const uint32_t ax = x & 0x7FFFFFFFu;
    if (ax > 0x7F800000u) return (uint8_t)(sign | 0x7F);
    float a;
    memcpy(&a, &ax, 4);
    if (a >= 464.0f) return (uint8_t)(sign | 0x7E); /* 464 is the tie between 448 and "480" */
    if (a < 0.0009765625f) return sign;             /* below half the smallest subnormal 2^-9: 2^-10 ties to even = 0 */
    int e;
    (void)frexpf(a, &e);                             /* a = m * 2^e, m in [0.5,1) -> exponent e-1 */
    int exp = e - 1;
    if (exp < -6) exp = -6;                          /* subnormal range shares the exponent of 2^-6 */
    const float ulp = ldexpf(1.0f, exp - 3);
    float q = a / ulp;                               /* exact: power-of-two scaling */
    float r = nearbyintf(q);                         /* default rounding mode: nearest even */
    float val = r * ulp;
    /* encode val (exactly representable now) */
    if (val == 0.0f) return sign;
    int e2;
    float m = frexpf(val, &e2);                      /* val = m * 2^e2, m in [0.5,1) */
    int ex = e2 - 1;
    uint8_t bits;
    if (ex < -6) {                                   /* subnormal: val = k * 2^-9 */
        bits = (uint8_t)(int)(val * 512.0f);
    } else {
        const int mant = (int)((m * 2.0f - 1.0f) * 8.0f);
        bits = (uint8_t)(((ex + 7) << 3) | mant);
    }
    if (bits > 0x7E) bits = 0x7E;
    return (uint8_t)(sign | bits);
}

ORACLE_API float oracle_e4m3_to_f32(uint8_t b) {
    const int sign = b & 0x80;
    const int ex = (b >> 3) & 0xF, mant = b & 7;
    float v;
    if (ex == 0xF && mant == 7) v = NAN;
    else if (ex == 0) v = (float)mant * 0.001953125f;              /* mant * 2^-9 */
    else v = ldexpf(1.0f + (float)mant / 8.0f, ex - 7);
    return sign ? -v : v;
}

/* csrc/smxx/quant/dynamic_fp8_quant.cu:38-112.  scales: [M, ceil(K/128)] row-major, or
 * [ceil(K/128), M] when m_major. */
ORACLE_API void oracle_dynamic_fp8_quant(const uint16_t* x_bf16, uint8_t* out, float* scales,
                                         int M, int K, int m_major) {
    const int nb = (K + 127) / 128;
    for (int r = 0; r < M; ++r)
        for (int b = 0; b < nb; ++b) {
            const int c0 = b * 128, c1 = (c0 + 128 < K) ? c0 + 128 : K;
            float amax = 0.0f;
            for (int c = c0; c < c1; ++c) amax = fmaxf(amax, fabsf(bf16_to_f32(x_bf16[(long)r * K + c])));
            const volatile float scale = (amax > 0.0f) ? (amax / 448.0f) : 1.0f;
            const volatile float inv = 1.0f / scale;
            scales[m_major ? ((long)b * M + r) : ((long)r * nb + b)] = scale;
            for (int c = c0; c < c1; ++c) {
                volatile float s = bf16_to_f32(x_bf16[(long)r * K + c]) * inv;
                float t = fminf(fmaxf(s, -448.0f), 448.0f);
                out[(long)r * K + c] = oracle_f32_to_e4m3(t);
            }
        }
}

/* bf16_to_nvfp4_grouped_detail.cuh:30-50 */
static int sf_offset(int row, int g, int padded_groups) {
    const int tile_row = row / 128, tile_grp = g / 4;
    const int rit = row % 128, git = g % 4;
    const int ntg = (padded_groups + 3) / 4;
    return (tile_row * ntg + tile_grp) * 512 + (rit % 32) * 16 + (rit / 32) * 4 + git;
}

/* bf16_to_nvfp4_grouped_detail.cuh:54-60 */
static uint8_t to_fp4(float v) {
    const uint8_t sign = (v < 0.0f) ? 8 : 0;
    const float a = fabsf(v);
    const uint8_t idx = (uint8_t)((a >= 0.25f) + (a >= 0.75f) + (a >= 1.25f) + (a >= 1.75f) +
                                  (a >= 2.5f) + (a >= 3.5f) + (a >= 5.0f));
    return idx | sign;
}

/* csrc/smxx/quant/bf16_to_nvfp4_grouped.cu:16-97 on values that are already bf16
 * (for the SwiGLU variant the caller passes the bf16-rounded activation).
 * sf_offsets_out[E+1] is computed as the binding does (bindings_python.cu:312-326);
 * scales must be zero-filled and hold sf_offsets_out[E] * K/16 bytes. */
ORACLE_API int oracle_nvfp4_sf_offsets(const int32_t* offs, int32_t* sf, int E) {
    int acc = 0;
    for (int e = 0; e <= E; ++e) {
        sf[e] = acc;
        if (e < E) acc += ((offs[e + 1] - offs[e] + 127) / 128) * 128;
    }
    return acc;
}

ORACLE_API void oracle_bf16_to_nvfp4_grouped(const uint16_t* x_bf16, uint8_t* packed,
                                             uint8_t* scales, const int32_t* offs,
                                             const int32_t* sf, const float* input_scales,
                                             int T, int E, int K) {
    const int gpr = K / 16;
    const int padded_groups = ((gpr + 3) / 4) * 4;
    for (int row = 0; row < T; ++row) {
        int e = 0;
        while (e < E - 1 && offs[e + 1] <= row) ++e; /* find_expert, :81-92 of the detail header */
        const int local_row = row - offs[e];
        float is = 1.0f;
        if (input_scales && input_scales[e] > 0.0f) is = input_scales[e];
        const long sf_base = (long)sf[e] * gpr;
        for (int g = 0; g < gpr; ++g) {
            float vals[16], amax = 0.0f;
            for (int i = 0; i < 16; ++i) {
                vals[i] = bf16_to_f32(x_bf16[(long)row * K + g * 16 + i]);
                amax = fmaxf(amax, fabsf(vals[i]));
            }
            const volatile float six_is = 6.0f * is;
            volatile float scale = amax / six_is;
            scale = fmaxf(scale, 0.001953125f);
            const uint8_t sbits = oracle_f32_to_e4m3(fminf(fmaxf(scale, 0.0f), 480.0f));
            float srepr = oracle_e4m3_to_f32(sbits);
            srepr = fmaxf(srepr, 1e-12f);
            scales[sf_base + sf_offset(local_row, g, padded_groups)] = sbits;
            const volatile float denom = srepr * is;
            const volatile float inv = 1.0f / denom;
            for (int i = 0; i < 16; i += 2) {
                const volatile float v0 = vals[i] * inv, v1 = vals[i + 1] * inv;
                packed[(long)row * (K / 2) + (g * 16 + i) / 2] =
                    (uint8_t)((to_fp4(v0) & 0xF) | ((to_fp4(v1) & 0xF) << 4));
            }
        }
    }
}
