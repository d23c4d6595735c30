/*
 * CPU oracle: a plain-C restatement of the reference algorithms on the GGUF
 * decode path.  TEST INFRASTRUCTURE ONLY - the library never links or calls
 * this; only the tests, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Each function cites the reference file:line it follows (paths relative to
 * the root of kkontosis/LayerStoRmGemmKernels).  The restatement keeps the
 * reference's own decomposition (one 4-value group at a time, w = A*Q + B),
 * which is deliberately NOT how the CUDA kernels regroup the math, so the two
 * are independent derivations of the same numbers.
 *
 * Build: see oracle/Makefile (gcc -O2 -shared -fPIC, no dependencies).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* Scalar conversions                                                       */
/* ------------------------------------------------------------------------ */
static float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3FFu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7F800000u | (man << 13);
    } else {
        u = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* fp32 -> fp16, round to nearest even (what __float2half does). */
static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    const uint32_t absx = x & 0x7FFFFFFFu;
    if (absx > 0x7F800000u) return (uint16_t)(sign | 0x7E00u);            /* NaN */
    if (absx >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);           /* >= 65520 -> inf */
    if (absx < 0x33000001u) return sign;                                   /* < 2^-25 (ties to 0) */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint16_t base;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint16_t)((e + 15) << 10);
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    return (uint16_t)(sign | (uint16_t)(base + q)); /* carry into the exponent is correct */
}

static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ------------------------------------------------------------------------ */
/* Block sizes (gguf_dequant_gemm.cu:292-307; Q4_0 = ggml's 18-byte block)   */
/* ------------------------------------------------------------------------ */
enum { T_Q2_K = 0, T_Q3_K, T_Q4_K, T_Q5_K, T_Q6_K, T_Q8_0, T_MXFP4, T_Q4_0 };

ORACLE_API int oracle_block_values(int type) {
    switch (type) {
        case T_Q2_K: case T_Q3_K: case T_Q4_K: case T_Q5_K: case T_Q6_K: return 256;
        case T_Q8_0: case T_MXFP4: case T_Q4_0: return 32;
    }
    return 0;
}

ORACLE_API int oracle_block_bytes(int type) {
    static const int b[8] = {84, 110, 144, 176, 210, 34, 17, 18};
    return (type >= 0 && type < 8) ? b[type] : 0;
}

/* ------------------------------------------------------------------------ */
/* Q8_1 quantizer - csrc/sm120/gemm/gguf/gguf_mmvq.cu:42-63                  */
/* One "warp" per 32 values; the sum is the 16,8,4,2,1 xor butterfly in fp32. */
/* out: M*(K/32) blocks of {fp16 d, fp16 sum, int8 q[32]} (q8_1_format.h:27) */
/* ------------------------------------------------------------------------ */
ORACLE_API void oracle_quantize_q8_1(const uint16_t* x_bf16, uint8_t* out, int M, int K) {
    const long nblk = (long)M * (K / 32);
    for (long b = 0; b < nblk; ++b) {
        float xi[32], amax[32], sum[32];
        for (int l = 0; l < 32; ++l) {
            xi[l] = bf16_to_f32(x_bf16[b * 32 + l]);
            amax[l] = fabsf(xi[l]);
            sum[l] = xi[l];
        }
        for (int o = 16; o > 0; o >>= 1) {
            float a2[32], s2[32];
            for (int l = 0; l < 32; ++l) {
                a2[l] = fmaxf(amax[l], amax[l ^ o]);
                s2[l] = sum[l] + sum[l ^ o];
            }
            memcpy(amax, a2, sizeof a2);
            memcpy(sum, s2, sizeof s2);
        }
        const volatile float d = amax[0] / 127.0f;
        uint8_t* blk = out + b * 36;
        const uint16_t dh = f32_to_f16(d), sh = f32_to_f16(sum[0]);
        blk[0] = (uint8_t)(dh & 0xFF); blk[1] = (uint8_t)(dh >> 8);
        blk[2] = (uint8_t)(sh & 0xFF); blk[3] = (uint8_t)(sh >> 8);
        for (int l = 0; l < 32; ++l) {
            int q = 0;
            if (amax[0] != 0.0f) {
                const volatile float r = xi[l] / d;
                q = (int)lrintf(r); /* round-half-even, as __float2int_rn */
            }
            blk[4 + l] = (uint8_t)(int8_t)q;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Helpers shared by the decoders                                            */
/* ------------------------------------------------------------------------ */
/* csrc/formats/kquant_common.h:36-46 */
static void scale_min_k4(int j, const uint8_t* q, int* d, int* m) {
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

/* csrc/formats/q3k_format.h:79-84 */
static int q3k_us(int is, const uint8_t* sc) {
    return is < 4  ? (sc[is] & 0xF) | (((sc[is + 8] >> 0) & 3) << 4)
         : is < 8  ? (sc[is] & 0xF) | (((sc[is + 4] >> 2) & 3) << 4)
         : is < 12 ? (sc[is - 8] >> 4) | (((sc[is] >> 4) & 3) << 4)
                   : (sc[is - 8] >> 4) | (((sc[is - 4] >> 6) & 3) << 4);
}

/* csrc/formats/mxfp4_format.h:96-104 */
static float e8m0_half(uint8_t x) {
    uint32_t bits = (x < 2) ? (0x00200000u << x) : ((uint32_t)(x - 1) << 23);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* csrc/formats/mxfp4_format.h:71-76 */
static int mxfp4_value(int code) {
    static const int8_t k[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
    return k[code & 0xF];
}

/* ------------------------------------------------------------------------ */
/* Integer form of one weight value: w[i] = A * Q + B                        */
/* (csrc/sm120/gemm/gguf/gguf_int_policy.h:62-230), i = position in block.   */
/* ------------------------------------------------------------------------ */
static void int_form(int type, const uint8_t* b, int i, int* Q, float* A, float* B) {
    switch (type) {
        case T_Q8_0: { /* :62-76 */
            *Q = (int8_t)b[2 + i];
            *A = f16_to_f32(rd16(b));
            *B = 0.0f;
            return;
        }
        case T_MXFP4: { /* :78-110: low nibbles first 16 values, high nibbles last 16 */
            const uint8_t byte = b[1 + (i & 15)];
            *Q = mxfp4_value(i < 16 ? (byte & 0xF) : (byte >> 4));
            *A = e8m0_half(b[0]);
            *B = 0.0f;
            return;
        }
        case T_Q4_0: { /* ggml block_q4_0: w = d * (q - 8) */
            const uint8_t byte = b[2 + (i & 15)];
            *Q = (i < 16 ? (byte & 0xF) : (byte >> 4)) - 8;
            *A = f16_to_f32(rd16(b));
            *B = 0.0f;
            return;
        }
        case T_Q4_K: { /* :112-131 */
            const float dw = f16_to_f32(rd16(b)), dmw = f16_to_f32(rd16(b + 2));
            const int pair = i / 64, within = i % 64, half = within / 32, l = within % 32;
            int sc, m;
            scale_min_k4(2 * pair + half, b + 4, &sc, &m);
            *A = dw * (float)sc;
            *B = -dmw * (float)m;
            const uint8_t byte = b[16 + pair * 32 + l];
            *Q = half ? (byte >> 4) : (byte & 0xF);
            return;
        }
        case T_Q5_K: { /* :133-160 */
            const float dw = f16_to_f32(rd16(b)), dmw = f16_to_f32(rd16(b + 2));
            const int il = i / 64, within = i % 64, half = within / 32, w = within % 32;
            int sc, m;
            scale_min_k4(2 * il + half, b + 4, &sc, &m);
            *A = dw * (float)sc;
            *B = -dmw * (float)m;
            const uint8_t ql = b[48 + 32 * il + w], qh = b[16 + w];
            const int nib = half ? (ql >> 4) : (ql & 0xF);
            *Q = nib | (((qh >> (2 * il + half)) & 1) << 4);
            return;
        }
        case T_Q6_K: { /* :162-186 */
            const float dw = f16_to_f32(rd16(b + 208));
            const int ip = i / 128, within = i % 128, quad = within / 32, il0 = within % 32;
            *A = dw * (float)(int8_t)b[192 + 8 * ip + il0 / 16 + 2 * quad];
            *B = 0.0f;
            const int qoff = (quad == 1 || quad == 3) ? 32 : 0;
            const uint8_t ql = b[64 * ip + qoff + il0], qh = b[128 + 32 * ip + il0];
            const int nib = (quad >= 2) ? (ql >> 4) : (ql & 0xF);
            *Q = (nib | (((qh >> (2 * quad)) & 3) << 4)) - 32;
            return;
        }
        case T_Q2_K: { /* :188-206 */
            const float dw = f16_to_f32(rd16(b + 80)), dmw = f16_to_f32(rd16(b + 82));
            const int ni = i / 128, within = i % 128, quad = within / 32, l0 = within % 32;
            const uint8_t scb = b[8 * ni + l0 / 16 + 2 * quad];
            *A = dw * (float)(scb & 0xF);
            *B = -dmw * (float)(scb >> 4);
            *Q = (b[16 + 32 * ni + l0] >> (2 * quad)) & 3;
            return;
        }
        case T_Q3_K: { /* :208-230 */
            const float dw = f16_to_f32(rd16(b + 108));
            const int ni = i / 128, within = i % 128, j = within / 32, w32 = within % 32;
            const int is = 8 * ni + 2 * j + w32 / 16;
            *A = dw * (float)(q3k_us(is, b + 96) - 32);
            *B = 0.0f;
            const int q2 = (b[32 + 32 * ni + w32] >> (2 * j)) & 3;
            const int hset = (b[w32] >> (4 * ni + j)) & 1;
            *Q = q2 - 4 + 4 * hset;
            return;
        }
    }
    *Q = 0; *A = 0.0f; *B = 0.0f;
}

/* ------------------------------------------------------------------------ */
/* Block dequant to fp32 - csrc/formats headers, dequant_*_block                  */
/* (q4k_format.h:112-133, q5k:58-86, q6k:60-80, q2k:59-78, q3k:60-95,        */
/*  q8_0:51-58, mxfp4:111-120).  Each value is  A*Q' - M  in the operation    */
/* order those functions use (scale*quant, then minus min).                  */
/* ------------------------------------------------------------------------ */
static void dequant_block(int type, const uint8_t* b, float* out) {
    const int n = oracle_block_values(type);
    switch (type) {
        case T_Q4_K: {
            const float d = f16_to_f32(rd16(b)), dmin = f16_to_f32(rd16(b + 2));
            for (int pair = 0; pair < 4; ++pair) {
                int s0, m0, s1, m1;
                scale_min_k4(2 * pair, b + 4, &s0, &m0);
                scale_min_k4(2 * pair + 1, b + 4, &s1, &m1);
                const float d1 = d * (float)s0, mm1 = dmin * (float)m0;
                const float d2 = d * (float)s1, mm2 = dmin * (float)m1;
                for (int l = 0; l < 32; ++l) {
                    const uint8_t q = b[16 + pair * 32 + l];
                    out[pair * 64 + l] = d1 * (float)(q & 0xF) - mm1;
                    out[pair * 64 + l + 32] = d2 * (float)(q >> 4) - mm2;
                }
            }
            return;
        }
        case T_Q5_K: {
            const float d = f16_to_f32(rd16(b)), dmin = f16_to_f32(rd16(b + 2));
            for (int il = 0; il < 4; ++il) {
                int s0, m0, s1, m1;
                scale_min_k4(2 * il, b + 4, &s0, &m0);
                scale_min_k4(2 * il + 1, b + 4, &s1, &m1);
                const float d1 = d * (float)s0, mm1 = dmin * (float)m0;
                const float d2 = d * (float)s1, mm2 = dmin * (float)m1;
                for (int l = 0; l < 32; ++l) {
                    const uint8_t ql = b[48 + 32 * il + l], qh = b[16 + l];
                    out[64 * il + l] = d1 * (float)((ql & 0xF) + ((qh >> (2 * il)) & 1 ? 16 : 0)) - mm1;
                    out[64 * il + 32 + l] = d2 * (float)((ql >> 4) + ((qh >> (2 * il + 1)) & 1 ? 16 : 0)) - mm2;
                }
            }
            return;
        }
        case T_Q2_K: {
            const float d = f16_to_f32(rd16(b + 80)), dmin = f16_to_f32(rd16(b + 82));
            for (int nn = 0; nn < 2; ++nn)
                for (int l = 0; l < 32; ++l) {
                    const int is = 8 * nn + l / 16;
                    const uint8_t q = b[16 + 32 * nn + l];
                    for (int quad = 0; quad < 4; ++quad) {
                        const uint8_t s = b[is + 2 * quad];
                        out[128 * nn + l + 32 * quad] =
                            d * (float)(s & 0xF) * (float)((q >> (2 * quad)) & 3) - dmin * (float)(s >> 4);
                    }
                }
            return;
        }
        default: { /* types without a min term: value = A * Q exactly as int_form */
            for (int i = 0; i < n; ++i) {
                int Q; float A, B;
                int_form(type, b, i, &Q, &A, &B);
                out[i] = A * (float)Q;
            }
            return;
        }
    }
}

ORACLE_API void oracle_dequant_blocks(int type, const uint8_t* packed, long n_blocks, float* out) {
    const int vals = oracle_block_values(type), bytes = oracle_block_bytes(type);
    for (long b = 0; b < n_blocks; ++b) dequant_block(type, packed + b * bytes, out + b * vals);
}

/* ------------------------------------------------------------------------ */
/* Integer mat-vec - csrc/sm120/gemm/gguf/gguf_mmvq_impl.cuh:43-70           */
/*   C[m,n] = sum over 4-value groups  dx * (A * dp4a(Q,qx) + B * sum(qx))   */
/* xq: Q8_1 blocks [M][K/32][36].  Accumulated in double, so that the result */
/* is the value any fp32 summation order of the same terms rounds around.    */
/* ------------------------------------------------------------------------ */
ORACLE_API void oracle_mmvq(int type, int M, int N, int K, const uint8_t* xq, const uint8_t* W,
                            double* out) {
    const int vals = oracle_block_values(type), bytes = oracle_block_bytes(type);
    const int nblk = K / vals;
    const long row_bytes = (long)nblk * bytes;
    const int xb = K / 32;
    for (int n = 0; n < N; ++n) {
        const uint8_t* wrow = W + (long)n * row_bytes;
        for (int m = 0; m < M; ++m) {
            const uint8_t* xrow = xq + (long)m * xb * 36;
            double acc = 0.0;
            for (int gg = 0; gg < K / 4; ++gg) {
                const int k0 = gg * 4;
                const uint8_t* wb = wrow + (long)(k0 / vals) * bytes;
                const uint8_t* xblk = xrow + (long)(k0 / 32) * 36;
                const float dx = f16_to_f32(rd16(xblk));
                int dot = 0, sumq = 0;
                float A = 0.0f, B = 0.0f;
                for (int t = 0; t < 4; ++t) {
                    int Q;
                    int_form(type, wb, (k0 % vals) + t, &Q, &A, &B);
                    const int qx = (int8_t)xblk[4 + (k0 % 32) + t];
                    dot += Q * qx;
                    sumq += qx;
                }
                acc += (double)dx * ((double)A * dot + (double)B * sumq);
            }
            out[(long)m * N + n] = acc;
        }
    }
}

/* ------------------------------------------------------------------------ */
/* Dequant GEMM - csrc/sm120/gemm/gguf/gguf_dequant_gemm.cu:94-142           */
/*   C[m,n] = sum_k bf16(A[m,k]) * dequant(W)[n,k], double accumulation.     */
/* ------------------------------------------------------------------------ */
ORACLE_API void oracle_dequant_gemm(int type, int M, int N, int K, const uint16_t* A_bf16,
                                    const uint8_t* W, double* out) {
    const int vals = oracle_block_values(type), bytes = oracle_block_bytes(type);
    const int nblk = K / vals;
    float* wrow = (float*)malloc(sizeof(float) * (size_t)K);
    for (int n = 0; n < N; ++n) {
        oracle_dequant_blocks(type, W + (long)n * nblk * bytes, nblk, wrow);
        for (int m = 0; m < M; ++m) {
            double acc = 0.0;
            for (int k = 0; k < K; ++k) acc += (double)bf16_to_f32(A_bf16[(long)m * K + k]) * wrow[k];
            out[(long)m * N + n] = acc;
        }
    }
    free(wrow);
}

/* fp32 <-> fp16 exposed for the tests of the oracle itself */
ORACLE_API uint16_t oracle_f32_to_f16(float f) { return f32_to_f16(f); }
ORACLE_API float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
