/*
 * oracle_port.c -- TEST INFRASTRUCTURE, not product code.
 *
 * Plain-C restatement of the CPU side of the quantized matvec path of ahmed-bensaad/QWENgine:
 * the ggml block layouts, the scalar reference (de)quantizers and the integer dot products of
 * each weight format against Q8_K activations.  Only tests, the smoke check and the CPU-baseline
 * leg of the benchmark may load this library; the CUDA product never does.
 *
 * Pinning: for IQ3_XXS, IQ3_S, IQ4_XS, Q4_K and Q6_K every function here is checked bit-for-bit
 * against the reference's own sources compiled in place (oracle/_ref, built by oracle/Makefile),
 * and the dequantizers of all seven formats against the gguf Python package.  Q5_K has no
 * counterpart at all in the reference and Q8_0 has only a dequantizer there: their dot products
 * are restatements of the K-quant pattern of the reference kernels (parity unpinned by the
 * reference; dequantized values pinned by gguf-py).
 *
 * Each function cites the reference file:line it follows (paths inside the reference project).
 * Compile with -ffp-contract=off: every fused multiply-add below is written out as fmaf().
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define Q38B_CODEBOOK_QUALIFIER static const
#include "../qwengine_b200/csrc/codebooks.inc"

#define QK_K 256

/* ggml type ids, include/q38rt/q38rt_types.h:36-67 */
enum {
    T_Q8_0 = 8, T_Q2_K = 10, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ3_XXS = 18,
    T_IQ1_S = 19, T_IQ3_S = 21, T_IQ2_S = 22, T_IQ4_XS = 23, T_IQ1_M = 29
};

/* ---------------------------------------------------------------------------------------------
 * Block layouts (src/quant/quant_formats.h:87-121; Q5_K: ggml-common.h block_q5_K, 176 bytes,
 * include/q38rt/q38rt_types.h:89 gives only its size).  Accessed through byte offsets so that no
 * packing pragma is needed.
 * ------------------------------------------------------------------------------------------- */
#define BB_Q8_0 34
#define BB_Q4_K 144
#define BB_Q5_K 176
#define BB_Q6_K 210
#define BB_IQ3_XXS 98
#define BB_IQ3_S 110
#define BB_IQ4_XS 136
#define BB_Q8_K 292
#define BB_Q2_K 84
#define BB_IQ2_XXS 66
#define BB_IQ2_XS 74
#define BB_IQ2_S 82
#define BB_IQ1_S 50
#define BB_IQ1_M 56

static inline uint16_t ld16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static inline uint32_t ld32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }

/* src/quant/quant_formats.h:29-51 : exact binary16 -> binary32 including subnormals. */
float q38o_fp16_to_fp32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    int exp = (h >> 10) & 0x1F;
    uint32_t mant = h & 0x3FFu, bits;
    if (exp == 0) {
        if (mant == 0) bits = sign;
        else {
            int e = 127 - 15 + 1;
            while (!(mant & 0x400u)) { mant <<= 1; e--; }
            bits = sign | ((uint32_t)e << 23) | ((mant & 0x3FFu) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (mant << 13);
    else bits = sign | ((uint32_t)(exp + 112) << 23) | (mant << 13);
    float f; memcpy(&f, &bits, 4); return f;
}

/* bfloat16 helpers for the prefill oracle (round to nearest even, as __float2bfloat16_rn). */
uint16_t q38o_fp32_to_bf16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}
float q38o_bf16_to_fp32(uint16_t b) { uint32_t x = (uint32_t)b << 16; float f; memcpy(&f, &x, 4); return f; }

/* float -> binary16 round to nearest even (src/quant/quant_formats.h:53-78), for the f16 weight check. */
uint16_t q38o_fp32_to_fp16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, a = x & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (a > 0x7F800000u ? 0x200u : 0));
    if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (a < 0x38800000u) {
        if (a < 0x33000000u) return (uint16_t)sign;
        const uint32_t e = a >> 23, m = (a & 0x7FFFFFu) | 0x800000u, sh = 126 - e;
        const uint32_t hm = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        return (uint16_t)(sign | (hm + ((rem > half || (rem == half && (hm & 1))) ? 1 : 0)));
    }
    uint32_t r = (a - 0x38000000u) >> 13;
    const uint32_t rem = a & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
    return (uint16_t)(sign | r);
}

size_t q38o_row_bytes(uint32_t t, int K) {
    switch (t) {
        case T_Q8_0: return (size_t)(K / 32) * BB_Q8_0;
        case T_Q4_K: return (size_t)(K / QK_K) * BB_Q4_K;
        case T_Q5_K: return (size_t)(K / QK_K) * BB_Q5_K;
        case T_Q6_K: return (size_t)(K / QK_K) * BB_Q6_K;
        case T_IQ3_XXS: return (size_t)(K / QK_K) * BB_IQ3_XXS;
        case T_IQ3_S: return (size_t)(K / QK_K) * BB_IQ3_S;
        case T_IQ4_XS: return (size_t)(K / QK_K) * BB_IQ4_XS;
        case T_Q2_K: return (size_t)(K / QK_K) * BB_Q2_K;
        case T_IQ2_XXS: return (size_t)(K / QK_K) * BB_IQ2_XXS;
        case T_IQ2_XS: return (size_t)(K / QK_K) * BB_IQ2_XS;
        case T_IQ2_S: return (size_t)(K / QK_K) * BB_IQ2_S;
        case T_IQ1_S: return (size_t)(K / QK_K) * BB_IQ1_S;
        case T_IQ1_M: return (size_t)(K / QK_K) * BB_IQ1_M;
        default: return 0;
    }
}

/* 6-bit scale / min of sub-block j of a Q4_K / Q5_K block: src/quant/quant_ref.cpp:24-32. */
static inline void scale_min_k4(int j, const uint8_t* q, int* sc, int* mn) {
    if (j < 4) { *sc = q[j] & 63; *mn = q[j + 4] & 63; }
    else { *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

/* Sign byte of a 7-bit IQ3_XXS sign index: the 8th bit restores even parity
 * (table ksigns_iq2xs, src/quant/iq_tables.inc:8; same rule as src/cpu/cpu_kernels.cpp:56-58). */
static inline uint32_t ksign8(uint32_t s7) { return s7 | ((uint32_t)__builtin_parity(s7) << 7); }

/* ---------------------------------------------------------------------------------------------
 * Scalar dequantizers: the ground truth for weight values (bit-exact contract).
 * ------------------------------------------------------------------------------------------- */

/* src/quant/quant_ref.cpp:302-308 */
static void dq_q8_0(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / 32; i++, b += BB_Q8_0) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        for (int j = 0; j < 32; j++) y[i * 32 + j] = (float)(int8_t)b[2 + j] * d;
    }
}

/* src/quant/quant_ref.cpp:57-76 */
static void dq_q4_K(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_Q4_K) {
        const float d = q38o_fp16_to_fp32(ld16(b)), mn = q38o_fp16_to_fp32(ld16(b + 2));
        const uint8_t *sc = b + 4, *q = b + 16;
        for (int p = 0; p < 4; p++, q += 32) {
            int s1, m1, s2, m2;
            scale_min_k4(2 * p, sc, &s1, &m1);
            scale_min_k4(2 * p + 1, sc, &s2, &m2);
            const float d1 = d * (float)s1, o1 = mn * (float)m1, d2 = d * (float)s2, o2 = mn * (float)m2;
            for (int l = 0; l < 32; l++) *y++ = d1 * (float)(q[l] & 0xF) - o1;
            for (int l = 0; l < 32; l++) *y++ = d2 * (float)(q[l] >> 4) - o2;
        }
    }
}

/* No reference counterpart (the reference rejects Q5_K, src/runtime/engine.cpp:648-650).  GGUF
 * format definition: d, dmin, 12 scale bytes as Q4_K, qh[32] (bit j of qh[l] = 5th bit of weight l
 * of sub-block j), qs[128] nibbles as Q4_K.  w = d*sc*q - dmin*m with q in 0..31. */
static void dq_q5_K(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_Q5_K) {
        const float d = q38o_fp16_to_fp32(ld16(b)), mn = q38o_fp16_to_fp32(ld16(b + 2));
        const uint8_t *sc = b + 4, *qh = b + 16, *q = b + 48;
        for (int p = 0; p < 4; p++, q += 32) {
            int s1, m1, s2, m2;
            scale_min_k4(2 * p, sc, &s1, &m1);
            scale_min_k4(2 * p + 1, sc, &s2, &m2);
            const float d1 = d * (float)s1, o1 = mn * (float)m1, d2 = d * (float)s2, o2 = mn * (float)m2;
            for (int l = 0; l < 32; l++) *y++ = d1 * (float)((q[l] & 0xF) + (((qh[l] >> (2 * p)) & 1) << 4)) - o1;
            for (int l = 0; l < 32; l++) *y++ = d2 * (float)((q[l] >> 4) + (((qh[l] >> (2 * p + 1)) & 1) << 4)) - o2;
        }
    }
}

/* src/quant/quant_ref.cpp:78-103 */
static void dq_q6_K(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_Q6_K) {
        const float d = q38o_fp16_to_fp32(ld16(b + 208));
        const uint8_t *ql = b, *qh = b + 128;
        const int8_t* sc = (const int8_t*)(b + 192);
        for (int h = 0; h < 2; h++, y += 128, ql += 64, qh += 32, sc += 8)
            for (int l = 0; l < 32; l++) {
                const int is = l / 16;
                const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
                const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                y[l] = d * (float)sc[is] * (float)q1;
                y[l + 32] = d * (float)sc[is + 2] * (float)q2;
                y[l + 64] = d * (float)sc[is + 4] * (float)q3;
                y[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
    }
}

/* src/quant/quant_ref.cpp:165-188 */
static void dq_iq3_xxs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ3_XXS) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        const uint8_t* qs = b + 2;
        for (int s = 0; s < 8; s++, qs += 8) {
            const uint32_t aux = ld32(b + 66 + 4 * s);
            const float db = d * (0.5f + (float)(aux >> 28)) * 0.5f;
            for (int l = 0; l < 4; l++) {
                const uint32_t sg = ksign8((aux >> (7 * l)) & 127);
                const uint32_t g1 = q38b_iq3xxs_grid[qs[2 * l]], g2 = q38b_iq3xxs_grid[qs[2 * l + 1]];
                for (int j = 0; j < 4; j++) {
                    y[j] = db * (float)((g1 >> (8 * j)) & 0xFF) * ((sg >> j) & 1 ? -1.f : 1.f);
                    y[j + 4] = db * (float)((g2 >> (8 * j)) & 0xFF) * ((sg >> (j + 4)) & 1 ? -1.f : 1.f);
                }
                y += 8;
            }
        }
    }
}

/* src/quant/quant_ref.cpp:190-225 */
static void dq_iq3_s(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ3_S) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *scl = b + 106;
        for (int s = 0; s < 8; s++, qs += 8, sg += 4) {
            const int ls = (scl[s / 2] >> (4 * (s & 1))) & 0xF;
            const float db = d * (float)(1 + 2 * ls);
            for (int l = 0; l < 4; l++) {
                const uint32_t g1 = q38b_iq3s_grid[qs[2 * l] | ((qh[s] << (8 - 2 * l)) & 256)];
                const uint32_t g2 = q38b_iq3s_grid[qs[2 * l + 1] | ((qh[s] << (7 - 2 * l)) & 256)];
                for (int j = 0; j < 4; j++) {
                    y[j] = db * (float)((g1 >> (8 * j)) & 0xFF) * ((sg[l] >> j) & 1 ? -1.f : 1.f);
                    y[j + 4] = db * (float)((g2 >> (8 * j)) & 0xFF) * ((sg[l] >> (j + 4)) & 1 ? -1.f : 1.f);
                }
                y += 8;
            }
        }
    }
}

/* 6-bit IQ4_XS sub-block scale: src/quant/quant_ref.cpp:290 */
static inline int iq4xs_ls(const uint8_t* b, int s) {
    const uint32_t sh = ld16(b + 2);
    return (int)(((b[4 + s / 2] >> (4 * (s & 1))) & 0xF) | (((sh >> (2 * s)) & 3) << 4));
}

/* src/quant/quant_ref.cpp:284-300 */
static void dq_iq4_xs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ4_XS) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        const uint8_t* qs = b + 8;
        for (int s = 0; s < 8; s++, qs += 16, y += 32) {
            const float dl = d * (float)(iq4xs_ls(b, s) - 32);
            for (int j = 0; j < 16; j++) {
                y[j] = dl * (float)q38b_iq4nl_levels[qs[j] & 0xF];
                y[j + 16] = dl * (float)q38b_iq4nl_levels[qs[j] >> 4];
            }
        }
    }
}

/* src/quant/quant_ref.cpp:323-351 (the seven formats of the hot path). Returns 0 on success. */
/* Value j (0..7) of an entry of the IQ2 grids ({8, 25, 43}) and of the IQ1 grid ({-1, 0, 1}): the tables keep eight
 * 2-bit level indices per entry (src/quant/iq_tables.inc:12-270, 440-959 hold the same grids as 8 bytes per entry). */
static inline int iq2_grid(uint32_t code, int j) { static const int lv[4] = {8, 25, 43, 0}; return lv[(code >> (2 * j)) & 3]; }
static inline int iq1_grid(uint32_t code, int j) { return (int)((code >> (2 * j)) & 3) - 1; }
#define IQ1S_DELTA 0.125f

/* src/quant/quant_ref.cpp:33-55 */
static void dq_q2_K(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_Q2_K) {
        const float d = q38o_fp16_to_fp32(ld16(b + 80)), mn = q38o_fp16_to_fp32(ld16(b + 82));
        const uint8_t* q = b + 16;
        int is = 0;
        for (int h = 0; h < 2; h++, q += 32) {
            int shift = 0;
            for (int j = 0; j < 4; j++, shift += 2)
                for (int half = 0; half < 2; half++) {
                    const uint8_t sc = b[is++];
                    const float dl = d * (sc & 0xF), ml = mn * (sc >> 4);
                    for (int l = 0; l < 16; l++) *y++ = dl * ((int8_t)((q[l + 16 * half] >> shift) & 3)) - ml;
                }
        }
    }
}

/* src/quant/quant_ref.cpp:105-124 */
static void dq_iq2_xxs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ2_XXS) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        for (int ib = 0; ib < 8; ib++) {
            const uint32_t a0 = ld32(b + 2 + 8 * ib), a1 = ld32(b + 6 + 8 * ib);
            const float db = d * (0.5f + (a1 >> 28)) * 0.25f;
            for (int l = 0; l < 4; l++) {
                const uint32_t code = q38b_iq2xxs_codes[(a0 >> (8 * l)) & 0xFF], sg = ksign8((a1 >> (7 * l)) & 127);
                for (int j = 0; j < 8; j++) *y++ = db * iq2_grid(code, j) * (((sg >> j) & 1) ? -1.f : 1.f);
            }
        }
    }
}

/* src/quant/quant_ref.cpp:126-144 */
static void dq_iq2_xs(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ2_XS) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        for (int ib = 0; ib < 8; ib++) {
            const uint8_t sc = b[66 + ib];
            const float db[2] = {d * (0.5f + (sc & 0xF)) * 0.25f, d * (0.5f + (sc >> 4)) * 0.25f};
            for (int l = 0; l < 4; l++) {
                const uint32_t qv = ld16(b + 2 + 2 * (4 * ib + l));
                const uint32_t code = q38b_iq2xs_codes[qv & 511], sg = ksign8(qv >> 9);
                for (int j = 0; j < 8; j++) *y++ = db[l / 2] * iq2_grid(code, j) * (((sg >> j) & 1) ? -1.f : 1.f);
            }
        }
    }
}

/* src/quant/quant_ref.cpp:146-168 */
static void dq_iq2_s(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ2_S) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        const uint8_t *qs = b + 2, *signs = b + 34, *qh = b + 66, *scl = b + 74;
        for (int ib = 0; ib < 8; ib++) {
            const float db[2] = {d * (0.5f + (scl[ib] & 0xF)) * 0.25f, d * (0.5f + (scl[ib] >> 4)) * 0.25f};
            for (int l = 0; l < 4; l++) {
                const uint32_t code = q38b_iq2s_codes[qs[4 * ib + l] | (((uint32_t)qh[ib] << (8 - 2 * l)) & 0x300)];
                const uint32_t sg = signs[4 * ib + l];
                for (int j = 0; j < 8; j++) *y++ = db[l / 2] * iq2_grid(code, j) * (((sg >> j) & 1) ? -1.f : 1.f);
            }
        }
    }
}

/* src/quant/quant_ref.cpp:227-245 */
static void dq_iq1_s(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ1_S) {
        const float d = q38o_fp16_to_fp32(ld16(b));
        for (int ib = 0; ib < 8; ib++) {
            const uint32_t qh = ld16(b + 34 + 2 * ib);
            const float dl = d * (2 * ((qh >> 12) & 7) + 1);
            const float delta = (qh & 0x8000) ? -IQ1S_DELTA : IQ1S_DELTA;
            for (int l = 0; l < 4; l++) {
                const uint32_t code = q38b_iq1s_codes[b[2 + 4 * ib + l] | (((qh >> (3 * l)) & 7) << 8)];
                for (int j = 0; j < 8; j++) *y++ = dl * (iq1_grid(code, j) + delta);
            }
        }
    }
}

/* src/quant/quant_ref.cpp:247-283 */
static void dq_iq1_m(const uint8_t* b, float* y, int64_t n) {
    for (int64_t i = 0; i < n / QK_K; i++, b += BB_IQ1_M) {
        uint16_t sc[4];
        memcpy(sc, b + 48, 8);
        const uint16_t su = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000));
        const float d = q38o_fp16_to_fp32(su);
        const uint8_t *qs = b, *qh = b + 32;
        for (int ib = 0; ib < 8; ib++, qs += 4, qh += 2) {
            const float dl[2] = {d * (2 * ((sc[ib / 2] >> (6 * (ib % 2) + 0)) & 0x7) + 1), d * (2 * ((sc[ib / 2] >> (6 * (ib % 2) + 3)) & 0x7) + 1)};
            for (int l = 0; l < 4; l++) {
                const uint32_t hn = (qh[l / 2] >> (4 * (l & 1))) & 0xF;       /* this group's nibble: 3 index bits + delta sign */
                const uint32_t code = q38b_iq1s_codes[qs[l] | ((hn & 7) << 8)];
                const float delta = (hn & 8) ? -IQ1S_DELTA : IQ1S_DELTA;
                for (int j = 0; j < 8; j++) *y++ = dl[l / 2] * (iq1_grid(code, j) + delta);
            }
        }
    }
}

int q38o_dequantize_row(uint32_t t, const void* src, float* dst, int64_t n) {
    const uint8_t* b = (const uint8_t*)src;
    switch (t) {
        case T_Q8_0: dq_q8_0(b, dst, n); return 0;
        case T_Q4_K: dq_q4_K(b, dst, n); return 0;
        case T_Q5_K: dq_q5_K(b, dst, n); return 0;
        case T_Q6_K: dq_q6_K(b, dst, n); return 0;
        case T_IQ3_XXS: dq_iq3_xxs(b, dst, n); return 0;
        case T_IQ3_S: dq_iq3_s(b, dst, n); return 0;
        case T_IQ4_XS: dq_iq4_xs(b, dst, n); return 0;
        case T_Q2_K: dq_q2_K(b, dst, n); return 0;
        case T_IQ2_XXS: dq_iq2_xxs(b, dst, n); return 0;
        case T_IQ2_XS: dq_iq2_xs(b, dst, n); return 0;
        case T_IQ2_S: dq_iq2_s(b, dst, n); return 0;
        case T_IQ1_S: dq_iq1_s(b, dst, n); return 0;
        case T_IQ1_M: dq_iq1_m(b, dst, n); return 0;
        default: return -1;
    }
}

/* ---------------------------------------------------------------------------------------------
 * Q8_K activation quantizer: src/quant/quant_ref.cpp:353-381 (nearest_int :17-22).
 * Block = float d, int8 qs[256], int16 bsums[16] (292 bytes).
 * ------------------------------------------------------------------------------------------- */
static inline int nearest_int(float v) {
    float t = v + 12582912.f;
    int i; memcpy(&i, &t, 4);
    return (i & 0x007fffff) - 0x00400000;
}

void q38o_quantize_row_q8_K(const float* x, void* vy, int64_t n) {
    uint8_t* y = (uint8_t*)vy;
    for (int64_t i = 0; i < n / QK_K; i++, x += QK_K, y += BB_Q8_K) {
        float max = 0, amax = 0;
        for (int j = 0; j < QK_K; j++) { const float ax = fabsf(x[j]); if (ax > amax) { amax = ax; max = x[j]; } }
        if (!amax) { memset(y, 0, BB_Q8_K); continue; }
        const float iscale = -127.f / max;
        int8_t* qs = (int8_t*)(y + 4);
        for (int j = 0; j < QK_K; j++) { const int v = nearest_int(iscale * x[j]); qs[j] = (int8_t)(v < 127 ? v : 127); }
        for (int j = 0; j < 16; j++) {
            int sum = 0;
            for (int k = 0; k < 16; k++) sum += qs[16 * j + k];
            const int16_t s16 = (int16_t)sum;
            memcpy(y + 260 + 2 * j, &s16, 2);
        }
        const float d = 1 / iscale;
        memcpy(y, &d, 4);
    }
}

/* ---------------------------------------------------------------------------------------------
 * Dot products against Q8_K.  Structure of the reference AVX2 kernels (src/cpu/cpu_kernels.cpp):
 * per 256-weight block an exact int32 sum per vector lane (lane l = weights 4l..4l+3 of every
 * 32-weight sub-block, each multiplied by its integer sub-block scale), then ONE fused
 * multiply-add per lane with the float block scale, and a fixed-order horizontal sum at the end
 * (hsum8, :25-31).  Restated with 8 scalar lanes so that results are bit-identical.
 * ------------------------------------------------------------------------------------------- */
typedef struct { float acc[8]; float acc_m; } col_acc;

static inline float hsum8(const float* a) {
    /* src/cpu/cpu_kernels.cpp:25-31 */
    const float s0 = a[0] + a[4], s1 = a[1] + a[5], s2 = a[2] + a[6], s3 = a[3] + a[7];
    return (s0 + s2) + (s1 + s3);
}

static inline const int8_t* xq_qs(const uint8_t* xb) { return (const int8_t*)(xb + 4); }
static inline float xq_d(const uint8_t* xb) { float d; memcpy(&d, xb, 4); return d; }
static inline int xq_bsum(const uint8_t* xb, int j) { int16_t s; memcpy(&s, xb + 260 + 2 * j, 2); return s; }

static inline void block_fma(col_acc* c, float scale, const int32_t* sumi) {
    for (int l = 0; l < 8; l++) c->acc[l] = fmaf(scale, (float)sumi[l], c->acc[l]);
}

/* weights w[32] (already signed integers) times the sub-block's activations, times integer scale */
static inline void sub_dot(int32_t* sumi, const int* w, const int8_t* q, int sc) {
    for (int l = 0; l < 8; l++) {
        int s = 0;
        for (int j = 0; j < 4; j++) s += w[4 * l + j] * q[4 * l + j];
        sumi[l] += sc * s;
    }
}

/* src/cpu/cpu_kernels.cpp:164-189 */
static void blk_iq3_xxs(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    const uint8_t* qs = b + 2;
    for (int s = 0; s < 8; s++) {
        const uint32_t aux = ld32(b + 66 + 4 * s);
        int w[32];
        for (int l = 0; l < 4; l++) {
            const uint32_t sg = ksign8((aux >> (7 * l)) & 127);
            for (int h = 0; h < 2; h++) {
                const uint32_t g = q38b_iq3xxs_grid[qs[8 * s + 2 * l + h]];
                for (int j = 0; j < 4; j++) {
                    const int m = (g >> (8 * j)) & 0xFF;
                    w[8 * l + 4 * h + j] = ((sg >> (4 * h + j)) & 1) ? -m : m;
                }
            }
        }
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, (int)(2 * (aux >> 28) + 1));
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb) * 0.25f, sumi);
}

/* src/cpu/cpu_kernels.cpp:130-162 */
static void blk_iq3_s(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *scl = b + 106;
    for (int s = 0; s < 8; s++) {
        int w[32];
        for (int l = 0; l < 4; l++)
            for (int h = 0; h < 2; h++) {
                const int sh = h ? 7 - 2 * l : 8 - 2 * l;
                const uint32_t g = q38b_iq3s_grid[qs[8 * s + 2 * l + h] | ((qh[s] << sh) & 256)];
                for (int j = 0; j < 4; j++) {
                    const int m = (g >> (8 * j)) & 0xFF;
                    w[8 * l + 4 * h + j] = ((sg[4 * s + l] >> (4 * h + j)) & 1) ? -m : m;
                }
            }
        const int ls = (scl[s / 2] >> (4 * (s & 1))) & 0xF;
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, 2 * ls + 1);
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb), sumi);
}

/* src/cpu/cpu_kernels.cpp:351-384 */
static void blk_iq4_xs(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    for (int s = 0; s < 8; s++) {
        const uint8_t* qs = b + 8 + 16 * s;
        int w[32];
        for (int j = 0; j < 16; j++) { w[j] = q38b_iq4nl_levels[qs[j] & 0xF]; w[j + 16] = q38b_iq4nl_levels[qs[j] >> 4]; }
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, iq4xs_ls(b, s) - 32);
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb), sumi);
}

/* src/cpu/cpu_kernels.cpp:386-433.  nbits = 4 restates the reference kernel; nbits = 5 is the
 * same pattern with the fifth bit taken from qh (no reference counterpart). */
static void blk_q45_K(const uint8_t* b, const uint8_t* xb, col_acc* c, int nbits) {
    int32_t sumi[8] = {0};
    const uint8_t *scb = b + 4, *qh = b + 16, *q = b + (nbits == 5 ? 48 : 16);
    int msum = 0;
    for (int s = 0; s < 8; s++) {
        int sc, mn, w[32];
        scale_min_k4(s, scb, &sc, &mn);
        const uint8_t* qp = q + 32 * (s / 2);
        for (int l = 0; l < 32; l++) {
            int v = (s & 1) ? (qp[l] >> 4) : (qp[l] & 0xF);
            if (nbits == 5) v += ((qh[l] >> s) & 1) << 4;
            w[l] = v;
        }
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, sc);
        msum += mn * (xq_bsum(xb, 2 * s) + xq_bsum(xb, 2 * s + 1));
    }
    const float d = q38o_fp16_to_fp32(ld16(b)), dmin = q38o_fp16_to_fp32(ld16(b + 2)), dx = xq_d(xb);
    block_fma(c, d * dx, sumi);
    c->acc_m = fmaf(dmin * dx, (float)msum, c->acc_m);   /* :427, contracted by the reference build */
}

/* src/cpu/cpu_kernels.cpp:479-515 */
static void blk_q6_K(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    const int8_t* sc = (const int8_t*)(b + 192);
    for (int s = 0; s < 8; s++) {
        const int half = s >> 2, quarter = s & 3;
        const uint8_t* ql = b + 64 * half + 32 * (quarter & 1);
        const uint8_t* qh = b + 128 + 32 * half;
        const int8_t* q = xq_qs(xb) + 32 * s;
        const int g = 8 * half + 2 * quarter;
        for (int l = 0; l < 8; l++) {
            int sum = 0;
            for (int j = 0; j < 4; j++) {
                const int k = 4 * l + j;
                const int v = ((ql[k] >> (4 * (quarter >> 1))) & 0xF) | (((qh[k] >> (2 * quarter)) & 3) << 4);
                sum += v * q[k];
            }
            sumi[l] += sc[g + (l >= 4)] * sum;
        }
    }
    int moff = 0;
    for (int j = 0; j < 16; j++) moff += sc[j] * xq_bsum(xb, j);
    const float d = q38o_fp16_to_fp32(ld16(b + 208)), dx = xq_d(xb);
    block_fma(c, d * dx, sumi);
    c->acc_m = fmaf(d * dx, (float)(32 * moff), c->acc_m);   /* :510 */
}

/* Q8_0 weights x Q8_K activations: no reference kernel exists (only the dequantizer,
 * src/quant/quant_ref.cpp:302-308).  Same pattern: exact int32 lane sums per 32-weight block,
 * one fused multiply-add per lane with d_w * d_x. */
static void blk_q8_0x8(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    for (int s = 0; s < 8; s++, b += BB_Q8_0) {
        int32_t sumi[8] = {0};
        int w[32];
        for (int j = 0; j < 32; j++) w[j] = (int8_t)b[2 + j];
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, 1);
        block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb), sumi);
    }
}

/* the same with one integer scale for the first 16 weights (lanes 0-3) and one for the last 16 (lanes 4-7) */
static inline void sub_dot2(int32_t* sumi, const int* w, const int8_t* q, int sc_lo, int sc_hi) {
    for (int l = 0; l < 8; l++) {
        int s = 0;
        for (int j = 0; j < 4; j++) s += w[4 * l + j] * q[4 * l + j];
        sumi[l] += (l < 4 ? sc_lo : sc_hi) * s;
    }
}

/* src/cpu/cpu_kernels.cpp:191-217 */
static void blk_iq2_xxs(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    for (int s = 0; s < 8; s++) {
        const uint32_t a0 = ld32(b + 2 + 8 * s), a1 = ld32(b + 6 + 8 * s);
        int w[32];
        for (int l = 0; l < 4; l++) {
            const uint32_t code = q38b_iq2xxs_codes[(a0 >> (8 * l)) & 0xFF], sg = ksign8((a1 >> (7 * l)) & 127);
            for (int j = 0; j < 8; j++) w[8 * l + j] = ((sg >> j) & 1) ? -iq2_grid(code, j) : iq2_grid(code, j);
        }
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, (int)(2 * (a1 >> 28) + 1));
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb) * 0.125f, sumi);
}

/* src/cpu/cpu_kernels.cpp:219-249 */
static void blk_iq2_xs(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    for (int s = 0; s < 8; s++) {
        int w[32];
        for (int l = 0; l < 4; l++) {
            const uint32_t qv = ld16(b + 2 + 2 * (4 * s + l));
            const uint32_t code = q38b_iq2xs_codes[qv & 511], sg = ksign8(qv >> 9);
            for (int j = 0; j < 8; j++) w[8 * l + j] = ((sg >> j) & 1) ? -iq2_grid(code, j) : iq2_grid(code, j);
        }
        sub_dot2(sumi, w, xq_qs(xb) + 32 * s, 2 * (b[66 + s] & 0xF) + 1, 2 * (b[66 + s] >> 4) + 1);
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb) * 0.125f, sumi);
}

/* src/cpu/cpu_kernels.cpp:251-281 */
static void blk_iq2_s(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    const uint8_t *qs = b + 2, *signs = b + 34, *qh = b + 66, *scl = b + 74;
    for (int s = 0; s < 8; s++) {
        int w[32];
        for (int l = 0; l < 4; l++) {
            const uint32_t code = q38b_iq2s_codes[qs[4 * s + l] | (((uint32_t)qh[s] << (8 - 2 * l)) & 0x300)];
            const uint32_t sg = signs[4 * s + l];
            for (int j = 0; j < 8; j++) w[8 * l + j] = ((sg >> j) & 1) ? -iq2_grid(code, j) : iq2_grid(code, j);
        }
        sub_dot2(sumi, w, xq_qs(xb) + 32 * s, 2 * (scl[s] & 0xF) + 1, 2 * (scl[s] >> 4) + 1);
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb) * 0.125f, sumi);
}

/* src/cpu/cpu_kernels.cpp:283-313: weights 8 * (grid + delta) = 8 * grid +- 1, block scale / 8 */
static void blk_iq1_s(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    for (int s = 0; s < 8; s++) {
        const uint32_t qh = ld16(b + 34 + 2 * s);
        const int dsgn = (qh & 0x8000) ? -1 : 1;
        int w[32];
        for (int l = 0; l < 4; l++) {
            const uint32_t code = q38b_iq1s_codes[b[2 + 4 * s + l] | (((qh >> (3 * l)) & 7) << 8)];
            for (int j = 0; j < 8; j++) w[8 * l + j] = 8 * iq1_grid(code, j) + dsgn;
        }
        sub_dot(sumi, w, xq_qs(xb) + 32 * s, (int)(2 * ((qh >> 12) & 7) + 1));
    }
    block_fma(c, q38o_fp16_to_fp32(ld16(b)) * xq_d(xb) * 0.125f, sumi);
}

/* src/cpu/cpu_kernels.cpp:315-349 */
static void blk_iq1_m(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    uint16_t sc[4];
    memcpy(sc, b + 48, 8);
    const uint16_t su = (uint16_t)((sc[0] >> 12) | ((sc[1] >> 8) & 0x00f0) | ((sc[2] >> 4) & 0x0f00) | (sc[3] & 0xf000));
    for (int s = 0; s < 8; s++) {
        int w[32];
        for (int l = 0; l < 4; l++) {
            const uint32_t hn = (b[32 + 2 * s + l / 2] >> (4 * (l & 1))) & 0xF;
            const uint32_t code = q38b_iq1s_codes[b[4 * s + l] | ((hn & 7) << 8)];
            for (int j = 0; j < 8; j++) w[8 * l + j] = 8 * iq1_grid(code, j) + ((hn & 8) ? -1 : 1);
        }
        const int t = sc[s / 2] >> (6 * (s % 2));
        sub_dot2(sumi, w, xq_qs(xb) + 32 * s, 2 * (t & 7) + 1, 2 * ((t >> 3) & 7) + 1);
    }
    block_fma(c, q38o_fp16_to_fp32(su) * xq_d(xb) * 0.125f, sumi);
}

/* src/cpu/cpu_kernels.cpp:435-477 */
static void blk_q2_K(const uint8_t* b, const uint8_t* xb, col_acc* c) {
    int32_t sumi[8] = {0};
    for (int sb = 0; sb < 8; sb++) {
        const int n = sb >> 2, j = sb & 3;
        int w[32];
        for (int l = 0; l < 32; l++) w[l] = (b[16 + 32 * n + l] >> (2 * j)) & 3;
        sub_dot2(sumi, w, xq_qs(xb) + 32 * sb, b[2 * sb] & 0xF, b[2 * sb + 1] & 0xF);
    }
    int msum = 0;
    for (int g = 0; g < 16; g++) msum += (b[g] >> 4) * xq_bsum(xb, g);
    const float dw = q38o_fp16_to_fp32(ld16(b + 80)), dmin = q38o_fp16_to_fp32(ld16(b + 82));
    block_fma(c, dw * xq_d(xb), sumi);
    c->acc_m = fmaf(dmin * xq_d(xb), (float)msum, c->acc_m);   /* :474, contracted by the reference build */
}

/* y[c] = W_row . x_c for c < nb; x_c = xq + c * x_stride blocks (src/cpu/cpu_kernels.h:19-22). */
int q38o_vec_dot_n(uint32_t t, int K, const void* w_row, const void* xq, size_t x_stride, int nb, float* y) {
    const size_t bb = q38o_row_bytes(t, QK_K);
    if (!bb || K % QK_K) return -1;
    for (int cidx = 0; cidx < nb; cidx++) {
        col_acc c;
        memset(&c, 0, sizeof(c));
        const uint8_t* b = (const uint8_t*)w_row;
        const uint8_t* xb = (const uint8_t*)xq + (size_t)cidx * x_stride * BB_Q8_K;
        for (int i = 0; i < K / QK_K; i++, b += bb, xb += BB_Q8_K) {
            switch (t) {
                case T_IQ3_XXS: blk_iq3_xxs(b, xb, &c); break;
                case T_IQ3_S: blk_iq3_s(b, xb, &c); break;
                case T_IQ4_XS: blk_iq4_xs(b, xb, &c); break;
                case T_Q4_K: blk_q45_K(b, xb, &c, 4); break;
                case T_Q5_K: blk_q45_K(b, xb, &c, 5); break;
                case T_Q6_K: blk_q6_K(b, xb, &c); break;
                case T_Q8_0: blk_q8_0x8(b, xb, &c); break;
                case T_Q2_K: blk_q2_K(b, xb, &c); break;
                case T_IQ2_XXS: blk_iq2_xxs(b, xb, &c); break;
                case T_IQ2_XS: blk_iq2_xs(b, xb, &c); break;
                case T_IQ2_S: blk_iq2_s(b, xb, &c); break;
                case T_IQ1_S: blk_iq1_s(b, xb, &c); break;
                case T_IQ1_M: blk_iq1_m(b, xb, &c); break;
            }
        }
        y[cidx] = hsum8(c.acc) - c.acc_m;
    }
    return 0;
}

/* Whole matrix: y[c*y_ld + r] = W[r,:] . x_c  (output convention of src/cuda/gemv.cu:49-55).
 * Rows are split over OpenMP threads when the library is built with -fopenmp. */
int q38o_gemv(uint32_t t, const void* W, size_t row_bytes, int K, int M, const void* xq, size_t x_stride, int nb,
              float* y, int y_ld) {
    if (!q38o_row_bytes(t, QK_K) || K % QK_K || nb < 1 || nb > 8) return -1;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < M; r++) {
        float yr[8];
        q38o_vec_dot_n(t, K, (const uint8_t*)W + (size_t)r * row_bytes, xq, x_stride, nb, yr);
        for (int c = 0; c < nb; c++) y[(size_t)c * y_ld + r] = yr[c];
    }
    return 0;
}

/* The reference tests' error metric (tests/kernels/test_cpu_gemv.cpp:100-125): per row the exact
 * double dot of dequantized weights with the dequantized Q8_K activations, and mag = sum |w*x|.
 * ref[r], mag[r] for column 0 only. */
int q38o_row_ref_mag(uint32_t t, const void* W, size_t row_bytes, int K, int M, const void* xq, double* ref,
                     double* mag) {
    if (!q38o_row_bytes(t, QK_K) || K % QK_K) return -1;
#pragma omp parallel
    {
        float* w = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (int r = 0; r < M; r++) {
            q38o_dequantize_row(t, (const uint8_t*)W + (size_t)r * row_bytes, w, K);
            double s = 0, m = 0;
            for (int k = 0; k < K; k++) {
                const uint8_t* xb = (const uint8_t*)xq + (size_t)(k / QK_K) * BB_Q8_K;
                const double xk = (double)xq_d(xb) * (double)xq_qs(xb)[k % QK_K];
                s += (double)w[k] * xk;
                m += fabs((double)w[k] * xk);
            }
            ref[r] = s;
            mag[r] = m;
        }
        free(w);
    }
    return 0;
}

/* h = silu(g) * u : CPU share of the FFN, src/runtime/engine.cpp:177-182 (expf). */
void q38o_swiglu(const float* g, const float* u, int n, float* h) {
    for (int i = 0; i < n; i++) h[i] = g[i] / (1.0f + expf(-g[i])) * u[i];
}

/* FP32 oracle of the prefill GEMM: Y[t][r] = sum_k dequant(W)[r][k] * X[t][k], accumulated in
 * double (src/reference/ref_model.cpp:89-104 sums four float lanes then doubles; double is the
 * tighter statement).  mag[t][r] = sum_k |w*x| for the tolerance.  X is [B][ldx] floats. */
int q38o_matmul_ref(uint32_t t, const void* W, size_t row_bytes, int K, int M, const float* X, int ldx, int B,
                    double* Y, double* mag) {
    if (!q38o_row_bytes(t, QK_K) || K % QK_K) return -1;
#pragma omp parallel
    {
        float* w = (float*)malloc(sizeof(float) * (size_t)K);
#pragma omp for schedule(static)
        for (int r = 0; r < M; r++) {
            q38o_dequantize_row(t, (const uint8_t*)W + (size_t)r * row_bytes, w, K);
            for (int tk = 0; tk < B; tk++) {
                const float* x = X + (size_t)tk * ldx;
                double s = 0, m = 0;
                for (int k = 0; k < K; k++) { const double p = (double)w[k] * (double)x[k]; s += p; m += fabs(p); }
                Y[(size_t)tk * M + r] = s;
                if (mag) mag[(size_t)tk * M + r] = m;
            }
        }
        free(w);
    }
    return 0;
}
