// q38b_decode1.cuh -- single-column (decode, nb = 1) dot products: one lane owns one "granule" of a weight row
// (32 weights; 64 for Q4_K / Q5_K whose sub-block pairs share bytes), keeps the matching int8 activations in
// registers across the rows of a tile, decodes the granule once and multiplies with dp4a.  Per granule the
// result is the exact integer sum of the reference CPU kernels (src/cpu/cpu_kernels.cpp:130-515 of the
// reference project) times the float block scales.
//
// A "slice" is 1024 consecutive weights of a row (four super-blocks): 32 granules, one per lane (Q4_K / Q5_K:
// 16 granules; lanes 16..31 work on the next row).  `row` points at the slice's first byte in shared memory.
// Compiles for the host too (the CPU unit test runs the 32 lanes one after the other).
#pragma once
#include "q38b_decode.cuh"

namespace q38b {

Q38B_HD int dp4a_ss(uint32_t a, uint32_t b, int c) {
#if defined(__CUDA_ARCH__)
    return __dp4a((int)a, (int)b, c);
#else
    for (int i = 0; i < 4; i++) c += (int)(int8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
    return c;
#endif
}
// unsigned weights times signed activations
Q38B_HD int dp4a_us(uint32_t a, uint32_t b, int c) {
#if defined(__CUDA_ARCH__)
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    for (int i = 0; i < 4; i++) c += (int)(uint8_t)(a >> (8 * i)) * (int)(int8_t)(b >> (8 * i));
    return c;
#endif
}

Q38B_HD uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t sh) {   // (hi:lo) >> sh, sh in 0..31
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(lo, hi, sh);
#else
    return sh ? (lo >> sh) | (hi << (32 - sh)) : lo;
#endif
}

// 8 bytes from a 2-byte aligned address: three aligned words and two funnel shifts
Q38B_HD void ld_8_a2(const uint8_t* p, uint32_t& lo, uint32_t& hi) {
    const uint32_t mis = (uint32_t)((uintptr_t)p & 2);
    const uint32_t* w = (const uint32_t*)(p - mis);   // pointer minus integer: the address space stays known
    const uint32_t sh = mis * 8;
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2];
    lo = funnel_r(w0, w1, sh);
    hi = funnel_r(w1, w2, sh);
}

// what a lane needs from the activations for one slice
template <int NWORDS> struct ActRegs {
    uint32_t q[NWORDS];   // int8 activations of the granule, in the format's staged order
    float dx;             // Q8_K block scale of the granule's super-block
};

template <int FMT> struct Gran;

// ---------------------------------------------------------------------------------------------------------------
// IQ3_XXS (layout and formula: see Unit<T_IQ3_XXS>).  sum = (2s+1) * (P - 2N): P = dot of the unsigned grid bytes,
// N = dot of the grid bytes whose sign bit is set.
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_IQ3_XXS> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    static Q38B_HD void load_acts(Acts& a, const uint8_t* aq, const float* ad, int lane) {
#pragma unroll
        for (int i = 0; i < 8; i++) a.q[i] = ld_u32(aq + 32 * lane + 4 * i);
        a.dx = ad[(lane >> 3) * 8] * 0.25f;
    }
    static Q38B_HD float dot(const uint8_t* row, const Acts& a, const Codebook& cb, int lane) {
        const uint8_t* p = row + 98 * (lane >> 3);
        const int s = lane & 7;
        uint32_t iw[2];
        ld_8_a2(p + 2 + 8 * s, iw[0], iw[1]);
        const uint32_t aux = ld_u16(p + 66 + 4 * s) | (ld_u16(p + 68 + 4 * s) << 16);
        int P = 0, N = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t s7 = (aux >> (7 * l)) & 127u;
            const uint32_t m_lo = sign_mask4(s7);
            const uint32_t m_hi = prmt((uint32_t)popc(s7) * 0x80000000u + s7 * 0x00020408u, 0u, 0xBA98u);
            const uint32_t w = iw[l >> 1] >> (16 * (l & 1));
            const uint32_t g0 = cb_lookup(cb, w & 0xFFu), g1 = cb_lookup(cb, (w >> 8) & 0xFFu);
            P = dp4a_us(g0, a.q[2 * l], P);
            P = dp4a_us(g1, a.q[2 * l + 1], P);
            N = dp4a_us(g0 & m_lo, a.q[2 * l], N);
            N = dp4a_us(g1 & m_hi, a.q[2 * l + 1], N);
        }
        const int sumi = (int)(2u * (aux >> 28) + 1u) * (P - 2 * N);
        return fp16_bits_to_float(ld_u16(p)) * a.dx * (float)sumi;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// IQ3_S
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_IQ3_S> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    static Q38B_HD void load_acts(Acts& a, const uint8_t* aq, const float* ad, int lane) {
#pragma unroll
        for (int i = 0; i < 8; i++) a.q[i] = ld_u32(aq + 32 * lane + 4 * i);
        a.dx = ad[(lane >> 3) * 8];
    }
    static Q38B_HD float dot(const uint8_t* row, const Acts& a, const Codebook& cb, int lane) {
        const uint8_t* p = row + 110 * (lane >> 3);
        const int s = lane & 7;
        uint32_t iw[2];
        ld_8_a2(p + 2 + 8 * s, iw[0], iw[1]);
        const uint32_t qh = ld_u8(p + 66 + s);
        const uint32_t sg = ld_u16(p + 74 + 4 * s) | (ld_u16(p + 76 + 4 * s) << 16);
        const uint32_t ls = (ld_u8(p + 106 + (s >> 1)) >> (4 * (s & 1))) & 0xFu;
        int P = 0, N = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t sb = (sg >> (8 * l)) & 0xFFu;
            const uint32_t m_lo = sign_mask4(sb & 0xFu), m_hi = sign_mask4(sb >> 4);
            const uint32_t w = iw[l >> 1] >> (16 * (l & 1));
            const uint32_t g0 = cb_lookup(cb, (w & 0xFFu) | (((qh >> (2 * l)) & 1u) << 8));
            const uint32_t g1 = cb_lookup(cb, ((w >> 8) & 0xFFu) | (((qh >> (2 * l + 1)) & 1u) << 8));
            P = dp4a_us(g0, a.q[2 * l], P);
            P = dp4a_us(g1, a.q[2 * l + 1], P);
            N = dp4a_us(g0 & m_lo, a.q[2 * l], N);
            N = dp4a_us(g1 & m_hi, a.q[2 * l + 1], N);
        }
        const int sumi = (int)(2u * ls + 1u) * (P - 2 * N);
        return fp16_bits_to_float(ld_u16(p)) * a.dx * (float)sumi;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// IQ4_XS: activations staged in the order the PRMT table lookup emits the weights (act_stage_pos)
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_IQ4_XS> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    static Q38B_HD void load_acts(Acts& a, const uint8_t* aq, const float* ad, int lane) {
#pragma unroll
        for (int i = 0; i < 8; i++) a.q[i] = ld_u32(aq + 32 * lane + 4 * i);
        a.dx = ad[(lane >> 3) * 8];
    }
    static Q38B_HD float dot(const uint8_t* row, const Acts& a, const Codebook&, int lane) {
        const uint8_t* p = row + 136 * (lane >> 3);
        const int s = lane & 7;
        uint32_t w[4];
        ld_u64(p + 8 + 16 * s, w[0], w[1]);
        ld_u64(p + 16 + 16 * s, w[2], w[3]);
        int dot = 0;
#pragma unroll
        for (int t = 0; t < 4; t++) {
            uint32_t x0, x1;
            Unit<T_IQ4_XS>::lut8(w[t], x0, x1);
            dot = dp4a_ss(x0, a.q[2 * t], dot);
            dot = dp4a_ss(x1, a.q[2 * t + 1], dot);
        }
        const uint32_t hdr = ld_u32(p);            // fp16 d | scales_h
        const uint32_t sl = ld_u8(p + 4 + (s >> 1));
        const int ls = (int)(((sl >> (4 * (s & 1))) & 0xFu) | ((((hdr >> 16) >> (2 * s)) & 3u) << 4)) - 32;
        return fp16_bits_to_float(hdr & 0xFFFFu) * a.dx * (float)(ls * dot);
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Q4_K / Q5_K: granule = pair of sub-blocks (32 bytes of nibbles).  Lanes 0..15 take the 16 pairs of one row's
// slice, lanes 16..31 those of the next row.  bs0 / bs1 are the sums of the activations of the two sub-blocks (the
// bsums of the Q8_K block), taken from the int8 values themselves.
// ---------------------------------------------------------------------------------------------------------------
template <int NBITS> struct GranQ45K {
    static constexpr int WORDS = 16, LANES_PER_ROW = 16;
    static constexpr int BB = NBITS == 5 ? 176 : 144, QS = NBITS == 5 ? 48 : 16;
    struct Acts { uint32_t q[16]; float dx; int bs0, bs1; };
    static Q38B_HD void load_acts(Acts& a, const uint8_t* aq, const float* ad, int lane) {
        const int pr = lane & 15;
#pragma unroll
        for (int i = 0; i < 16; i++) a.q[i] = ld_u32(aq + 64 * pr + 4 * i);
        a.dx = ad[(pr >> 2) * 8];
        a.bs0 = 0; a.bs1 = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) { a.bs0 = dp4a_ss(0x01010101u, a.q[i], a.bs0); a.bs1 = dp4a_ss(0x01010101u, a.q[8 + i], a.bs1); }
    }
    static Q38B_HD float dot(const uint8_t* row, const Acts& a, const Codebook&, int lane) {
        const int pr = lane & 15, pp = pr & 3;
        const uint8_t* p = row + BB * (pr >> 2);
        uint32_t w[8];
#if defined(__CUDA_ARCH__)
        {
            const uint4 v0 = *(const uint4*)(p + QS + 32 * pp), v1 = *(const uint4*)(p + QS + 32 * pp + 16);
            w[0] = v0.x; w[1] = v0.y; w[2] = v0.z; w[3] = v0.w; w[4] = v1.x; w[5] = v1.y; w[6] = v1.z; w[7] = v1.w;
        }
#else
        memcpy(w, p + QS + 32 * pp, 32);
#endif
        const uint32_t dd = ld_u32(p), u0 = ld_u32(p + 4), u1 = ld_u32(p + 8), u2 = ld_u32(p + 12);
        // 6-bit scales / mins of sub-blocks 2pp, 2pp+1 (get_scale_min_k4, src/quant/quant_ref.cpp:24-32)
        const bool hi_half = pp >= 2;
        const uint32_t sc4 = hi_half ? ((u2 & 0x0F0F0F0Fu) | ((u0 >> 2) & 0x30303030u)) : (u0 & 0x3F3F3F3Fu);
        const uint32_t mn4 = hi_half ? (((u2 >> 4) & 0x0F0F0F0Fu) | ((u1 >> 2) & 0x30303030u)) : (u1 & 0x3F3F3F3Fu);
        const uint32_t sh = 16u * (uint32_t)(pp & 1);
        const int sc0 = (int)((sc4 >> sh) & 0xFFu), sc1 = (int)((sc4 >> (sh + 8)) & 0xFFu);
        const int mn0 = (int)((mn4 >> sh) & 0xFFu), mn1 = (int)((mn4 >> (sh + 8)) & 0xFFu);
        int lo = 0, hi = 0;
        if (NBITS == 4) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                lo = dp4a_ss(w[i] & 0x0F0F0F0Fu, a.q[i], lo);
                hi = dp4a_us(w[i] & 0xF0F0F0F0u, a.q[8 + i], hi);   // 16 * nibble, exact; divided below
            }
            hi >>= 4;
        } else {
            uint32_t h[8];
#if defined(__CUDA_ARCH__)
            {
                const uint4 v0 = *(const uint4*)(p + 16), v1 = *(const uint4*)(p + 32);
                h[0] = v0.x; h[1] = v0.y; h[2] = v0.z; h[3] = v0.w; h[4] = v1.x; h[5] = v1.y; h[6] = v1.z; h[7] = v1.w;
            }
#else
            memcpy(h, p + 16, 32);
#endif
            const uint32_t b0 = 2u * (uint32_t)pp;   // bit of qh for the low-nibble sub-block; b0 + 1 for the other
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t hb = h[i] >> b0;
                lo = dp4a_ss((w[i] & 0x0F0F0F0Fu) | ((hb << 4) & 0x10101010u), a.q[i], lo);
                hi = dp4a_ss(((w[i] >> 4) & 0x0F0F0F0Fu) | ((hb << 3) & 0x10101010u), a.q[8 + i], hi);
            }
        }
        const int sumi = sc0 * lo + sc1 * hi;
        const int msum = mn0 * a.bs0 + mn1 * a.bs1;
        const float d = fp16_bits_to_float(dd & 0xFFFFu), dmin = fp16_bits_to_float(dd >> 16);
        return d * a.dx * (float)sumi - dmin * a.dx * (float)msum;
    }
};
template <> struct Gran<T_Q4_K> : GranQ45K<4> {};
template <> struct Gran<T_Q5_K> : GranQ45K<5> {};

// ---------------------------------------------------------------------------------------------------------------
// Q6_K: granule = weights {128n + 32j + 8i .. +7 : j = 0..3} of a super-block (n = half, i = 0..3): 8 bytes of ql at
// two places and 8 bytes of qh.  Lane: super-block lane/8, n = (lane/4) & 1, i = lane & 3.
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_Q6_K> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    static Q38B_HD void load_acts(Acts& a, const uint8_t* aq, const float* ad, int lane) {
        const int sb = lane >> 3, n = (lane >> 2) & 1, i = lane & 3;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            a.q[2 * j] = ld_u32(aq + 256 * sb + 128 * n + 32 * j + 8 * i);
            a.q[2 * j + 1] = ld_u32(aq + 256 * sb + 128 * n + 32 * j + 8 * i + 4);
        }
        a.dx = ad[sb * 8];
    }
    static Q38B_HD float dot(const uint8_t* row, const Acts& a, const Codebook&, int lane) {
        const int n = (lane >> 2) & 1, i = lane & 3;
        const uint8_t* p = row + 210 * (lane >> 3);
        uint32_t qa[2], qb[2], qh[2];
        ld_8_a2(p + 64 * n + 8 * i, qa[0], qa[1]);
        ld_8_a2(p + 64 * n + 32 + 8 * i, qb[0], qb[1]);
        ld_8_a2(p + 128 + 32 * n + 8 * i, qh[0], qh[1]);
        int d4[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 2; k++) {
            d4[0] = dp4a_ss(Unit<T_Q6_K>::q6(qa[k], qh[k] << 4), a.q[k], d4[0]);
            d4[1] = dp4a_ss(Unit<T_Q6_K>::q6(qb[k], qh[k] << 2), a.q[2 + k], d4[1]);
            d4[2] = dp4a_ss(Unit<T_Q6_K>::q6(qa[k] >> 4, qh[k]), a.q[4 + k], d4[2]);
            d4[3] = dp4a_ss(Unit<T_Q6_K>::q6(qb[k] >> 4, qh[k] >> 2), a.q[6 + k], d4[3]);
        }
        // scale of group 8n + 2j + (i >> 1)
        const uint8_t* sc = p + 192 + 8 * n + (i >> 1);
        int sumi = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) sumi += (int)(int8_t)ld_u8(sc + 2 * j) * d4[j];
        return fp16_bits_to_float(ld_u16(p + 208)) * a.dx * (float)sumi;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Q8_0: granule = one 34-byte block
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_Q8_0> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    static Q38B_HD void load_acts(Acts& a, const uint8_t* aq, const float* ad, int lane) {
#pragma unroll
        for (int i = 0; i < 8; i++) a.q[i] = ld_u32(aq + 32 * lane + 4 * i);
        a.dx = ad[(lane >> 3) * 8];
    }
    static Q38B_HD float dot(const uint8_t* row, const Acts& a, const Codebook&, int lane) {
        const uint8_t* p = row + 34 * lane;
        int dot = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t lo, hi;
            ld_8_a2(p + 2 + 8 * i, lo, hi);
            dot = dp4a_ss(lo, a.q[2 * i], dot);
            dot = dp4a_ss(hi, a.q[2 * i + 1], dot);
        }
        return fp16_bits_to_float(ld_u16(p)) * a.dx * (float)dot;
    }
};

}  // namespace q38b
