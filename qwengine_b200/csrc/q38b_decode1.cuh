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
#if !defined(__CUDA_ARCH__)
#include <cstdio>
#include <cstdlib>
#endif

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

// ---------------------------------------------------------------------------------------------------------------
// Staged bytes are addressed through SP: on the device a 32-bit shared-space address (loads are ld.shared with
// immediate offsets, no 64-bit pointer arithmetic and no generic-to-shared conversion per load), on the host a pointer.
// ---------------------------------------------------------------------------------------------------------------
#if defined(__CUDA_ARCH__)
struct SP { uint32_t a; };
__device__ __forceinline__ SP sp_from(const void* p) { return SP{(uint32_t)__cvta_generic_to_shared(p)}; }
__device__ __forceinline__ uint32_t sp_low2(SP p) { return p.a & 2u; }
__device__ __forceinline__ uint32_t sp_ld8(SP p, int o = 0) { uint32_t v; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(p.a + o)); return v; }
__device__ __forceinline__ int sp_ld8s(SP p, int o = 0) { int v; asm volatile("ld.shared.s8 %0, [%1];" : "=r"(v) : "r"(p.a + o)); return v; }
__device__ __forceinline__ uint32_t sp_ld16(SP p, int o = 0) { uint32_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(p.a + o)); return v; }
__device__ __forceinline__ uint32_t sp_ld32(SP p, int o = 0) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(p.a + o)); return v; }
__device__ __forceinline__ float sp_ldf(SP p, int o = 0) { float v; asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(p.a + o)); return v; }
__device__ __forceinline__ void sp_ld64(SP p, int o, uint32_t& x, uint32_t& y) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(x), "=r"(y) : "r"(p.a + o));
}
__device__ __forceinline__ void sp_ld128(SP p, int o, uint32_t (&v)[4]) {
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(p.a + o));
}
#else
struct SP { const uint8_t* a; };
inline SP sp_from(const void* p) { return SP{(const uint8_t*)p}; }
inline uint32_t sp_low2(SP p) { return (uint32_t)((uintptr_t)p.a & 2); }
inline uint32_t sp_ld8(SP p, int o = 0) { return p.a[o]; }
inline int sp_ld8s(SP p, int o = 0) { return (int8_t)p.a[o]; }
// the host versions refuse what the device would fault on: an address that is not a multiple of the access size
inline void sp_check_aligned(const uint8_t* p, int n) { if ((uintptr_t)p % (uintptr_t)n) { fprintf(stderr, "misaligned %d-byte shared load\n", n); abort(); } }
inline uint32_t sp_ld16(SP p, int o = 0) { uint16_t v; sp_check_aligned(p.a + o, 2); memcpy(&v, p.a + o, 2); return v; }
inline uint32_t sp_ld32(SP p, int o = 0) { uint32_t v; sp_check_aligned(p.a + o, 4); memcpy(&v, p.a + o, 4); return v; }
inline float sp_ldf(SP p, int o = 0) { float v; sp_check_aligned(p.a + o, 4); memcpy(&v, p.a + o, 4); return v; }
inline void sp_ld64(SP p, int o, uint32_t& x, uint32_t& y) { sp_check_aligned(p.a + o, 8); memcpy(&x, p.a + o, 4); memcpy(&y, p.a + o + 4, 4); }
inline void sp_ld128(SP p, int o, uint32_t (&v)[4]) { sp_check_aligned(p.a + o, 16); memcpy(v, p.a + o, 16); }
#endif
Q38B_HD SP operator+(SP p, int o) { return SP{p.a + o}; }
Q38B_HD SP operator-(SP p, int o) { return SP{p.a - o}; }

// 8 bytes from a 2-byte aligned address: three aligned words and two funnel shifts.  `mis` = address & 2.
Q38B_HD void sp_ld8b_a2(SP p, uint32_t mis, uint32_t& lo, uint32_t& hi) {
    const SP w = p - (int)mis;
    const uint32_t sh = mis * 8;
    const uint32_t w0 = sp_ld32(w, 0), w1 = sp_ld32(w, 4), w2 = sp_ld32(w, 8);
    lo = funnel_r(w0, w1, sh);
    hi = funnel_r(w1, w2, sh);
}

// Codebook replicated 32 x in shared memory: entry e for lane l is the word at base + e * 128 + l * 4.
// IQ3_XXS also keeps its 128 sign codes there as pairs of byte masks (0xFF where the weight is negative), replicated
// 16 x: code c for lane l is the 8 bytes at sign_base + c * 128 + (l & 15) * 8 (a 64-bit load is served per half warp).
struct Codebook1 { SP lane_base; SP sign_base; };
Q38B_HD uint32_t cb1(const Codebook1& cb, uint32_t e_times_128) { return sp_ld32(cb.lane_base + (int)e_times_128); }
constexpr int KSIGN_TABLE_BYTES = 128 * 128;
// masks of sign code c (7 bits + the parity bit that makes the number of negative weights even, ksigns_iq2xs of ggml)
Q38B_HD void ksign_entry(uint32_t c, uint32_t& lo, uint32_t& hi) {
    uint32_t sg = c, par = c;
    par ^= par >> 4; par ^= par >> 2; par ^= par >> 1;
    sg |= (par & 1u) << 7;
    lo = 0; hi = 0;
    for (int j = 0; j < 4; j++) {
        if ((sg >> j) & 1u) lo |= 0xFFu << (8 * j);
        if ((sg >> (4 + j)) & 1u) hi |= 0xFFu << (8 * j);
    }
}

// byte k of w, times 128 (the stride of a replicated codebook entry)
Q38B_HD uint32_t byte_x128(uint32_t w, int k) { return (k == 0 ? (w << 7) : (w >> (8 * k - 7))) & 0x7F80u; }

// byte k of w, times 64 (the stride of an entry of a codebook replicated 16 x)
Q38B_HD uint32_t byte_x64(uint32_t w, int k) { return (k == 0 ? (w << 6) : (w >> (8 * k - 6))) & 0x3FC0u; }
// replicas of the single-column kernels' shared-memory codebooks: IQ3_XXS (256 entries) 32, every lane its own bank;
// IQ3_S (512 entries) 16, lanes l and l + 16 share a replica (32 KB instead of 64)
Q38B_HD constexpr int cb1_rep_log2(int fmt) { return fmt == T_IQ3_S ? 4 : fmt == T_IQ3_XXS ? 5 : 0; }

// Staged int8 activations of a 1024-weight slice: the chunks that the lanes of a warp fetch with ONE load instruction
// are consecutive (16 bytes per lane, 8 for Q6_K), so that the load is served in the fewest wavefronts; in the natural
// order a lane's 32 (or 64) bytes are consecutive and eight lanes meet on the same banks.  k: byte of the slice in the
// format's own order (after act_stage_pos); result: its place in the staged slice.
Q38B_HD constexpr int act_slice_pos(int fmt, int k) {
    if (fmt == T_Q4_K || fmt == T_Q5_K) return ((k >> 4) & 3) * 256 + (k >> 6) * 16 + (k & 15);   // lane pair pr = k / 64, chunk i
    if (fmt == T_Q6_K) return ((k >> 5) & 3) * 256 + ((k >> 8) * 8 + ((k >> 7) & 1) * 4 + ((k >> 3) & 3)) * 8 + (k & 7);   // (sb, n, i) = lane, j
    return ((k >> 4) & 1) * 512 + (k >> 5) * 16 + (k & 15);   // lane = k / 32, half
}

// what a lane needs from the activations for one slice
template <int NWORDS> struct ActRegs {
    uint32_t q[NWORDS];   // int8 activations of the granule, in the format's staged order
    float dx;             // Q8_K block scale of the granule's super-block (per-32 activations: the scale of the granule's 32)
};
// Activation scales come in two layouts of the same array (32 floats per slice = 8 per super-block): Q8_K activations
// keep one scale per super-block in slot 8 * sb; per-32 activations (the reference GPU path's ActQ8,
// src/cuda/gemv.cuh:14-21) one scale per 32 weights in slot 8 * sb + j.  A32 selects the second.

template <int FMT> struct Gran;

// ---------------------------------------------------------------------------------------------------------------
// IQ3_XXS (layout and formula: see Unit<T_IQ3_XXS>).  sum = (2s+1) * (P - 2N): P = dot of the unsigned grid bytes,
// N = dot of the grid bytes whose sign bit is set.
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_IQ3_XXS> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        uint32_t v[4];
        sp_ld128(aq, 16 * lane, v);
        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(aq, 512 + 16 * lane, v);
        a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        a.dx = sp_ldf(ad, A32 ? 4 * lane : (lane >> 3) * 32) * 0.25f;
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) { return dot(row, a, cb, lane); }
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 98 * (lane >> 3);
        const int s = lane & 7;
        const SP ip = p + (2 + 8 * s);
        const uint32_t aux = sp_ld16(p, 66 + 4 * s) | (sp_ld16(p, 68 + 4 * s) << 16);
        int P = 0, N = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            // the index bytes come as single-byte loads (no alignment fix-up, no extraction); 128 * index + base is one
            // multiply-add; the sign masks come from the table
            const uint32_t c128 = (l == 0 ? (aux << 7) : (aux >> (7 * l - 7))) & 0x3F80u;
            uint32_t m_lo, m_hi;
            sp_ld64(cb.sign_base + (int)c128, 0, m_lo, m_hi);
            const uint32_t g0 = cb1(cb, sp_ld8(ip, 2 * l) * 128u), g1 = cb1(cb, sp_ld8(ip, 2 * l + 1) * 128u);
            P = dp4a_us(g0, a.q[2 * l], P);
            P = dp4a_us(g1, a.q[2 * l + 1], P);
            N = dp4a_us(g0 & m_lo, a.q[2 * l], N);
            N = dp4a_us(g1 & m_hi, a.q[2 * l + 1], N);
        }
        const int sumi = (int)(2u * (aux >> 28) + 1u) * (P - 2 * N);
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * (float)sumi;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// IQ3_S: 512-entry codebook, 9th index bits in qh, explicit sign bytes
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_IQ3_S> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        uint32_t v[4];
        sp_ld128(aq, 16 * lane, v);
        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(aq, 512 + 16 * lane, v);
        a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        a.dx = sp_ldf(ad, A32 ? 4 * lane : (lane >> 3) * 32);
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) { return dot(row, a, cb, lane); }
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 110 * (lane >> 3);
        const int s = lane & 7;
        uint32_t iw[2];
        sp_ld8b_a2(p + (2 + 8 * s), sp_low2(p) ^ 2u, iw[0], iw[1]);
        const uint32_t qh = sp_ld8(p, 66 + s) << 14;               // bit j of qh now sits at bit 14 + j: entry 256 * 64
        const uint32_t sg = sp_ld16(p, 74 + 4 * s) | (sp_ld16(p, 76 + 4 * s) << 16);
        const uint32_t ls = (sp_ld8(p, 106 + (s >> 1)) >> (4 * (s & 1))) & 0xFu;
        int P = 0, N = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t sb = sg >> (8 * l);
            const uint32_t m_lo = sign_mask4(sb & 0xFu), m_hi = sign_mask4((sb >> 4) & 0xFu);
            const uint32_t w = iw[l >> 1];
            const uint32_t g0 = cb1(cb, byte_x64(w, 2 * (l & 1)) | ((qh >> (2 * l)) & 0x4000u));
            const uint32_t g1 = cb1(cb, byte_x64(w, 2 * (l & 1) + 1) | ((qh >> (2 * l + 1)) & 0x4000u));
            P = dp4a_us(g0, a.q[2 * l], P);
            P = dp4a_us(g1, a.q[2 * l + 1], P);
            N = dp4a_us(g0 & m_lo, a.q[2 * l], N);
            N = dp4a_us(g1 & m_hi, a.q[2 * l + 1], N);
        }
        const int sumi = (int)(2u * ls + 1u) * (P - 2 * N);
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * (float)sumi;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// IQ4_XS: activations staged in the order the PRMT table lookup emits the weights (act_stage_pos)
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_IQ4_XS> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        uint32_t v[4];
        sp_ld128(aq, 16 * lane, v);
        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(aq, 512 + 16 * lane, v);
        a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        a.dx = sp_ldf(ad, A32 ? 4 * lane : (lane >> 3) * 32);
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) { return dot(row, a, cb, lane); }
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1&, int lane) {
        const SP p = row + 136 * (lane >> 3);
        const int s = lane & 7;
        uint32_t w[4];
        sp_ld64(p, 8 + 16 * s, w[0], w[1]);
        sp_ld64(p, 16 + 16 * s, w[2], w[3]);
        // The 16 levels split into the eight negative ones (nibbles 0..7) and the eight positive ones (8..15).  PRMT with a
        // nibble of the data word as its selector picks one of eight table bytes by the nibble's low three bits, and
        // returns the SIGN of that byte in all eight bits when the nibble's top bit is set.  With two tables of
        // non-negative bytes -- the negated negative levels, looked up with the word itself, and the positive levels in
        // reverse order, looked up with the complemented word (nibble 8 + m becomes 7 - m, nibbles below 8 get their top
        // bit set) -- each look-up yields the level's magnitude where the nibble belongs to its half and zero elsewhere:
        // sum = dp4a(positive part) - dp4a(negated negative part), no masks and no third PRMT to merge the halves.
        constexpr uint32_t NL0 = Unit<T_IQ4_XS>::NL0, NL1 = Unit<T_IQ4_XS>::NL1;   // 127, 104, 83, 65 | 49, 35, 22, 10
        constexpr uint32_t HR0 = Unit<T_IQ4_XS>::HR0, HR1 = Unit<T_IQ4_XS>::HR1;   // 113, 89, 69, 53 | 38, 25, 13, 1
        int pos = 0, neg = 0;
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const uint32_t nw = ~w[t];
            neg = dp4a_ss(prmt(NL0, NL1, w[t]), a.q[2 * t], neg);
            pos = dp4a_ss(prmt(HR0, HR1, nw), a.q[2 * t], pos);
            neg = dp4a_ss(prmt(NL0, NL1, w[t] >> 16), a.q[2 * t + 1], neg);
            pos = dp4a_ss(prmt(HR0, HR1, nw >> 16), a.q[2 * t + 1], pos);
        }
        const int dot = pos - neg;
        const uint32_t hdr = sp_ld32(p, 0);            // fp16 d | scales_h
        const uint32_t sl = sp_ld8(p, 4 + (s >> 1));
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
    struct Acts { uint32_t q[16]; float dx, dx1; int bs0, bs1; };   // dx1: scale of the second sub-block (per-32 activations)
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        const int pr = lane & 15;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t v[4];
            sp_ld128(aq, 256 * i + 16 * pr, v);
            a.q[4 * i] = v[0]; a.q[4 * i + 1] = v[1]; a.q[4 * i + 2] = v[2]; a.q[4 * i + 3] = v[3];
        }
        a.dx = sp_ldf(ad, A32 ? 8 * pr : (pr >> 2) * 32);
        a.dx1 = A32 ? sp_ldf(ad, 8 * pr + 4) : a.dx;
        a.bs0 = 0; a.bs1 = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) { a.bs0 = dp4a_ss(0x01010101u, a.q[i], a.bs0); a.bs1 = dp4a_ss(0x01010101u, a.q[8 + i], a.bs1); }
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1&, int lane) {
        const int pr = lane & 15, pp = pr & 3;
        const SP p = row + BB * (pr >> 2);
        uint32_t w[8], hd[4];
        {
            uint32_t v[4];
            sp_ld128(p, QS + 32 * pp, v);
            w[0] = v[0]; w[1] = v[1]; w[2] = v[2]; w[3] = v[3];
            sp_ld128(p, QS + 32 * pp + 16, v);
            w[4] = v[0]; w[5] = v[1]; w[6] = v[2]; w[7] = v[3];
        }
        sp_ld128(p, 0, hd);                        // d | dmin, scales[12]
        const uint32_t dd = hd[0], u0 = hd[1], u1 = hd[2], u2 = hd[3];
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
            {
                uint32_t v[4];
                sp_ld128(p, 16, v);
                h[0] = v[0]; h[1] = v[1]; h[2] = v[2]; h[3] = v[3];
                sp_ld128(p, 32, v);
                h[4] = v[0]; h[5] = v[1]; h[6] = v[2]; h[7] = v[3];
            }
            const uint32_t b0 = 2u * (uint32_t)pp;   // bit of qh for the low-nibble sub-block; b0 + 1 for the other
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t hb = h[i] >> b0;
                lo = dp4a_ss((w[i] & 0x0F0F0F0Fu) | ((hb << 4) & 0x10101010u), a.q[i], lo);
                hi = dp4a_ss(((w[i] >> 4) & 0x0F0F0F0Fu) | ((hb << 3) & 0x10101010u), a.q[8 + i], hi);
            }
        }
        const float d = fp16_bits_to_float(dd & 0xFFFFu), dmin = fp16_bits_to_float(dd >> 16);
        if (A32)   // each sub-block of the pair has its own activation scale
            return d * (a.dx * (float)(sc0 * lo) + a.dx1 * (float)(sc1 * hi)) - dmin * (a.dx * (float)(mn0 * a.bs0) + a.dx1 * (float)(mn1 * a.bs1));
        const int sumi = sc0 * lo + sc1 * hi;
        const int msum = mn0 * a.bs0 + mn1 * a.bs1;
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
    struct Acts { uint32_t q[8]; float dx; float dxs[4]; };   // dxs: scales of the granule's four 32-weight groups (per-32 activations)
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        const int sb = lane >> 3, n = (lane >> 2) & 1, i = lane & 3;
#pragma unroll
        for (int j = 0; j < 4; j++) sp_ld64(aq, 256 * j + 8 * lane, a.q[2 * j], a.q[2 * j + 1]);
        a.dx = sp_ldf(ad, sb * 32);
#pragma unroll
        for (int j = 0; j < 4; j++) a.dxs[j] = A32 ? sp_ldf(ad, sb * 32 + 16 * n + 4 * j) : a.dx;
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1&, int lane) {
        const int n = (lane >> 2) & 1, i = lane & 3;
        const SP p = row + 210 * (lane >> 3);
        const uint32_t mis = sp_low2(p);
        uint32_t qa[2], qb[2], qh[2];
        sp_ld8b_a2(p + (64 * n + 8 * i), mis, qa[0], qa[1]);
        sp_ld8b_a2(p + (64 * n + 32 + 8 * i), mis, qb[0], qb[1]);
        sp_ld8b_a2(p + (128 + 32 * n + 8 * i), mis, qh[0], qh[1]);
        int d4[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 2; k++) {
            d4[0] = dp4a_ss(Unit<T_Q6_K>::q6(qa[k], qh[k] << 4), a.q[k], d4[0]);
            d4[1] = dp4a_ss(Unit<T_Q6_K>::q6(qb[k], qh[k] << 2), a.q[2 + k], d4[1]);
            d4[2] = dp4a_ss(Unit<T_Q6_K>::q6(qa[k] >> 4, qh[k]), a.q[4 + k], d4[2]);
            d4[3] = dp4a_ss(Unit<T_Q6_K>::q6(qb[k] >> 4, qh[k] >> 2), a.q[6 + k], d4[3]);
        }
        const SP sc = p + (192 + 8 * n + (i >> 1));          // scale of group 8n + 2j + (i >> 1)
        if (A32) {   // group j of the granule lies in 32-weight block 4n + j of the super-block
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; j++) acc += a.dxs[j] * (float)(sp_ld8s(sc, 2 * j) * d4[j]);
            return fp16_bits_to_float(sp_ld16(p, 208)) * acc;
        }
        int sumi = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) sumi += sp_ld8s(sc, 2 * j) * d4[j];
        return fp16_bits_to_float(sp_ld16(p, 208)) * a.dx * (float)sumi;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Q8_0: granule = one 34-byte block
// ---------------------------------------------------------------------------------------------------------------
template <> struct Gran<T_Q8_0> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        uint32_t v[4];
        sp_ld128(aq, 16 * lane, v);
        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(aq, 512 + 16 * lane, v);
        a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        a.dx = sp_ldf(ad, A32 ? 4 * lane : (lane >> 3) * 32);
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) { return dot(row, a, cb, lane); }
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1&, int lane) {
        const SP p = row + 34 * lane;
        const uint32_t mis = sp_low2(p) ^ 2u;                // the int8 values start 2 bytes into the block
        int dot = 0;
        // 32 bytes from a 2-byte aligned address: nine aligned words, eight funnel shifts
        const SP wbase = p + 2 - (int)mis;
        const uint32_t sh = mis * 8;
        uint32_t prev = sp_ld32(wbase, 0);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t next = sp_ld32(wbase, 4 * i + 4);
            dot = dp4a_ss(funnel_r(prev, next, sh), a.q[i], dot);
            prev = next;
        }
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * (float)dot;
    }
};

// ---------------------------------------------------------------------------------------------------------------
// IQ2_XXS, IQ2_XS, IQ2_S, IQ1_S, IQ1_M, Q2_K (integer sums of src/cpu/cpu_kernels.cpp:191-349, 435-477).  The grids of
// the i-quants hold eight values out of three levels per entry; shared memory keeps them as 16-bit codes (eight 2-bit
// level indices, one copy: cb.lane_base points at it) and PRMT expands four indices into four bytes from a register.
// ---------------------------------------------------------------------------------------------------------------
// 8 bits = four 2-bit indices -> PRMT selector with index i in nibble i
Q38B_HD uint32_t sel_from_codes(uint32_t x) {
    const uint32_t t = (x | (x << 4)) & 0x0F0Fu;
    return (t | (t << 2)) & 0x3333u;
}
Q38B_HD uint32_t iq2_bytes(uint32_t code8) { return prmt(0x002B1908u, 0u, sel_from_codes(code8)); }      // levels 8, 25, 43
// 8 * {-1, 0, 1} + 1 = -7, 1, 9 and 8 * {-1, 0, 1} - 1 = -9, -1, 7 as int8
Q38B_HD uint32_t iq1_bytes(uint32_t code8, bool minus) { return prmt(minus ? 0x0007FFF7u : 0x000901F9u, 0u, sel_from_codes(code8)); }
Q38B_HD uint32_t ksign_byte(uint32_t s7) { return s7 | ((uint32_t)(popc(s7) & 1) << 7); }
Q38B_HD uint32_t code16(const Codebook1& cb, uint32_t idx) { return sp_ld16(cb.lane_base + (int)(2u * idx)); }

// 8 signed weights of one grid entry against two activation words: P += |g| . q, N += (negative |g|) . q
Q38B_HD void iq2_group(uint32_t code, uint32_t sign8, uint32_t q0, uint32_t q1, int& P, int& N) {
    const uint32_t g0 = iq2_bytes(code & 0xFFu), g1 = iq2_bytes(code >> 8);
    P = dp4a_us(g0, q0, P);
    P = dp4a_us(g1, q1, P);
    N = dp4a_us(g0 & sign_mask4(sign8 & 0xFu), q0, N);
    N = dp4a_us(g1 & sign_mask4(sign8 >> 4), q1, N);
}

template <int FMT> struct GranPlain {   // the common activation side: one 32-weight sub-block per lane
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    using Acts = ActRegs<WORDS>;
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        uint32_t v[4];
        sp_ld128(aq, 16 * lane, v);
        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(aq, 512 + 16 * lane, v);
        a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        a.dx = sp_ldf(ad, A32 ? 4 * lane : (lane >> 3) * 32);
    }
};

template <> struct Gran<T_IQ2_XXS> : GranPlain<T_IQ2_XXS> {
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 66 * (lane >> 3);
        const int ib = lane & 7;
        uint32_t a0, a1;
        sp_ld8b_a2(p + (2 + 8 * ib), sp_low2(p) ^ 2u, a0, a1);
        int P = 0, N = 0;
#pragma unroll
        for (int l = 0; l < 4; l++)
            iq2_group(code16(cb, (a0 >> (8 * l)) & 0xFFu), ksign_byte((a1 >> (7 * l)) & 127u), a.q[2 * l], a.q[2 * l + 1], P, N);
        const int sumi = (int)(2u * (a1 >> 28) + 1u) * (P - 2 * N);
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * 0.125f * (float)sumi;
    }
};

template <> struct Gran<T_IQ2_XS> : GranPlain<T_IQ2_XS> {
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 74 * (lane >> 3);
        const int ib = lane & 7;
        uint32_t w[2];
        sp_ld8b_a2(p + (2 + 8 * ib), sp_low2(p) ^ 2u, w[0], w[1]);
        const uint32_t sc = sp_ld8(p, 66 + ib);
        int P[2] = {0, 0}, N[2] = {0, 0};
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t qv = (w[l >> 1] >> (16 * (l & 1))) & 0xFFFFu;
            iq2_group(code16(cb, qv & 511u), ksign_byte(qv >> 9), a.q[2 * l], a.q[2 * l + 1], P[l >> 1], N[l >> 1]);
        }
        const int sumi = (int)(2u * (sc & 0xFu) + 1u) * (P[0] - 2 * N[0]) + (int)(2u * (sc >> 4) + 1u) * (P[1] - 2 * N[1]);
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * 0.125f * (float)sumi;
    }
};

template <> struct Gran<T_IQ2_S> : GranPlain<T_IQ2_S> {
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 82 * (lane >> 3);
        const int ib = lane & 7;
        const uint32_t qs = sp_ld16(p, 2 + 4 * ib) | (sp_ld16(p, 4 + 4 * ib) << 16);
        const uint32_t sg = sp_ld16(p, 34 + 4 * ib) | (sp_ld16(p, 36 + 4 * ib) << 16);
        const uint32_t qh = sp_ld8(p, 66 + ib), sc = sp_ld8(p, 74 + ib);
        int P[2] = {0, 0}, N[2] = {0, 0};
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t idx = ((qs >> (8 * l)) & 0xFFu) | ((qh << (8 - 2 * l)) & 0x300u);
            iq2_group(code16(cb, idx), (sg >> (8 * l)) & 0xFFu, a.q[2 * l], a.q[2 * l + 1], P[l >> 1], N[l >> 1]);
        }
        const int sumi = (int)(2u * (sc & 0xFu) + 1u) * (P[0] - 2 * N[0]) + (int)(2u * (sc >> 4) + 1u) * (P[1] - 2 * N[1]);
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * 0.125f * (float)sumi;
    }
};

template <> struct Gran<T_IQ1_S> : GranPlain<T_IQ1_S> {
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 50 * (lane >> 3);
        const int ib = lane & 7;
        const uint32_t qs = sp_ld16(p, 2 + 4 * ib) | (sp_ld16(p, 4 + 4 * ib) << 16);
        const uint32_t qh = sp_ld16(p, 34 + 2 * ib);
        const bool minus = (qh & 0x8000u) != 0;
        int S = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t code = code16(cb, ((qs >> (8 * l)) & 0xFFu) | (((qh >> (3 * l)) & 7u) << 8));
            S = dp4a_ss(iq1_bytes(code & 0xFFu, minus), a.q[2 * l], S);
            S = dp4a_ss(iq1_bytes(code >> 8, minus), a.q[2 * l + 1], S);
        }
        const int sumi = (int)(2u * ((qh >> 12) & 7u) + 1u) * S;
        return fp16_bits_to_float(sp_ld16(p, 0)) * a.dx * 0.125f * (float)sumi;
    }
};

template <> struct Gran<T_IQ1_M> : GranPlain<T_IQ1_M> {
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1& cb, int lane) {
        const SP p = row + 56 * (lane >> 3);
        const int ib = lane & 7;
        const uint32_t qs = sp_ld16(p, 4 * ib) | (sp_ld16(p, 4 * ib + 2) << 16);
        const uint32_t qh = sp_ld16(p, 32 + 2 * ib);                 // nibble l: 3 index bits and the delta sign of group l
        const uint32_t s0 = sp_ld16(p, 48), s1 = sp_ld16(p, 50), s2 = sp_ld16(p, 52), s3 = sp_ld16(p, 54);
        const uint32_t su = (s0 >> 12) | ((s1 >> 8) & 0x00F0u) | ((s2 >> 4) & 0x0F00u) | (s3 & 0xF000u);   // the scattered fp16 super-scale
        const uint32_t scw = (ib >> 1) == 0 ? s0 : (ib >> 1) == 1 ? s1 : (ib >> 1) == 2 ? s2 : s3;
        const uint32_t t = scw >> (6 * (ib & 1));
        int S[2] = {0, 0};
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t hn = (qh >> (4 * l)) & 0xFu;
            const uint32_t code = code16(cb, ((qs >> (8 * l)) & 0xFFu) | ((hn & 7u) << 8));
            const bool minus = (hn & 8u) != 0;
            S[l >> 1] = dp4a_ss(iq1_bytes(code & 0xFFu, minus), a.q[2 * l], S[l >> 1]);
            S[l >> 1] = dp4a_ss(iq1_bytes(code >> 8, minus), a.q[2 * l + 1], S[l >> 1]);
        }
        const int sumi = (int)(2u * (t & 7u) + 1u) * S[0] + (int)(2u * ((t >> 3) & 7u) + 1u) * S[1];
        return fp16_bits_to_float(su) * a.dx * 0.125f * (float)sumi;
    }
};

// Q2_K: 84 bytes = scales[16] (low nibble scale, high nibble min, per 16 weights) | qs[64] | fp16 d | fp16 dmin; sub-block
// 4n + j of a super-block = bits 2j, 2j+1 of the 32 bytes qs[32n ..]; w = d * sc * q - dmin * m.  Rows must be 4-byte
// aligned.  bs0 / bs1: sums of the activations of the sub-block's two halves (the Q8_K bsums), from the int8 values.
template <> struct Gran<T_Q2_K> {
    static constexpr int WORDS = 8, LANES_PER_ROW = 32;
    struct Acts { uint32_t q[8]; float dx; int bs0, bs1; };
    template <bool A32>
    static Q38B_HD void load_acts(Acts& a, SP aq, SP ad, int lane) {
        uint32_t v[4];
        sp_ld128(aq, 16 * lane, v);
        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(aq, 512 + 16 * lane, v);
        a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        a.dx = sp_ldf(ad, A32 ? 4 * lane : (lane >> 3) * 32);
        a.bs0 = 0; a.bs1 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) { a.bs0 = dp4a_ss(0x01010101u, a.q[i], a.bs0); a.bs1 = dp4a_ss(0x01010101u, a.q[4 + i], a.bs1); }
    }
    template <bool A32>
    static Q38B_HD float dot(SP row, const Acts& a, const Codebook1&, int lane) {
        const SP p = row + 84 * (lane >> 3);
        const int ib = lane & 7, n = ib >> 2, j = ib & 3;
        int S0 = 0, S1 = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            S0 = dp4a_us((sp_ld32(p, 16 + 32 * n + 4 * i) >> (2 * j)) & 0x03030303u, a.q[i], S0);
            S1 = dp4a_us((sp_ld32(p, 32 + 32 * n + 4 * i) >> (2 * j)) & 0x03030303u, a.q[4 + i], S1);
        }
        const uint32_t sc = sp_ld16(p, 2 * ib);                      // scale bytes of the two 16-weight groups
        const int sumi = (int)(sc & 0xFu) * S0 + (int)((sc >> 8) & 0xFu) * S1;
        const int msum = (int)((sc >> 4) & 0xFu) * a.bs0 + (int)(sc >> 12) * a.bs1;
        const uint32_t dd = sp_ld32(p, 80);
        return fp16_bits_to_float(dd & 0xFFFFu) * a.dx * (float)sumi - fp16_bits_to_float(dd >> 16) * a.dx * (float)msum;
    }
};

// ===============================================================================================================
// Eight lanes per row ("row-group" mapping), for rows that start 8 bytes aligned and are a multiple of 8 bytes apart
// (K a multiple of 1024 with packed rows): a warp pass covers ONE super-block of FOUR rows, lane = (row lane / 8,
// sub-block s = lane % 8).  Blocks of IQ3_XXS are 98 bytes, so block b of a 4-block slice starts at 2b (mod 8) in
// every row: the alignment of every field is a compile-time property of b and each field is fetched with the widest
// aligned load (64-bit for the index bytes where they sit 8-byte aligned, one 32-bit load for the sign word where it
// sits 4-byte aligned).  The activations of a sub-block are the same for the four rows of a pass and for every pass
// of a tile, so they are kept in registers twice -- as they are and negated -- and the signs of the weights are
// applied to THEM: one PRMT picks q or -q per byte with a selector taken from a 128-entry table (one 32-bit load
// per 8 weights), one dp4a multiplies with the unsigned codebook word.  Row sums accumulate in a register over the
// blocks of the slice and are reduced over the 8 lanes of the row at the end (3 shuffles).
// ===============================================================================================================

// PRMT selectors of sign code c: low half for weights 0..3, high half for weights 4..7 of the group of eight (weight 7
// takes the parity bit): nibble i = i (keep byte i of q) or 4 + i (byte i of -q).
Q38B_HD uint32_t ksign_selectors(uint32_t c) {
    uint32_t sg = c, par = c;
    par ^= par >> 4; par ^= par >> 2; par ^= par >> 1;
    sg |= (par & 1u) << 7;
    uint32_t r = 0x32103210u;
    for (int j = 0; j < 8; j++)
        if ((sg >> j) & 1u) r |= 4u << (4 * j);
    return r;
}

// bytewise negation of four int8 values (none of them -128)
Q38B_HD uint32_t neg_bytes4(uint32_t w) { return (0x80808080u - (w & 0x7F7F7F7Fu)) ^ (~w & 0x80808080u); }

// Staged activations of the row-group mapping: 512 bytes per super-block, chunk k (0, 1: the 32 int8 values of a
// sub-block in two halves; 2, 3: their negations) of sub-block s at k * 128 + s * 16, so that the eight sub-blocks'
// k-th chunks are one conflict-free 128-byte line.  Position of activation j (0..255) of a block, negated or not:
Q38B_HD int actr_pos(int j, int negated) { return (2 * negated + ((j >> 4) & 1)) * 128 + (j >> 5) * 16 + (j & 15); }
constexpr int ACTR_BLOCK_BYTES = 512;

// tables of the row-group decoders in shared memory: codebook entry e, replica l at cb + e * 128 + l * 4; sign
// selectors of code c, replica l at sgn + c * 128 + l * 4.  The lane's offset (bits 2..6) is OR-ed into the entry's
// offset (bits 7 and up) by the same LOP3 that masks the entry number out of its word, and the table bases are the
// addresses of static arrays, i.e. immediates of the loads: a look-up costs a shift, a LOP3 and the load.
struct TablesR { SP cb; SP sgn; uint32_t lane4; };   // bases of the tables; 4 * lane
// offset of this lane's replica of the entry whose number starts at bit `bit` of w: the number moved to bit 7, masked, | lane4
Q38B_HD uint32_t entry_offset(uint32_t w, int bit, uint32_t mask, uint32_t lane4) {
    const uint32_t moved = bit < 7 ? (w << (7 - bit)) : (w >> (bit - 7));
#if defined(__CUDA_ARCH__)
    uint32_t r;   // written as the instruction: the compiler would turn the OR of disjoint bits back into an add and hoist lane4 into the base
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(moved), "r"(mask), "r"(lane4));
    return r;
#else
    return (moved & mask) | lane4;
#endif
}

struct ActsR { uint32_t q[8], nq[8]; float dx; };

template <int FMT> struct GranR;

template <> struct GranR<T_IQ3_XXS> {
    static constexpr int BB = 98;
    static Q38B_HD void load_acts(ActsR& a, SP act_block, SP actd_block, int s) {
        uint32_t v[4];
        sp_ld128(act_block, 16 * s, v);        a.q[0] = v[0]; a.q[1] = v[1]; a.q[2] = v[2]; a.q[3] = v[3];
        sp_ld128(act_block, 128 + 16 * s, v);  a.q[4] = v[0]; a.q[5] = v[1]; a.q[6] = v[2]; a.q[7] = v[3];
        sp_ld128(act_block, 256 + 16 * s, v);  a.nq[0] = v[0]; a.nq[1] = v[1]; a.nq[2] = v[2]; a.nq[3] = v[3];
        sp_ld128(act_block, 384 + 16 * s, v);  a.nq[4] = v[0]; a.nq[5] = v[1]; a.nq[6] = v[2]; a.nq[7] = v[3];
        a.dx = sp_ldf(actd_block, 0) * 0.25f;
    }
    // `row`: first byte of this lane's row in the slice (a multiple of 8); B: block of the slice, 0..3
    template <int B>
    static Q38B_HD float dot(SP row, int s, const ActsR& a, const TablesR& t) {
        const SP r8 = row + 8 * s, r4 = row + 4 * s;
        constexpr int P = BB * B;                    // block start; P % 8 == 2 * B
        uint32_t i0, i1, aux;
        if (B == 0) {                                // index bytes at P + 2 (mod 8 = 2), sign word at 2 (mod 4)
            uint32_t x0, x1;
            sp_ld64(r8, P, x0, x1);
            const uint32_t h = sp_ld16(r8, P + 8);
            i0 = funnel_r(x0, x1, 16);
            i1 = prmt(x1, h, 0x5432u);
            aux = prmt(sp_ld16(r4, P + 66), sp_ld16(r4, P + 68), 0x5410u);
        } else if (B == 1) {                         // index bytes at 4 (mod 8), sign word at 0 (mod 4)
            i0 = sp_ld32(r8, P + 2);
            i1 = sp_ld32(r8, P + 6);
            aux = sp_ld32(r4, P + 66);
        } else if (B == 2) {                         // index bytes at 6 (mod 8), sign word at 2 (mod 4)
            uint32_t x0, x1;
            const uint32_t h = sp_ld16(r8, P + 2);
            sp_ld64(r8, P + 4, x0, x1);
            i0 = prmt(h, x0, 0x5410u);
            i1 = funnel_r(x0, x1, 16);
            aux = prmt(sp_ld16(r4, P + 66), sp_ld16(r4, P + 68), 0x5410u);
        } else {                                     // index bytes at 0 (mod 8), sign word at 0 (mod 4)
            sp_ld64(r8, P + 2, i0, i1);
            aux = sp_ld32(r4, P + 66);
        }
        int sum = 0;
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint32_t sel = sp_ld32(t.sgn + (int)entry_offset(aux, 7 * l, 0x3F80u, t.lane4));
            const uint32_t w = l < 2 ? i0 : i1;
            const uint32_t g0 = sp_ld32(t.cb + (int)entry_offset(w, 16 * (l & 1), 0x7F80u, t.lane4));
            const uint32_t g1 = sp_ld32(t.cb + (int)entry_offset(w, 16 * (l & 1) + 8, 0x7F80u, t.lane4));
            sum = dp4a_us(g0, prmt(a.q[2 * l], a.nq[2 * l], sel), sum);
            sum = dp4a_us(g1, prmt(a.q[2 * l + 1], a.nq[2 * l + 1], sel >> 16), sum);
        }
        const int sumi = (int)(2u * (aux >> 28) + 1u) * sum;
        return fp16_bits_to_float(sp_ld16(row, P)) * a.dx * (float)sumi;
    }
};

}  // namespace q38b
