// q38b_decode.cuh -- per-format tensor-core fragment builders of the quantized matvec.
//
// One warp multiplies a 16-row x 128-weight slice of a GGUF weight matrix (half of a 256-weight
// super-block of each of 16 rows, staged in shared memory in its file layout) with up to 8
// int8 activation columns.  Lane (g = lane / 4, t = lane % 4) decodes weights of rows g and g + 8
// straight into the A fragments of mma.sync.m16n8k32.s8 (m16n8k16 for Q6_K, whose scale changes
// every 16 weights); the activations are the B fragments.  Each mma yields exact int32 dot
// products of one 32-weight sub-block, which are multiplied by the integer sub-block scale and
// summed in int32; one float multiply-add per half super-block applies d_weight * d_activation.
// These are the same exact integer sums as the reference CPU kernels form
// (src/cpu/cpu_kernels.cpp:130-515 of the reference project), so results differ from them only by
// the order of the float additions.
//
// The order of the 32 k-slots of one mma is free as long as A and B agree.  Every format maps lane
// t to the 8 weights that its own bytes hold, so no data is exchanged between lanes:
//   IQ3_XXS, IQ3_S, Q4_K, Q5_K, Q8_0: weights 8t..8t+7 of the sub-block (B = 8 consecutive int8);
//   IQ4_XS: weights 4t..4t+3 and 16+4t..19+4t interleaved (activations are staged in that order);
//   Q6_K:   weights 4t..4t+3 of each 16-weight group (k16 mma).
//
// The file compiles for the device and, with the warp-collective operations replaced by an
// emulation that the CPU unit test provides, for the host.
#pragma once
#include <cstdint>
#include <cstring>
#include <cmath>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define Q38B_HD __host__ __device__ __forceinline__
#else
#define Q38B_HD inline
#endif

namespace q38b {

// ggml type ids (the reference keeps them verbatim: include/q38rt/q38rt_types.h:36-67)
enum : int { T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ3_XXS = 18, T_IQ3_S = 21, T_IQ4_XS = 23,
              // one-column kernel, dequantizer and prefill GEMM only (several columns run one after the other):
              T_Q2_K = 10, T_IQ2_XXS = 16, T_IQ2_XS = 17, T_IQ1_S = 19, T_IQ2_S = 22, T_IQ1_M = 29 };

#if !defined(__CUDA_ARCH__)
// Host emulation hooks (defined by the CPU unit test): current lane, warp-wide mma and shuffle.
int emul_lane();
void emul_mma(int (&c)[4], const uint32_t* a, int n_a, const uint32_t* b, int n_b);
uint32_t emul_shfl(uint32_t v, int src_lane);
#endif

// ------------------------------------------------------------------------------------------------
// Scalar helpers
// ------------------------------------------------------------------------------------------------
Q38B_HD int lane_id() {
#if defined(__CUDA_ARCH__)
    return (int)(threadIdx.x & 31u);
#else
    return emul_lane();
#endif
}

// PRMT: byte i of the result = byte (sel nibble i & 7) of {a (bytes 0-3), b (bytes 4-7)}; nibble bit 3 set
// replicates that byte's sign bit instead.
Q38B_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
#else
    const uint64_t v = (uint64_t)a | ((uint64_t)b << 32);
    uint32_t r = 0;
    for (int i = 0; i < 4; i++) {
        const uint32_t n = (sel >> (4 * i)) & 0xF;
        uint32_t byte = (uint32_t)(v >> (8 * (n & 7))) & 0xFF;
        if (n & 8) byte = (byte & 0x80) ? 0xFF : 0x00;
        r |= byte << (8 * i);
    }
    return r;
#endif
}

Q38B_HD int popc(uint32_t v) {
#if defined(__CUDA_ARCH__)
    return __popc(v);
#else
    return __builtin_popcount(v);
#endif
}

Q38B_HD float fp16_bits_to_float(uint32_t h) {
#if defined(__CUDA_ARCH__)
    return __half2float(__ushort_as_half((unsigned short)h));   // exact, subnormals included
#else
    const uint32_t sign = (h & 0x8000u) << 16;
    int exp = (h >> 10) & 0x1F;
    uint32_t mant = h & 0x3FFu, bits;
    if (exp == 0) {
        if (!mant) bits = sign;
        else { int e = 113; while (!(mant & 0x400u)) { mant <<= 1; e--; } bits = sign | ((uint32_t)e << 23) | ((mant & 0x3FFu) << 13); }
    } else if (exp == 31) bits = sign | 0x7F800000u | (mant << 13);
    else bits = sign | ((uint32_t)(exp + 112) << 23) | (mant << 13);
    float f; memcpy(&f, &bits, 4); return f;
#endif
}

// Loads from the staged bytes (shared memory on the device).  Blocks of several formats are only
// 2-byte aligned, so 32-bit fields of those formats are read as two halves.
Q38B_HD uint32_t ld_u8(const uint8_t* p) { return *p; }
Q38B_HD uint32_t ld_u16(const uint8_t* p) { return *(const uint16_t*)p; }
Q38B_HD uint32_t ld_u32(const uint8_t* p) { return *(const uint32_t*)p; }
Q38B_HD uint32_t ld_u32_a2(const uint8_t* p) { return ld_u16(p) | (ld_u16(p + 2) << 16); }
Q38B_HD void ld_u64(const uint8_t* p, uint32_t& lo, uint32_t& hi) {
#if defined(__CUDA_ARCH__)
    const uint2 v = *(const uint2*)p;
    lo = v.x; hi = v.y;
#else
    memcpy(&lo, p, 4); memcpy(&hi, p + 4, 4);
#endif
}

// D(16x8,s32) = A(16x32,s8) * B(32x8,s8) + C.  Fragment layout of PTX mma.m16n8k32 (g = lane/4, t = lane%4):
// a0 = A[g][4t..4t+3], a1 = A[g+8][4t..], a2 = A[g][16+4t..], a3 = A[g+8][16+4t..]; b0 = B[4t..4t+3][g],
// b1 = B[16+4t..][g]; c0,c1 = C[g][2t,2t+1], c2,c3 = C[g+8][2t,2t+1].
Q38B_HD void mma_k32(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
#if defined(__CUDA_ARCH__)
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
#else
    const uint32_t a[4] = {a0, a1, a2, a3}, b[2] = {b0, b1};
    emul_mma(c, a, 4, b, 2);
#endif
}
// k16 variant: a0 = A[g][4t..4t+3], a1 = A[g+8][4t..]; b0 = B[4t..4t+3][g].
Q38B_HD void mma_k16(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
#if defined(__CUDA_ARCH__)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(b0));
#else
    const uint32_t a[2] = {a0, a1}, b[1] = {b0};
    emul_mma(c, a, 2, b, 1);
#endif
}

// Byte mask (0xFF where the sign bit is set) for 4 weights from a 4-bit field: one multiply moves
// bit i to the top bit of byte i (the shifted copies never overlap, so no carries), PRMT's
// sign-replicate mode widens each top bit to a whole byte.  `nib` may carry garbage in bits 4..6.
Q38B_HD uint32_t sign_mask4(uint32_t nib) { return prmt(nib * 0x10204080u, 0u, 0xBA98u); }

// Negate the bytes of g selected by mask m (0xFF / 0x00 per byte).  Codebook magnitudes are never 0,
// so (g ^ 0xFF) + 1 = 256 - g stays inside its byte.
Q38B_HD uint32_t negate_bytes(uint32_t g, uint32_t m) { return (g ^ m) + (m & 0x01010101u); }

// Activation operand of one lane for one super-block.
struct ActLane {
    const uint8_t* q;   // int8 activations of column g for this super-block (256 bytes, staged order); unused if !valid
    bool valid;         // column g < nb
    float dx0, dx1;     // Q8_K block scales of columns 2t and 2t+1 (0 beyond nb)
};

Q38B_HD void load_b64(const ActLane& a, int off, uint32_t& b0, uint32_t& b1) {
    b0 = 0; b1 = 0;
    if (a.valid) ld_u64(a.q + off, b0, b1);
}
Q38B_HD uint32_t load_b32(const ActLane& a, int off) { return a.valid ? ld_u32(a.q + off) : 0u; }

// Codebook in shared memory, replicated so that lane l reads bank l: entry e, replica r at
// word (e << rep_log2) + r, r = lane & (2^rep_log2 - 1).
struct Codebook {
    const uint32_t* words;
    int rep_log2;
    uint32_t lane_word;   // lane & (replicas - 1)
};
Q38B_HD uint32_t cb_lookup(const Codebook& cb, uint32_t e) { return cb.words[(e << cb.rep_log2) + cb.lane_word]; }

// Position inside a 32-activation sub-block at which activation k is staged for a format.
Q38B_HD int act_stage_pos(int fmt, int k) {
    if (fmt != T_IQ4_XS) return k;
    // lane t holds qs bytes 4t..4t+3; nibbles in selector order: (4t, 16+4t, 4t+1, 17+4t | 4t+2, 18+4t, 4t+3, 19+4t)
    const int hi = k >> 4, r = k & 15, t = r >> 2, i = r & 3;
    return 8 * t + 2 * i + hi;
}

template <int FMT> struct Unit;

// ------------------------------------------------------------------------------------------------
// IQ3_XXS: 98 bytes = fp16 d | 64 grid indices | 8 x u32 (4 x 7 sign-index bits + 4-bit scale).
// w = d * (0.5 + s) * 0.5 * grid * sign (src/quant/quant_ref.cpp:165-188); integer form
// sum (2s+1) * grid * sign * q8, scaled by d * dx * 0.25 (src/cpu/cpu_kernels.cpp:164-189).
// ------------------------------------------------------------------------------------------------
template <> struct Unit<T_IQ3_XXS> {
    static constexpr int BLOCK_BYTES = 98;
    static constexpr int CODEBOOK_ENTRIES = 256;

    // 8 signed weights of one row: grid words of two index bytes with the 7+1 parity-coded signs applied.
    static Q38B_HD void row_frag(const uint8_t* p, int s, int t, const Codebook& cb, uint32_t& lo, uint32_t& hi, int& scale) {
        const uint32_t idx = ld_u16(p + 2 + 8 * s + 2 * t);
        const uint32_t aux = ld_u32_a2(p + 66 + 4 * s);
        const uint32_t s7 = (aux >> (7 * t)) & 127u;
        const uint32_t g0 = cb_lookup(cb, idx & 0xFFu), g1 = cb_lookup(cb, idx >> 8);
        // signs 0..3: low bits of s7; signs 4..6: bits 4..6; sign 7 = parity of the seven (top bit of byte 3)
        const uint32_t m_lo = sign_mask4(s7);
        const uint32_t hi_spread = (uint32_t)popc(s7) * 0x80000000u + s7 * 0x00020408u;
        const uint32_t m_hi = prmt(hi_spread, 0u, 0xBA98u);
        lo = negate_bytes(g0, m_lo);
        hi = negate_bytes(g1, m_hi);
        scale = (int)(2u * (aux >> 28) + 1u);
    }

    static Q38B_HD void run(const uint8_t* pA, const uint8_t* pB, int h, const ActLane& act, const Codebook& cb, float (&acc)[4]) {
        const int t = lane_id() & 3;
        int sumi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int s = 4 * h + j;
            uint32_t a0, a1, a2, a3, b0, b1;
            int scA, scB;
            row_frag(pA, s, t, cb, a0, a2, scA);
            row_frag(pB, s, t, cb, a1, a3, scB);
            load_b64(act, 32 * s + 8 * t, b0, b1);
            int c[4] = {0, 0, 0, 0};
            mma_k32(c, a0, a1, a2, a3, b0, b1);
            sumi[0] += scA * c[0]; sumi[1] += scA * c[1];
            sumi[2] += scB * c[2]; sumi[3] += scB * c[3];
        }
        const float dA = fp16_bits_to_float(ld_u16(pA)), dB = fp16_bits_to_float(ld_u16(pB));
        acc[0] = fmaf(dA * act.dx0 * 0.25f, (float)sumi[0], acc[0]);
        acc[1] = fmaf(dA * act.dx1 * 0.25f, (float)sumi[1], acc[1]);
        acc[2] = fmaf(dB * act.dx0 * 0.25f, (float)sumi[2], acc[2]);
        acc[3] = fmaf(dB * act.dx1 * 0.25f, (float)sumi[3], acc[3]);
    }
};

// ------------------------------------------------------------------------------------------------
// IQ3_S: 110 bytes = fp16 d | qs[64] | qh[8] (9th index bits) | signs[32] | scales[4] (nibbles).
// w = d * (1 + 2 ls) * grid * sign (src/quant/quant_ref.cpp:190-225; src/cpu/cpu_kernels.cpp:130-162).
// ------------------------------------------------------------------------------------------------
template <> struct Unit<T_IQ3_S> {
    static constexpr int BLOCK_BYTES = 110;
    static constexpr int CODEBOOK_ENTRIES = 512;

    static Q38B_HD void row_frag(const uint8_t* p, int s, int t, const Codebook& cb, uint32_t& lo, uint32_t& hi, int& scale) {
        const uint32_t idx = ld_u16(p + 2 + 8 * s + 2 * t);
        const uint32_t qh = ld_u8(p + 66 + s);
        const uint32_t sg = ld_u8(p + 74 + 4 * s + t);
        const uint32_t ls = (ld_u8(p + 106 + (s >> 1)) >> (4 * (s & 1))) & 0xFu;
        // bit 2t of qh is the 9th bit of the first index, bit 2t+1 of the second
        const uint32_t hb = qh >> (2 * t);
        const uint32_t g0 = cb_lookup(cb, (idx & 0xFFu) | ((hb & 1u) << 8));
        const uint32_t g1 = cb_lookup(cb, (idx >> 8) | ((hb & 2u) << 7));
        lo = negate_bytes(g0, sign_mask4(sg & 0xFu));
        hi = negate_bytes(g1, sign_mask4(sg >> 4));
        scale = (int)(2u * ls + 1u);
    }

    static Q38B_HD void run(const uint8_t* pA, const uint8_t* pB, int h, const ActLane& act, const Codebook& cb, float (&acc)[4]) {
        const int t = lane_id() & 3;
        int sumi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int s = 4 * h + j;
            uint32_t a0, a1, a2, a3, b0, b1;
            int scA, scB;
            row_frag(pA, s, t, cb, a0, a2, scA);
            row_frag(pB, s, t, cb, a1, a3, scB);
            load_b64(act, 32 * s + 8 * t, b0, b1);
            int c[4] = {0, 0, 0, 0};
            mma_k32(c, a0, a1, a2, a3, b0, b1);
            sumi[0] += scA * c[0]; sumi[1] += scA * c[1];
            sumi[2] += scB * c[2]; sumi[3] += scB * c[3];
        }
        const float dA = fp16_bits_to_float(ld_u16(pA)), dB = fp16_bits_to_float(ld_u16(pB));
        acc[0] = fmaf(dA * act.dx0, (float)sumi[0], acc[0]);
        acc[1] = fmaf(dA * act.dx1, (float)sumi[1], acc[1]);
        acc[2] = fmaf(dB * act.dx0, (float)sumi[2], acc[2]);
        acc[3] = fmaf(dB * act.dx1, (float)sumi[3], acc[3]);
    }
};

// ------------------------------------------------------------------------------------------------
// IQ4_XS: 136 bytes = fp16 d | u16 scales_h | scales_l[4] | qs[128] nibbles (low = weights 0-15, high = 16-31 of
// each 32).  w = d * (ls - 32) * levels[nibble] (src/quant/quant_ref.cpp:284-300; cpu_kernels.cpp:351-384).
// The 16-entry level table lives in four registers; PRMT uses four nibbles of the data word directly as its
// selector: the low 3 bits pick among the 8 entries of a half, and with the top bit set PRMT returns the picked byte's
// sign (zero for these tables), which separates the halves (see run).
// ------------------------------------------------------------------------------------------------
template <> struct Unit<T_IQ4_XS> {
    static constexpr int BLOCK_BYTES = 136;
    static constexpr int CODEBOOK_ENTRIES = 0;

    // levels -127,-104,-83,-65,-49,-35,-22,-10 | 1,13,25,38,53,69,89,113 as two tables of non-negative bytes: the negative
    // ones negated (127, 104, 83, 65 | 49, 35, 22, 10) and the positive ones in reverse order (113, 89, 69, 53 |
    // 38, 25, 13, 1), looked up with the data word and with its complement: see Gran<T_IQ4_XS>::dot
    static constexpr uint32_t NL0 = 0x4153687Fu, NL1 = 0x0A162331u, HR0 = 0x35455971u, HR1 = 0x010D1926u;

    static Q38B_HD int scale(const uint8_t* p, int s) {
        const uint32_t sh = ld_u16(p + 2), sl = ld_u8(p + 4 + (s >> 1));
        return (int)(((sl >> (4 * (s & 1))) & 0xFu) | (((sh >> (2 * s)) & 3u) << 4)) - 32;
    }

    static Q38B_HD void run(const uint8_t* pA, const uint8_t* pB, int h, const ActLane& act, const Codebook&, float (&acc)[4]) {
        const int t = lane_id() & 3;
        int sumi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int s = 4 * h + j;
            // The levels as two fragments of non-negative bytes, positive part and negated negative part (the two-table
            // PRMT look-up of the one-column decoder): two mma on the same activations and a subtraction cost less than
            // the masks and the merging PRMT of a single signed fragment; the tensor pipe is idle anyway.
            uint32_t b0, b1;
            const uint32_t wA = ld_u32(pA + 8 + 16 * s + 4 * t), wB = ld_u32(pB + 8 + 16 * s + 4 * t);
            load_b64(act, 32 * s + 8 * t, b0, b1);
            int c[4] = {0, 0, 0, 0}, cn[4] = {0, 0, 0, 0};
            mma_k32(c, prmt(HR0, HR1, ~wA), prmt(HR0, HR1, ~wB), prmt(HR0, HR1, ~wA >> 16), prmt(HR0, HR1, ~wB >> 16), b0, b1);
            mma_k32(cn, prmt(NL0, NL1, wA), prmt(NL0, NL1, wB), prmt(NL0, NL1, wA >> 16), prmt(NL0, NL1, wB >> 16), b0, b1);
#pragma unroll
            for (int i = 0; i < 4; i++) c[i] -= cn[i];
            const int scA = scale(pA, s), scB = scale(pB, s);
            sumi[0] += scA * c[0]; sumi[1] += scA * c[1];
            sumi[2] += scB * c[2]; sumi[3] += scB * c[3];
        }
        const float dA = fp16_bits_to_float(ld_u16(pA)), dB = fp16_bits_to_float(ld_u16(pB));
        acc[0] = fmaf(dA * act.dx0, (float)sumi[0], acc[0]);
        acc[1] = fmaf(dA * act.dx1, (float)sumi[1], acc[1]);
        acc[2] = fmaf(dB * act.dx0, (float)sumi[2], acc[2]);
        acc[3] = fmaf(dB * act.dx1, (float)sumi[3], acc[3]);
    }
};

// ------------------------------------------------------------------------------------------------
// Q4_K (144 bytes: fp16 d, dmin | scales[12] | qs[128]) and Q5_K (176 bytes: ... | qh[32] | qs[128]).
// w = d * sc * q - dmin * m (src/quant/quant_ref.cpp:57-76; src/cpu/cpu_kernels.cpp:386-433; Q5_K has no
// reference code: q gets a fifth bit from qh).  The min term sum_s m_s * (sum of the sub-block's activations) is a
// second mma whose A operand is m_s in every slot, accumulated over the four sub-blocks, so no activation block
// sums are needed.
// ------------------------------------------------------------------------------------------------
template <int NBITS> struct UnitQ45K {
    static constexpr int BLOCK_BYTES = NBITS == 5 ? 176 : 144;
    static constexpr int CODEBOOK_ENTRIES = 0;
    static constexpr int QS_OFF = NBITS == 5 ? 48 : 16;

    // 6-bit scales and mins of sub-blocks 4h..4h+3 as four bytes each (get_scale_min_k4, quant_ref.cpp:24-32)
    static Q38B_HD void scales4(const uint8_t* p, int h, uint32_t& sc4, uint32_t& mn4) {
        const uint32_t u0 = ld_u32(p + 4), u1 = ld_u32(p + 8), u2 = ld_u32(p + 12);
        if (h == 0) {
            sc4 = u0 & 0x3F3F3F3Fu;
            mn4 = u1 & 0x3F3F3F3Fu;
        } else {
            sc4 = (u2 & 0x0F0F0F0Fu) | ((u0 >> 2) & 0x30303030u);
            mn4 = ((u2 >> 4) & 0x0F0F0F0Fu) | ((u1 >> 2) & 0x30303030u);
        }
    }

    static Q38B_HD void run(const uint8_t* pA, const uint8_t* pB, int h, const ActLane& act, const Codebook&, float (&acc)[4]) {
        const int t = lane_id() & 3;
        uint32_t scA4, mnA4, scB4, mnB4;
        scales4(pA, h, scA4, mnA4);
        scales4(pB, h, scB4, mnB4);
        uint32_t hA0 = 0, hA1 = 0, hB0 = 0, hB1 = 0;
        if (NBITS == 5) {
            ld_u64(pA + 16 + 8 * t, hA0, hA1);
            ld_u64(pB + 16 + 8 * t, hB0, hB1);
        }
        int sumi[4] = {0, 0, 0, 0};
        int cm[4] = {0, 0, 0, 0};
#pragma unroll
        for (int pp = 0; pp < 2; pp++) {
            const int pair = 2 * h + pp;
            uint32_t wA0, wA1, wB0, wB1;
            ld_u64(pA + QS_OFF + 32 * pair + 8 * t, wA0, wA1);
            ld_u64(pB + QS_OFF + 32 * pair + 8 * t, wB0, wB1);
#pragma unroll
            for (int hn = 0; hn < 2; hn++) {   // low nibbles = sub-block 2*pair, high nibbles = 2*pair + 1
                const int s = 2 * pair + hn, j = 2 * pp + hn;
                uint32_t a0 = (wA0 >> (4 * hn)) & 0x0F0F0F0Fu, a2 = (wA1 >> (4 * hn)) & 0x0F0F0F0Fu;
                uint32_t a1 = (wB0 >> (4 * hn)) & 0x0F0F0F0Fu, a3 = (wB1 >> (4 * hn)) & 0x0F0F0F0Fu;
                if (NBITS == 5) {   // bit s of qh[l] -> bit 4 of weight l
                    a0 |= ((hA0 >> s) << 4) & 0x10101010u; a2 |= ((hA1 >> s) << 4) & 0x10101010u;
                    a1 |= ((hB0 >> s) << 4) & 0x10101010u; a3 |= ((hB1 >> s) << 4) & 0x10101010u;
                }
                uint32_t b0, b1;
                load_b64(act, 32 * s + 8 * t, b0, b1);
                int c[4] = {0, 0, 0, 0};
                mma_k32(c, a0, a1, a2, a3, b0, b1);
                const int scA = (int)((scA4 >> (8 * j)) & 0xFFu), scB = (int)((scB4 >> (8 * j)) & 0xFFu);
                sumi[0] += scA * c[0]; sumi[1] += scA * c[1];
                sumi[2] += scB * c[2]; sumi[3] += scB * c[3];
                const uint32_t mA = prmt(mnA4, 0u, 0x1111u * (uint32_t)j), mB = prmt(mnB4, 0u, 0x1111u * (uint32_t)j);
                mma_k32(cm, mA, mB, mA, mB, b0, b1);
            }
        }
        const uint32_t dd_A = ld_u32(pA), dd_B = ld_u32(pB);
        const float dA = fp16_bits_to_float(dd_A & 0xFFFFu), mA = fp16_bits_to_float(dd_A >> 16);
        const float dB = fp16_bits_to_float(dd_B & 0xFFFFu), mB = fp16_bits_to_float(dd_B >> 16);
        acc[0] = fmaf(dA * act.dx0, (float)sumi[0], acc[0]) - mA * act.dx0 * (float)cm[0];
        acc[1] = fmaf(dA * act.dx1, (float)sumi[1], acc[1]) - mA * act.dx1 * (float)cm[1];
        acc[2] = fmaf(dB * act.dx0, (float)sumi[2], acc[2]) - mB * act.dx0 * (float)cm[2];
        acc[3] = fmaf(dB * act.dx1, (float)sumi[3], acc[3]) - mB * act.dx1 * (float)cm[3];
    }
};
template <> struct Unit<T_Q4_K> : UnitQ45K<4> {};
template <> struct Unit<T_Q5_K> : UnitQ45K<5> {};

// ------------------------------------------------------------------------------------------------
// Q6_K: 210 bytes = ql[128] | qh[64] | int8 scales[16] | fp16 d.  w = d * sc[group of 16] * (q - 32)
// (src/quant/quant_ref.cpp:78-103; src/cpu/cpu_kernels.cpp:479-515).  One k16 mma per 16-weight group.
// Half h of the block = weights 128h..128h+127; lane t reads ql bytes l..l+3 and l+32..l+35 and qh bytes l..l+3
// for l = 16e + 4t (e = 0, 1), which hold four groups (j = 0..3): weights 128h + 32j + 16e + 4t .. +3.
// ------------------------------------------------------------------------------------------------
template <> struct Unit<T_Q6_K> {
    static constexpr int BLOCK_BYTES = 210;
    static constexpr int CODEBOOK_ENTRIES = 0;

    // four 6-bit weights per byte lane, minus 32, as int8
    static Q38B_HD uint32_t q6(uint32_t low4, uint32_t high2_at_bit4) {
        const uint32_t v = (low4 & 0x0F0F0F0Fu) | (high2_at_bit4 & 0x30303030u);
        return (v + 0x60606060u) ^ 0x80808080u;   // +96 then flip the top bit = -32 per byte, no carries (v <= 63)
    }

    static Q38B_HD void row_words(const uint8_t* p, int h, int e, int t, uint32_t (&w)[4]) {
        const int l = 16 * e + 4 * t;
        const uint32_t qa = ld_u32_a2(p + 64 * h + l), qb = ld_u32_a2(p + 64 * h + 32 + l);
        const uint32_t qh = ld_u32_a2(p + 128 + 32 * h + l);
        w[0] = q6(qa, qh << 4);
        w[1] = q6(qb, qh << 2);
        w[2] = q6(qa >> 4, qh);
        w[3] = q6(qb >> 4, qh >> 2);
    }

    static Q38B_HD void run(const uint8_t* pA, const uint8_t* pB, int h, const ActLane& act, const Codebook&, float (&acc)[4]) {
        const int t = lane_id() & 3;
        int sumi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int e = 0; e < 2; e++) {
            uint32_t wA[4], wB[4];
            row_words(pA, h, e, t, wA);
            row_words(pB, h, e, t, wB);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int grp = 8 * h + 2 * j + e;
                const uint32_t b0 = load_b32(act, 128 * h + 32 * j + 16 * e + 4 * t);
                int c[4] = {0, 0, 0, 0};
                mma_k16(c, wA[j], wB[j], b0);
                const int scA = (int)(int8_t)ld_u8(pA + 192 + grp), scB = (int)(int8_t)ld_u8(pB + 192 + grp);
                sumi[0] += scA * c[0]; sumi[1] += scA * c[1];
                sumi[2] += scB * c[2]; sumi[3] += scB * c[3];
            }
        }
        const float dA = fp16_bits_to_float(ld_u16(pA + 208)), dB = fp16_bits_to_float(ld_u16(pB + 208));
        acc[0] = fmaf(dA * act.dx0, (float)sumi[0], acc[0]);
        acc[1] = fmaf(dA * act.dx1, (float)sumi[1], acc[1]);
        acc[2] = fmaf(dB * act.dx0, (float)sumi[2], acc[2]);
        acc[3] = fmaf(dB * act.dx1, (float)sumi[3], acc[3]);
    }
};

// ------------------------------------------------------------------------------------------------
// Q8_0: eight 34-byte blocks (fp16 d | int8 qs[32]) per 256 weights; w = d * q (src/quant/quant_ref.cpp:302-308;
// the reference has no dot kernel for it).  The float scale changes every 32 weights, so each mma result is
// converted and accumulated in float.
// ------------------------------------------------------------------------------------------------
template <> struct Unit<T_Q8_0> {
    static constexpr int BLOCK_BYTES = 272;   // bytes per 256 weights
    static constexpr int CODEBOOK_ENTRIES = 0;

    static Q38B_HD void run(const uint8_t* pA, const uint8_t* pB, int h, const ActLane& act, const Codebook&, float (&acc)[4]) {
        const int t = lane_id() & 3;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int s = 4 * h + j;
            const uint8_t *bA = pA + 34 * s, *bB = pB + 34 * s;
            const uint32_t a0 = ld_u32_a2(bA + 2 + 8 * t), a2 = ld_u32_a2(bA + 6 + 8 * t);
            const uint32_t a1 = ld_u32_a2(bB + 2 + 8 * t), a3 = ld_u32_a2(bB + 6 + 8 * t);
            uint32_t b0, b1;
            load_b64(act, 32 * s + 8 * t, b0, b1);
            int c[4] = {0, 0, 0, 0};
            mma_k32(c, a0, a1, a2, a3, b0, b1);
            const float dA = fp16_bits_to_float(ld_u16(bA)), dB = fp16_bits_to_float(ld_u16(bB));
            acc[0] = fmaf(dA * act.dx0, (float)c[0], acc[0]);
            acc[1] = fmaf(dA * act.dx1, (float)c[1], acc[1]);
            acc[2] = fmaf(dB * act.dx0, (float)c[2], acc[2]);
            acc[3] = fmaf(dB * act.dx1, (float)c[3], acc[3]);
        }
    }
};

// The reference's other six formats (block layouts: src/quant/quant_formats.h:92,97-99,102-103): sizes only here; their
// decoders are the granule decoders of q38b_decode1.cuh and the exact dequantizer of q38b_act.cuh.  Their grids hold eight
// values out of three levels per entry and are kept as eight 2-bit level indices (codebooks.inc): CODE16_ENTRIES.
template <> struct Unit<T_Q2_K> { static constexpr int BLOCK_BYTES = 84, CODEBOOK_ENTRIES = 0, CODE16_ENTRIES = 0; };
template <> struct Unit<T_IQ2_XXS> { static constexpr int BLOCK_BYTES = 66, CODEBOOK_ENTRIES = 0, CODE16_ENTRIES = 256; };
template <> struct Unit<T_IQ2_XS> { static constexpr int BLOCK_BYTES = 74, CODEBOOK_ENTRIES = 0, CODE16_ENTRIES = 512; };
template <> struct Unit<T_IQ2_S> { static constexpr int BLOCK_BYTES = 82, CODEBOOK_ENTRIES = 0, CODE16_ENTRIES = 1024; };
template <> struct Unit<T_IQ1_S> { static constexpr int BLOCK_BYTES = 50, CODEBOOK_ENTRIES = 0, CODE16_ENTRIES = 2048; };
template <> struct Unit<T_IQ1_M> { static constexpr int BLOCK_BYTES = 56, CODEBOOK_ENTRIES = 0, CODE16_ENTRIES = 2048; };

// 16-bit grid codes a format keeps in shared memory (0 for the formats without such a table)
Q38B_HD constexpr int code16_entries(int fmt) {
    return fmt == T_IQ2_XXS ? 256 : fmt == T_IQ2_XS ? 512 : fmt == T_IQ2_S ? 1024 : (fmt == T_IQ1_S || fmt == T_IQ1_M) ? 2048 : 0;
}
// formats that only the one-column kernel decodes
Q38B_HD constexpr bool one_column_only(int fmt) {
    return fmt == T_Q2_K || fmt == T_IQ2_XXS || fmt == T_IQ2_XS || fmt == T_IQ2_S || fmt == T_IQ1_S || fmt == T_IQ1_M;
}

// bytes of one 256-weight super-block
Q38B_HD int block_bytes(int fmt) {
    switch (fmt) {
        case T_Q8_0: return 272; case T_Q4_K: return 144; case T_Q5_K: return 176; case T_Q6_K: return 210;
        case T_IQ3_XXS: return 98; case T_IQ3_S: return 110; case T_IQ4_XS: return 136;
        case T_Q2_K: return 84; case T_IQ2_XXS: return 66; case T_IQ2_XS: return 74; case T_IQ2_S: return 82;
        case T_IQ1_S: return 50; case T_IQ1_M: return 56; default: return 0;
    }
}

}  // namespace q38b
