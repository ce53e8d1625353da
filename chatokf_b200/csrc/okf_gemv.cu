// Decode matvec kernels (1..8 activation columns) for Q4_K, Q8_0, Q2_0 and
// IQ2_XXS.  Replaces the reference's kq_gemv_impl / kq_gemm_nb_impl / q2_0_gemv
// families (LLM/metal/Kernels.metal:26-109, :1572-1753).  See okf_gemv_mma.cuh
// for the data path and the MMA operand layout.
//
// Work split.  A tile is 16 consecutive output rows; a unit is 256 consecutive
// k of a row (one Q4_K / IQ2_XXS super-block, eight Q8_0 blocks, two Q2_0
// blocks).  A CTA owns a contiguous range of tiles.  The producer thread brings
// tiles into a ring of shared-memory stages; when whole rows fit, a stage is a
// few tiles (or half a tile) of consecutive rows and one contiguous bulk copy,
// otherwise rows are cut into k-chunks and a stage takes one segment per row.
// The eight consumer
// warps deal the units of a stage among themselves, add what they computed
// into their own slots of a partial-sum buffer, and after a group of tiles the
// slots are summed in warp order and stored, so results do not depend on
// timing.
//
// Column trick ("SEP", one or two effective columns).  MMA column g stands for
// (quarter g / 2 of the unit, effective column g % 2).  Thread c of a quad owns
// the k of quarter c and feeds x only into that quarter's columns, so the
// accumulator a thread reads back is the raw integer sum over exactly the 64 k
// whose block scales it decoded; scales, mins and biases are applied in fp32.
// More columns than two are run as several passes over column pairs, except
// for Q4_K, which has a single-pass variant ("PRE") for up to eight.
#include "okf_gemv_mma.cuh"
#include "okf_kernels.h"

namespace okf {

template <int TY> struct UnitGeom;
template <> struct UnitGeom<T_Q4_K> { static constexpr uint32_t bytes = 144; };
template <> struct UnitGeom<T_Q8_0> { static constexpr uint32_t bytes = 272; };
template <> struct UnitGeom<T_Q2_0> { static constexpr uint32_t bytes = 68; };
template <> struct UnitGeom<T_IQ2_XXS> { static constexpr uint32_t bytes = 66; };

struct GemvLayout {
    uint32_t mode;         // 0: stage = tps x 16 whole rows, 1: stage = 8 whole rows, 2: stage = 16 row segments
    uint32_t rs;           // bytes between rows inside a stage
    uint32_t stage_bytes;
    uint32_t nstage;       // ring depth
    uint32_t tps;          // tiles per stage (mode 0 only, else 1)
    uint32_t ragged;       // mode 2: row segments do not start on 16-byte boundaries
    uint32_t group;        // tiles summed per barrier
    uint32_t nc;           // real activation columns of this pass
    uint32_t ecols;        // effective (fp16) columns staged in shared memory
    uint32_t lo_off;       // fp32 activations: effective column of the lo half of column 0
    uint32_t es;           // bytes between effective columns of the x panel
    uint32_t panel;        // k-chunks whose slice of x is staged together
    uint32_t xs_off, xsum_off, red_off, zero_off, grid_off;  // byte offsets in dynamic shared memory
    uint32_t smem_bytes;
};

constexpr uint32_t kBarBytes = 256;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kConsumers = kGemvWarps * 32;
constexpr uint32_t kZeroBytes = 3 * 144 + 64 + 128;  // a column's worth of zeros for idle MMA columns

__device__ __forceinline__ uint4 lds128(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }

// 4 * NW bytes from a 2-byte aligned shared-memory address, as aligned 32-bit
// loads plus a funnel shift when the address is 2 mod 4.
template <int NW>
__device__ __forceinline__ void lds_a2(const uint8_t *p, uint32_t (&out)[NW]) {
    const uint32_t *base = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(p) & ~(uintptr_t)3);
    const uint32_t sh = ((uint32_t)reinterpret_cast<uintptr_t>(p) & 2u) * 8u;
    uint32_t w[NW + 1];
#pragma unroll
    for (int i = 0; i <= NW; i++) w[i] = base[i];
#pragma unroll
    for (int i = 0; i < NW; i++) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
}

// 6-bit (scale, min) of Q4_K sub-blocks 2c and 2c+1 (ggml get_scale_min_k4,
// LLM/Quantize/KQuants.swift:86-101), as byte pairs in the low 16 bits.
__device__ __forceinline__ void q4k_scale_min(const uint4 &h, uint32_t c, uint32_t &sc, uint32_t &mn) {
    const uint32_t sh = (c & 1) * 16;
    const uint32_t a = h.y >> sh, b = h.z >> sh, e = h.w >> sh;
    if (c < 2) {
        sc = a & 0x3F3Fu;
        mn = b & 0x3F3Fu;
    } else {
        sc = (e & 0x0F0Fu) | ((a >> 2) & 0x3030u);
        mn = ((e >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u);
    }
}

// ---- per-unit arithmetic, SEP -------------------------------------------------
// ua / ub: the unit in rows g and g + 8.  xf: this thread's 32 fp16 pairs of x in
// the order stage_x() writes them.  xq: sums of x over the two 32-wide halves of
// the thread's quarter, {lo half col 0, col 1, hi half col 0, col 1}.
// acc: rows g, g + 8 x effective columns 0, 1.
//
// Weights become exact integers in the low mantissa bits of fp16 (subnormals
// v * 2^-24), which the tensor cores multiply and sum exactly in fp32.
template <int TY>
__device__ __forceinline__ void unit_sep(const uint8_t *ua, const uint8_t *ub, uint32_t c,
                                         const uint32_t (&xf)[32], const float4 &xq,
                                         const uint64_t *grid, float (&acc)[4]) {
    float lo0[4] = {0.f, 0.f, 0.f, 0.f}, lo1[4] = {0.f, 0.f, 0.f, 0.f};  // first 32 k of the quarter
    float hi0[4] = {0.f, 0.f, 0.f, 0.f}, hi1[4] = {0.f, 0.f, 0.f, 0.f};  // last 32 k
    if constexpr (TY == T_Q4_K) {
        // {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} (LLM/Quantize/KQuants.swift:104-125).
        // Group c of qs (32 bytes): low nibbles = sub-block 2c, high = 2c+1.
        const uint4 ha = lds128(ua), hb = lds128(ub);
        const uint4 a0 = lds128(ua + 16 + 32 * c), a1 = lds128(ua + 32 + 32 * c);
        const uint4 b0 = lds128(ub + 16 + 32 * c), b1 = lds128(ub + 32 + 32 * c);
        const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            {   // bytes (b0, b2) and (b1, b3) pair up; low nibble at mantissa bit 0, high at bit 4
                const uint32_t ta = wa[i] >> 8, tb = wb[i] >> 8;
                mma_f16(lo0, wa[i] & 0x000F000Fu, wb[i] & 0x000F000Fu, ta & 0x000F000Fu, tb & 0x000F000Fu,
                        xf[2 * i], xf[2 * i + 1]);
                mma_f16(hi0, wa[i] & 0x00F000F0u, wb[i] & 0x00F000F0u, ta & 0x00F000F0u, tb & 0x00F000F0u,
                        xf[16 + 2 * i], xf[16 + 2 * i + 1]);
            }
            {
                const uint32_t ta = wa[i + 1] >> 8, tb = wb[i + 1] >> 8;
                mma_f16(lo1, wa[i + 1] & 0x000F000Fu, wb[i + 1] & 0x000F000Fu, ta & 0x000F000Fu, tb & 0x000F000Fu,
                        xf[2 * i + 2], xf[2 * i + 3]);
                mma_f16(hi1, wa[i + 1] & 0x00F000F0u, wb[i + 1] & 0x00F000F0u, ta & 0x00F000F0u, tb & 0x00F000F0u,
                        xf[16 + 2 * i + 2], xf[16 + 2 * i + 3]);
            }
        }
        uint32_t sca, mna, scb, mnb;
        q4k_scale_min(ha, c, sca, mna);
        q4k_scale_min(hb, c, scb, mnb);
        const float da = f16bits(ha.x & 0xFFFF), dma = f16bits(ha.x >> 16);
        const float db = f16bits(hb.x & 0xFFFF), dmb = f16bits(hb.x >> 16);
        // 2^24 and 2^20 undo the mantissa placement of the low and high nibbles
        const float sa0 = da * 16777216.f * byte_to_f32(sca, 0), sa1 = da * 1048576.f * byte_to_f32(sca, 1);
        const float sb0 = db * 16777216.f * byte_to_f32(scb, 0), sb1 = db * 1048576.f * byte_to_f32(scb, 1);
        const float ma0 = dma * byte_to_f32(mna, 0), ma1 = dma * byte_to_f32(mna, 1);
        const float mb0 = dmb * byte_to_f32(mnb, 0), mb1 = dmb * byte_to_f32(mnb, 1);
        acc[0] += sa0 * (lo0[0] + lo1[0]) + sa1 * (hi0[0] + hi1[0]) - ma0 * xq.x - ma1 * xq.z;
        acc[1] += sa0 * (lo0[1] + lo1[1]) + sa1 * (hi0[1] + hi1[1]) - ma0 * xq.y - ma1 * xq.w;
        acc[2] += sb0 * (lo0[2] + lo1[2]) + sb1 * (hi0[2] + hi1[2]) - mb0 * xq.x - mb1 * xq.z;
        acc[3] += sb0 * (lo0[3] + lo1[3]) + sb1 * (hi0[3] + hi1[3]) - mb0 * xq.y - mb1 * xq.w;
    } else if constexpr (TY == T_Q8_0) {
        // eight blocks {f16 d; i8 q[32]} (LLM/Gemma/Gemma4Quant.swift:51-69); thread c
        // takes blocks 2c and 2c+1.  q + 128 is an unsigned byte in the mantissa;
        // the bias leaves again as 128 * sum(x).
        uint32_t wa[17], wb[17];
        lds_a2<17>(ua + 68 * c, wa);  // {d0, q0[32], d1, q1[32]} = 68 bytes, 2-byte aligned
        lds_a2<17>(ub + 68 * c, wb);
        // word 0 = d0 | q0[0..1] << 16 ...: shift the first run of quants by two bytes;
        // the second run (after d1 in the high half of word 8) starts on word 9
        uint32_t qa[16], qb[16];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            qa[i] = __funnelshift_r(wa[i], wa[i + 1], 16);
            qb[i] = __funnelshift_r(wb[i], wb[i + 1], 16);
            qa[8 + i] = wa[9 + i];
            qb[8 + i] = wb[9 + i];
        }
        const uint32_t bias = 0x80808080u, m = 0x00FF00FFu;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t la = qa[i + h] ^ bias, lb = qb[i + h] ^ bias;
                const uint32_t ha_ = qa[8 + i + h] ^ bias, hb_ = qb[8 + i + h] ^ bias;
                mma_f16(h ? lo1 : lo0, la & m, lb & m, (la >> 8) & m, (lb >> 8) & m, xf[2 * (i + h)], xf[2 * (i + h) + 1]);
                mma_f16(h ? hi1 : hi0, ha_ & m, hb_ & m, (ha_ >> 8) & m, (hb_ >> 8) & m, xf[16 + 2 * (i + h)],
                        xf[16 + 2 * (i + h) + 1]);
            }
        }
        const float da0 = f16bits(wa[0] & 0xFFFF), da1 = f16bits(wa[8] >> 16);
        const float db0 = f16bits(wb[0] & 0xFFFF), db1 = f16bits(wb[8] >> 16);
        const float s = 16777216.f;
        acc[0] += da0 * (s * (lo0[0] + lo1[0]) - 128.f * xq.x) + da1 * (s * (hi0[0] + hi1[0]) - 128.f * xq.z);
        acc[1] += da0 * (s * (lo0[1] + lo1[1]) - 128.f * xq.y) + da1 * (s * (hi0[1] + hi1[1]) - 128.f * xq.w);
        acc[2] += db0 * (s * (lo0[2] + lo1[2]) - 128.f * xq.x) + db1 * (s * (hi0[2] + hi1[2]) - 128.f * xq.z);
        acc[3] += db0 * (s * (lo0[3] + lo1[3]) - 128.f * xq.y) + db1 * (s * (hi0[3] + hi1[3]) - 128.f * xq.w);
    } else if constexpr (TY == T_Q2_0) {
        // two blocks {f16 d; u8 qs[32]} of 128 ternary codes, weight = (code - 1) * d
        // (LLM/Base/Quant.swift:2-25).  Thread c takes half (c & 1) of block c >> 1:
        // 16 bytes = 64 codes.  A 2-bit code sits at mantissa bit p in {0,2,4,6,8};
        // x was staged multiplied by 2^(4-p), so every product is code * x * 2^-20.
        const uint8_t *pa = ua + 34 * (c >> 1), *pb = ub + 34 * (c >> 1);
        uint32_t wa[4], wb[4];
        lds_a2<4>(pa + 2 + 16 * (c & 1), wa);
        lds_a2<4>(pb + 2 + 16 * (c & 1), wb);
        const float da = f16bits(*reinterpret_cast<const uint16_t *>(pa));
        const float db = f16bits(*reinterpret_cast<const uint16_t *>(pb));
#pragma unroll
        for (int j = 0; j < 4; j++) {  // word j = 16 codes = k 16j .. 16j+15 of the quarter
            const uint32_t va = wa[j], vb = wb[j], ta = va >> 10, tb = vb >> 10;
            float(&c0)[4] = j < 2 ? lo0 : hi0;
            float(&c1)[4] = j < 2 ? lo1 : hi1;
            mma_f16(c0, va & 0x00030003u, vb & 0x00030003u, va & 0x000C000Cu, vb & 0x000C000Cu, xf[8 * j], xf[8 * j + 1]);
            mma_f16(c1, va & 0x00300030u, vb & 0x00300030u, va & 0x00C000C0u, vb & 0x00C000C0u, xf[8 * j + 2], xf[8 * j + 3]);
            mma_f16(c0, va & 0x03000300u, vb & 0x03000300u, ta & 0x00030003u, tb & 0x00030003u, xf[8 * j + 4], xf[8 * j + 5]);
            mma_f16(c1, ta & 0x000C000Cu, tb & 0x000C000Cu, ta & 0x00300030u, tb & 0x00300030u, xf[8 * j + 6], xf[8 * j + 7]);
        }
        const float s = 1048576.f;
        acc[0] += da * (s * (lo0[0] + lo1[0] + hi0[0] + hi1[0]) - xq.x - xq.z);
        acc[1] += da * (s * (lo0[1] + lo1[1] + hi0[1] + hi1[1]) - xq.y - xq.w);
        acc[2] += db * (s * (lo0[2] + lo1[2] + hi0[2] + hi1[2]) - xq.x - xq.z);
        acc[3] += db * (s * (lo0[3] + lo1[3] + hi0[3] + hi1[3]) - xq.y - xq.w);
    } else {
        // IQ2_XXS {f16 d; 8 x (u32 a0: four grid indices, u32 a1: four 7-bit sign
        // indices + 4-bit scale)} (LLM/Quantize/IQ2XXS.swift:34-53).  Thread c takes
        // sub-blocks 2c and 2c+1.  Magnitudes (8, 25, 43) go into the mantissa, the
        // sign into the fp16 sign bit; db = d * (0.5 + s) * 0.25 is applied in fp32.
        uint32_t wa[4], wb[4];
        lds_a2<4>(ua + 2 + 16 * c, wa);
        lds_a2<4>(ub + 2 + 16 * c, wb);
        const float da = f16bits(*reinterpret_cast<const uint16_t *>(ua));
        const float db = f16bits(*reinterpret_cast<const uint16_t *>(ub));
        const uint32_t m = 0x00FF00FFu, sm = 0x80008000u;
#pragma unroll
        for (int sb = 0; sb < 2; sb++) {
            const uint32_t a0a = wa[2 * sb], a1a = wa[2 * sb + 1], a0b = wb[2 * sb], a1b = wb[2 * sb + 1];
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint64_t ea = grid[(a0a >> (8 * l)) & 0xFF], eb = grid[(a0b >> (8 * l)) & 0xFF];
                // sign byte times 0x4001: bit i stays at i, bit i + 2 lands on bit i + 16
                const uint32_t sa = iq2_signs((a1a >> (7 * l)) & 127u) * 0x4001u;
                const uint32_t sb_ = iq2_signs((a1b >> (7 * l)) & 127u) * 0x4001u;
                const uint32_t la = (uint32_t)ea, ha = (uint32_t)(ea >> 32), lb = (uint32_t)eb, hb = (uint32_t)(eb >> 32);
                float(&cc)[4] = sb == 0 ? (l & 1 ? lo1 : lo0) : (l & 1 ? hi1 : hi0);
                // registers hold magnitudes (0, 2), (1, 3) then (4, 6), (5, 7) with their signs
                mma_f16(cc, (la & m) ^ ((sa << 15) & sm), (lb & m) ^ ((sb_ << 15) & sm),
                        ((la >> 8) & m) ^ ((sa << 14) & sm), ((lb >> 8) & m) ^ ((sb_ << 14) & sm),
                        xf[16 * sb + 4 * l], xf[16 * sb + 4 * l + 1]);
                mma_f16(cc, (ha & m) ^ ((sa << 11) & sm), (hb & m) ^ ((sb_ << 11) & sm),
                        ((ha >> 8) & m) ^ ((sa << 10) & sm), ((hb >> 8) & m) ^ ((sb_ << 10) & sm),
                        xf[16 * sb + 4 * l + 2], xf[16 * sb + 4 * l + 3]);
            }
        }
        // db * 2^24 = d * (0.5 + s) * 2^22
        const float sa0 = da * (0.5f + (float)(wa[1] >> 28)) * 4194304.f, sa1 = da * (0.5f + (float)(wa[3] >> 28)) * 4194304.f;
        const float sb0 = db * (0.5f + (float)(wb[1] >> 28)) * 4194304.f, sb1 = db * (0.5f + (float)(wb[3] >> 28)) * 4194304.f;
        acc[0] += sa0 * (lo0[0] + lo1[0]) + sa1 * (hi0[0] + hi1[0]);
        acc[1] += sa0 * (lo0[1] + lo1[1]) + sa1 * (hi0[1] + hi1[1]);
        acc[2] += sb0 * (lo0[2] + lo1[2]) + sb1 * (hi0[2] + hi1[2]);
        acc[3] += sb0 * (lo0[3] + lo1[3]) + sb1 * (hi0[3] + hi1[3]);
    }
}

// ---- per-unit arithmetic, Q4_K with up to eight columns ("PRE") ---------------
// The 6-bit scale is multiplied into the fp16 nibbles (exact: <= 945 * 2^-24), the
// eight sub-block sums share one accumulator, and a second MMA chain with the
// 6-bit mins in place of the weights gives the min term.
__device__ __forceinline__ void unit_q4k_pre(const uint8_t *ua, const uint8_t *ub, uint32_t c,
                                             const uint32_t (&xf)[32], float (&acc)[4]) {
    const uint4 ha = lds128(ua), hb = lds128(ub);
    const uint4 a0 = lds128(ua + 16 + 32 * c), a1 = lds128(ua + 32 + 32 * c);
    const uint4 b0 = lds128(ub + 16 + 32 * c), b1 = lds128(ub + 32 + 32 * c);
    const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    uint32_t sca, mna, scb, mnb;
    q4k_scale_min(ha, c, sca, mna);
    q4k_scale_min(hb, c, scb, mnb);
    const uint32_t sa_lo = h2_bcast(byte_to_f32(sca, 0)), sa_hi = h2_bcast(byte_to_f32(sca, 1) * 0.0625f);
    const uint32_t sb_lo = h2_bcast(byte_to_f32(scb, 0)), sb_hi = h2_bcast(byte_to_f32(scb, 1) * 0.0625f);
    const uint32_t ma_lo = h2_bcast(byte_to_f32(mna, 0)), ma_hi = h2_bcast(byte_to_f32(mna, 1));
    const uint32_t mb_lo = h2_bcast(byte_to_f32(mnb, 0)), mb_hi = h2_bcast(byte_to_f32(mnb, 1));
    float cf0[4] = {0.f, 0.f, 0.f, 0.f}, cf1[4] = {0.f, 0.f, 0.f, 0.f};
    float cm0[4] = {0.f, 0.f, 0.f, 0.f}, cm1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t ta = wa[i] >> 8, tb = wb[i] >> 8;
        mma_f16(cf0, hmul2_u(wa[i] & 0x000F000Fu, sa_lo), hmul2_u(wb[i] & 0x000F000Fu, sb_lo),
                hmul2_u(ta & 0x000F000Fu, sa_lo), hmul2_u(tb & 0x000F000Fu, sb_lo), xf[2 * i], xf[2 * i + 1]);
        mma_f16(cm0, ma_lo, mb_lo, ma_lo, mb_lo, xf[2 * i], xf[2 * i + 1]);
        mma_f16(cf1, hmul2_u(wa[i] & 0x00F000F0u, sa_hi), hmul2_u(wb[i] & 0x00F000F0u, sb_hi),
                hmul2_u(ta & 0x00F000F0u, sa_hi), hmul2_u(tb & 0x00F000F0u, sb_hi), xf[16 + 2 * i], xf[16 + 2 * i + 1]);
        mma_f16(cm1, ma_hi, mb_hi, ma_hi, mb_hi, xf[16 + 2 * i], xf[16 + 2 * i + 1]);
    }
    const float da = f16bits(ha.x & 0xFFFF), dma = f16bits(ha.x >> 16);
    const float db = f16bits(hb.x & 0xFFFF), dmb = f16bits(hb.x >> 16);
    const float fa = da * 16777216.f, fb = db * 16777216.f;
    acc[0] += fa * (cf0[0] + cf1[0]) - dma * (cm0[0] + cm1[0]);
    acc[1] += fa * (cf0[1] + cf1[1]) - dma * (cm0[1] + cm1[1]);
    acc[2] += fb * (cf0[2] + cf1[2]) - dmb * (cm0[2] + cm1[2]);
    acc[3] += fb * (cf0[3] + cf1[3]) - dmb * (cm0[3] + cm1[3]);
}

// ---- staging x ------------------------------------------------------------------
// One item is 16 consecutive k of one real column: converted to fp16 (hi and lo
// parts for fp32 input), re-ordered into the eight registers the unit code
// expects, and summed; two neighbouring items make one 32-wide sum.
//   Q4_K / Q8_0 / IQ2_XXS: register 2q + (j & 1) = (x[4q + j], x[4q + j + 2])
//   Q2_0:                  register i = (x[i], x[i + 8]) * 2^(4 - p(i)), p = 0,2,4,6,8,0,2,4
template <int TY, int XDT>
__device__ __forceinline__ void stage_x(uint8_t *xs, float *xsum, const GemvLayout &L, const void *x,
                                        uint32_t kdim, uint32_t u_first, uint32_t nu, uint32_t tid) {
    const uint32_t items_per_col = nu * 16;
    const uint32_t total = (L.nc * items_per_col + 31) & ~31u;  // whole warps, for the shuffles below
    for (uint32_t i = tid; i < total; i += kConsumers) {
        const bool live = i < L.nc * items_per_col;
        const uint32_t col = live ? i / items_per_col : 0, it = live ? i % items_per_col : 0;
        const uint32_t u = it >> 4, c = (it >> 2) & 3, q = it & 3;  // unit, quarter, 16-k piece of the quarter
        const size_t src = (size_t)col * kdim + (size_t)(u_first + u) * 256 + c * 64 + q * 16;
        float v[16];
        if (live) {
            if constexpr (XDT == DT_F32) {
                const float4 *p = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(x) + src);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float4 f = __ldg(p + j);
                    v[4 * j] = f.x; v[4 * j + 1] = f.y; v[4 * j + 2] = f.z; v[4 * j + 3] = f.w;
                }
            } else {
                const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(x) + src);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    const uint4 r = __ldg(p + j);
                    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if constexpr (XDT == DT_F16) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e]));
                            v[8 * j + 2 * e] = f.x; v[8 * j + 2 * e + 1] = f.y;
                        } else {
                            v[8 * j + 2 * e] = __uint_as_float(w[e] << 16);
                            v[8 * j + 2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
                        }
                    }
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = 0.f;
        }
        float hi[16], lo[16], shi = 0.f, slo = 0.f;
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const float cl = fminf(fmaxf(v[j], -65504.f), 65504.f);
            hi[j] = __half2float(__float2half_rn(cl));
            lo[j] = cl - hi[j];
            shi += hi[j];
            slo += lo[j];
        }
        // 32-wide sums: items 2m and 2m + 1 sit in neighbouring lanes
        shi += __shfl_xor_sync(0xffffffffu, shi, 1);
        slo += __shfl_xor_sync(0xffffffffu, slo, 1);
        if (!live) continue;
        uint32_t rh[8], rl[8];
#pragma unroll
        for (int r = 0; r < 8; r++) {
            int k0, k1;
            float sc = 1.f;
            if constexpr (TY == T_Q2_0) {
                k0 = r; k1 = r + 8;
                const int p = (r < 5 ? r : r - 5) * 2;
                sc = p == 0 ? 16.f : p == 2 ? 4.f : p == 4 ? 1.f : p == 6 ? 0.25f : 0.0625f;
            } else {
                k0 = 4 * (r >> 1) + (r & 1); k1 = k0 + 2;
            }
            if constexpr (TY == T_Q2_0) {  // the scaled copy must stay finite in fp16
                rh[r] = pack_h2(fminf(fmaxf(hi[k0] * sc, -65504.f), 65504.f), fminf(fmaxf(hi[k1] * sc, -65504.f), 65504.f));
            } else {
                rh[r] = pack_h2(hi[k0], hi[k1]);
            }
            rl[r] = pack_h2(lo[k0] * sc, lo[k1] * sc);
        }
        uint8_t *dst = xs + col * L.es + u * kXsUnit + c * 144 + q * 32;
        *reinterpret_cast<uint4 *>(dst) = make_uint4(rh[0], rh[1], rh[2], rh[3]);
        *reinterpret_cast<uint4 *>(dst + 16) = make_uint4(rh[4], rh[5], rh[6], rh[7]);
        if constexpr (XDT == DT_F32) {
            uint8_t *dl = dst + (size_t)L.lo_off * L.es;
            *reinterpret_cast<uint4 *>(dl) = make_uint4(rl[0], rl[1], rl[2], rl[3]);
            *reinterpret_cast<uint4 *>(dl + 16) = make_uint4(rl[4], rl[5], rl[6], rl[7]);
        }
        if ((q & 1) == 0 && xsum) {
            // xsum[(unit * 8 + sub-block) * 2 + effective column]; only the SEP layout uses it
            float *s = xsum + ((size_t)u * 8 + c * 2 + (q >> 1)) * 2;
            if constexpr (XDT == DT_F32) { s[0] = shi; s[1] = slo; }
            else s[col] = shi;
        }
    }
}

// ---- the kernel ---------------------------------------------------------------------
// Hooks for a timing harness that includes this file; they compile to nothing here.
#ifndef OKF_GEMV_TRACE
#define OKF_GEMV_TRACE_INIT
#define OKF_GEMV_TRACE(tag)
#endif

// Position in the ring of stages; the producer and the consumers step through it
// in the same order, so both keep one of these.
struct RingPos {
    uint32_t s = 0, use = 0;  // slot, and how many times the ring wrapped
    __device__ __forceinline__ void next(uint32_t nstage) {
        if (++s == nstage) { s = 0; use++; }
    }
};

template <int TY, int XDT, bool SEP>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_kernel(GemvArgs p, GemvLayout L) {
    constexpr uint32_t UB = UnitGeom<TY>::bytes;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kMaxStages);
    uint8_t *stages = smem + kBarBytes;
    uint8_t *xs = smem + L.xs_off;
    float *xsum = reinterpret_cast<float *>(smem + L.xsum_off);  // [unit][sub-block][2]
    float *red = reinterpret_cast<float *>(smem + L.red_off);    // [tile in group][warp][16][nc]
    uint8_t *zeros = smem + L.zero_off;
    const uint64_t *grid = reinterpret_cast<const uint64_t *>(smem + L.grid_off);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const uint32_t t0 = (uint32_t)((uint64_t)p.tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((uint64_t)p.tiles * (blockIdx.x + 1) / gridDim.x);
    const uint32_t ntl = t1 - t0;
    const uint32_t spt = L.mode == 1 ? 2 : 1;  // stages per step (two half-tiles in mode 1)
    OKF_GEMV_TRACE_INIT;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < L.nstage; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kGemvWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (TY == T_IQ2_XXS) {
        uint64_t *gw = reinterpret_cast<uint64_t *>(smem + L.grid_off);
        for (uint32_t i = threadIdx.x; i < 256; i += kGemvThreads) gw[i] = g_iq2xxs_grid[i];
    }
    __syncthreads();

    // Steps are visited in the same order by the producer and the consumers: group
    // by group, inside a group k-chunk by k-chunk, inside that `tps` tiles at a time.
    if (warp == kGemvWarps) {
        // ---- producer (one thread): weights do not depend on the previous kernel,
        // so it does not wait for it
        if (lane != 0) return;
        RingPos rp;
        uint32_t issued = 0;
        for (uint32_t gb = 0; gb < ntl; gb += L.group) {
            const uint32_t gn = min(L.group, ntl - gb);
            for (uint32_t j = 0; j < p.nchunk; j++) {
                const uint32_t u0 = j * p.cb, nu = min(p.cb, p.nunit - u0);
                for (uint32_t tl = gb; tl < gb + gn; tl += L.tps) {
                    const uint32_t tn = min(L.tps, gb + gn - tl);
                    for (uint32_t half = 0; half < spt; half++, issued++) {
                        if (rp.use > 0 &&
                            !mbar_wait(&empty[rp.s], (rp.use - 1) & 1, abort_flag, p.status, kStatusEmptyTimeout)) {
                            // giving up: let the copies already issued land before the CTA goes away
                            const uint32_t first = issued > L.nstage ? issued - L.nstage : 0;
                            for (uint32_t d = first; d < issued; d++) {
                                bool landed = false;
                                for (uint32_t i = 0; i < kSpinLimit && !landed; i++)
                                    landed = mbar_try_wait(&full[d % L.nstage], (d / L.nstage) & 1);
                            }
                            return;
                        }
                        const uint32_t row0 = (t0 + tl) * 16 + half * 8;
                        uint8_t *dst = stages + (size_t)rp.s * L.stage_bytes;
                        if (L.mode != 2) {
                            // whole rows: one copy; the byte count is rounded up to 16, which may
                            // read a few bytes past the last row (weight buffers are padded)
                            const uint32_t want = L.mode == 1 ? 8u : 16u * tn;
                            const uint32_t nrows = row0 < p.m ? min(want, p.m - row0) : 0u;
                            const uint32_t bytes = (nrows * p.row_bytes + 15u) & ~15u;
                            mbar_expect_tx(&full[rp.s], bytes);
                            if (bytes) bulk_g2s(dst, p.w + (size_t)row0 * p.row_bytes, bytes, &full[rp.s]);
                        } else {
                            // one copy per row segment.  A segment may start anywhere (2-byte
                            // aligned layouts): the copy starts at the 16-byte boundary below it
                            // and the consumers skip the same few bytes.
                            const uint32_t seg = nu * UB;
                            uint32_t total = 0;
                            for (uint32_t r = 0; r < 16; r++) {
                                const size_t src = (size_t)min(row0 + r, p.m - 1) * p.row_bytes + (size_t)u0 * UB;
                                total += ((uint32_t)(src & 15) + seg + 15u) & ~15u;
                            }
                            mbar_expect_tx(&full[rp.s], total);
                            for (uint32_t r = 0; r < 16; r++) {
                                const size_t src = (size_t)min(row0 + r, p.m - 1) * p.row_bytes + (size_t)u0 * UB;
                                const uint32_t skew = (uint32_t)(src & 15);
                                bulk_g2s(dst + (size_t)r * L.rs, p.w + (src - skew), (skew + seg + 15u) & ~15u, &full[rp.s]);
                            }
                        }
                        OKF_GEMV_TRACE(1);
                        rp.next(L.nstage);
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    OKF_GEMV_TRACE(2);
    pdl_wait();  // activations come from the previous kernel; outputs may still be read by it
    OKF_GEMV_TRACE(3);

    const uint32_t tid = threadIdx.x;  // 0 .. kConsumers - 1
    // A wait that gives up marks the warp dead; a dead warp skips further waits but
    // keeps walking the loops, so the barriers among the consumer warps still match.
    bool alive = true;
    auto wait_full = [&](uint32_t s, uint32_t use) {
        bool ok = true;
        if (alive && lane == 0) ok = mbar_wait(&full[s], use & 1, abort_flag, p.status, kStatusFullTimeout);
        alive = alive && __shfl_sync(0xffffffffu, ok, 0);
    };
    auto consumer_sync = [&]() { named_bar_sync(1, kConsumers); };

    // Which effective column of x this thread feeds into the MMA (column g of B).
    // Threads with nothing to feed read a block of zeros laid out like a column,
    // so the inner loop has no divergence.
    bool x_active;
    uint32_t x_col;
    if constexpr (SEP) {
        x_col = g & 1;
        x_active = (g >> 1) == c && x_col < L.ecols;
    } else {
        x_col = g;
        x_active = XDT == DT_F32 ? (g & 3) < p.n : g < p.n;
    }
    const uint8_t *xs_mine = x_active ? xs + x_col * L.es + c * 144 : zeros + c * 144 + (g & 1) * 64;
    const uint32_t xs_ustride = x_active ? kXsUnit : 0;
    if (tid < kZeroBytes / 4) reinterpret_cast<uint32_t *>(zeros)[tid] = 0u;

    RingPos rp;
    uint32_t rot = 0;  // the deal of units to warps rotates from step to step
    for (uint32_t gb = 0; gb < ntl; gb += L.group) {
        const uint32_t gn = min(L.group, ntl - gb);
        for (uint32_t i = tid; i < gn * kGemvWarps * 16 * L.nc; i += kConsumers) red[i] = 0.f;
        for (uint32_t j0 = 0; j0 < p.nchunk; j0 += L.panel) {
            const uint32_t j1 = min(j0 + L.panel, p.nchunk);
            const uint32_t pu0 = j0 * p.cb, pnu = min(j1 * p.cb, p.nunit) - pu0;
            if (gb == 0 || L.panel < p.nchunk) {
                // the previous panel is still being read until every warp gets here
                if (gb > 0 || j0 > 0) consumer_sync();
                stage_x<TY, XDT>(xs, SEP ? xsum : nullptr, L, p.x, p.k, pu0, pnu, tid);
            }
            consumer_sync();
            OKF_GEMV_TRACE(4);
            for (uint32_t j = j0; j < j1; j++) {
                const uint32_t u0 = j * p.cb, nu = min(p.cb, p.nunit - u0);
                const uint32_t pu = u0 - pu0;  // first unit of the chunk inside the panel
                // in whole-row stages a row holds every unit; in segment stages only this chunk's
                const uint32_t ubase = L.mode == 2 ? 0 : u0;
                for (uint32_t tl = gb; tl < gb + gn; tl += L.tps) {
                    const uint32_t tn = min(L.tps, gb + gn - tl);
                    const uint32_t sA = rp.s;
                    OKF_GEMV_TRACE(5);
                    wait_full(rp.s, rp.use);
                    rp.next(L.nstage);
                    const uint32_t sB = rp.s;
                    if (spt == 2) {
                        wait_full(rp.s, rp.use);
                        rp.next(L.nstage);
                    }
                    OKF_GEMV_TRACE(6);
                    // rows g and g + 8 of the step's first tile
                    const uint8_t *ra = stages + (size_t)sA * L.stage_bytes + (size_t)g * L.rs;
                    const uint8_t *rb = L.mode == 1 ? stages + (size_t)sB * L.stage_bytes + (size_t)g * L.rs
                                                    : ra + (size_t)8 * L.rs;
                    if (L.mode == 2 && L.ragged) {  // skip what the copy fetched below each segment's start
                        const uint32_t row = (t0 + tl) * 16 + g;
                        ra += ((size_t)min(row, p.m - 1) * p.row_bytes + (size_t)u0 * UB) & 15;
                        rb += ((size_t)min(row + 8, p.m - 1) * p.row_bytes + (size_t)u0 * UB) & 15;
                    }
                    const uint32_t tile_bytes = 16 * L.rs;
                    // this warp's units: v = first, first + 8, ... of the step's tn * nu,
                    // unit v being unit v % nu of tile v / nu
                    const uint32_t total = tn * nu;
                    uint32_t v = (warp + kGemvWarps - rot) & (kGemvWarps - 1);
                    rot = (rot + total) & (kGemvWarps - 1);
                    uint32_t ti = 0, u = v;
                    while (u >= nu && ti < tn) { u -= nu; ti++; }
                    while (v < total) {
                        float acc[4] = {0.f, 0.f, 0.f, 0.f};
                        const uint32_t cur = ti;
                        const uint8_t *ta = ra + (size_t)cur * tile_bytes, *tb = rb + (size_t)cur * tile_bytes;
                        do {
                            uint32_t xf[32];
                            {
                                const uint4 *xp = reinterpret_cast<const uint4 *>(xs_mine + (pu + u) * xs_ustride);
#pragma unroll
                                for (int q = 0; q < 8; q++) {
                                    const uint4 w4 = xp[q];
                                    xf[4 * q] = w4.x; xf[4 * q + 1] = w4.y; xf[4 * q + 2] = w4.z; xf[4 * q + 3] = w4.w;
                                }
                            }
                            const uint32_t off = (ubase + u) * UB;
                            if constexpr (SEP) {
                                const float4 xq = *reinterpret_cast<const float4 *>(xsum + ((pu + u) * 8 + 2 * c) * 2);
                                unit_sep<TY>(ta + off, tb + off, c, xf, xq, grid, acc);
                            } else {
                                unit_q4k_pre(ta + off, tb + off, c, xf, acc);
                            }
                            v += kGemvWarps;
                            u += kGemvWarps;
                            while (u >= nu && v < total) { u -= nu; ti++; }
                        } while (v < total && ti == cur);
                        // add into this warp's own slot of the tile's partial sums
                        float *dst = red + ((size_t)(tl - gb + cur) * kGemvWarps + warp) * 16 * L.nc;
                        if constexpr (SEP) {
                            // each thread of the quad covered another quarter: add them up
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
                                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
                            }
                            if (c == 0) {
                                if constexpr (XDT == DT_F32) {  // columns 0 / 1 are the hi / lo halves of x
                                    dst[g] += acc[0] + acc[1];
                                    dst[g + 8] += acc[2] + acc[3];
                                } else {
                                    dst[g * L.nc] += acc[0];
                                    dst[(g + 8) * L.nc] += acc[2];
                                    if (L.nc > 1) {
                                        dst[g * L.nc + 1] += acc[1];
                                        dst[(g + 8) * L.nc + 1] += acc[3];
                                    }
                                }
                            }
                        } else {
                            if constexpr (XDT == DT_F32) {  // columns 4..7 hold the lo halves of columns 0..3
#pragma unroll
                                for (int e = 0; e < 4; e++) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
                            }
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const uint32_t col = 2 * c + (e & 1);
                                if (col < L.nc) dst[(g + 8 * (e >> 1)) * L.nc + col] += acc[e];
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&empty[sA]);
                        if (spt == 2) mbar_arrive(&empty[sB]);
                    }
                    OKF_GEMV_TRACE(7);
                }
            }
        }
        // every warp's partials of this group are in: add them in warp order and store
        consumer_sync();
        const uint32_t per_tile = 16 * L.nc;
        for (uint32_t i = tid; i < gn * per_tile; i += kConsumers) {
            const uint32_t tl = i / per_tile, r = (i % per_tile) / L.nc, col = i % L.nc;
            const float *src = red + (size_t)tl * kGemvWarps * per_tile + r * L.nc + col;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kGemvWarps; w++) sum += src[(size_t)w * per_tile];
            const uint32_t row = (t0 + gb + tl) * 16 + r;
            if (row < p.m) p.out[(size_t)col * p.m + row] = sum;
        }
        if (gb + L.group < ntl) consumer_sync();  // before the buffer is zeroed again
    }
    OKF_GEMV_TRACE(8);
}

// Shared-memory plan.  Two CTAs share an SM (this kernel's and the next one's,
// already prefetching), so each gets at most 112 KB.
//
// Ring stages.  A bulk copy costs the copy engine about 50 ns however small it
// is, and a stage hand-over costs the producer a few hundred, so stages are
// large (20 - 46 KB) and filled by as few copies as possible: when whole rows fit,
// a stage is up to four tiles (or half a tile) of consecutive rows and one
// contiguous copy -- which also makes the 2-byte-aligned layouts copyable, since
// 8 rows always start on a 16-byte boundary -- otherwise rows are cut into
// segments of at least 2.4 KB, one copy per row, which needs 16-byte aligned rows
// and segments.  `tiles_per_cta` is the most tiles any CTA of the launch gets.
static bool gemv_layout(int ty, uint32_t nunit, uint32_t n, int xdt, bool sep, uint32_t tiles_per_cta,
                        GemvArgs &a, GemvLayout &L) {
    const uint32_t ub = ty == T_Q4_K ? 144 : ty == T_Q8_0 ? 272 : ty == T_Q2_0 ? 68 : 66;
    L.nc = n;
    L.ecols = xdt == DT_F32 ? (sep ? 2 : 8) : n;
    L.lo_off = sep ? 1 : 4;
    const uint32_t budget = 112 * 1024;
    const uint32_t per_tile = kGemvWarps * 16 * n * 4;
    L.group = 8192 / per_tile;
    if (L.group < 1) L.group = 1;
    if (L.group > tiles_per_cta) L.group = tiles_per_cta;
    const uint32_t red_bytes = L.group * per_tile;
    const uint32_t grid_bytes = ty == T_IQ2_XXS ? 2048 : 0;
    const uint32_t stage_cap = 46 * 1024;
    const uint32_t row_bytes = nunit * ub;
    // candidate plans, best first: 16 whole rows, 8 whole rows, then ever shorter row segments
    for (uint32_t plan = 0; plan < 2 + nunit; plan++) {
        uint32_t nchunk, cb, rs, stage;
        L.tps = 1;
        L.ragged = 0;
        if (plan == 0) {
            L.mode = 0; nchunk = 1; cb = nunit; rs = row_bytes;
            // several tiles per stage while they fit and the CTA still gets two steps
            while (L.tps < 4 && (L.tps + 1) * 16 * rs <= stage_cap && (L.tps + 1) * 2 <= tiles_per_cta) L.tps++;
            stage = (L.tps * 16 * rs + 15) & ~15u;
        } else if (plan == 1) { L.mode = 1; nchunk = 1; cb = nunit; rs = row_bytes; stage = (8 * rs + 15) & ~15u; }
        else {
            L.mode = 2;
            nchunk = plan;  // 2, 3, ...
            cb = (nunit + nchunk - 1) / nchunk;
            if ((nunit + cb - 1) / cb != nchunk) continue;
            const uint32_t seg = cb * ub;
            L.ragged = (row_bytes % 16 || seg % 16) ? 1 : 0;
            // Q4_K reads its blocks with 16-byte loads, and its rows are always aligned
            if (L.ragged && ty != T_IQ2_XXS && ty != T_Q2_0) continue;
            rs = L.ragged ? ((seg + 15 + 15) & ~15u) : seg;  // room for the skipped bytes and the round-up
            if (rs % 32 != 16) rs += 16;                      // rows g and g + 1 on different banks
            stage = 16 * rs;
        }
        if (stage > stage_cap) continue;
        a.nchunk = nchunk;
        a.cb = cb;
        L.rs = rs;
        L.stage_bytes = stage;
        const uint32_t per_chunk = L.ecols * cb * kXsUnit + cb * 8 * 2 * 4;  // x and its block sums
        const uint32_t small = kBarBytes + red_bytes + kZeroBytes + grid_bytes + 64 + L.ecols * 128;
        const uint32_t min_stages = L.mode == 1 ? 4 : 2;
        if (small + min_stages * stage + per_chunk > budget) continue;
        uint32_t nstage, panel;
        if (small + min_stages * stage + nchunk * per_chunk <= budget) {
            panel = nchunk;  // all of x resident, the rest goes to the ring
            nstage = (budget - small - nchunk * per_chunk) / stage;
        } else {
            nstage = min_stages;
            panel = (budget - small - min_stages * stage) / per_chunk;
        }
        // no deeper than the steps a CTA takes
        const uint32_t steps = ((tiles_per_cta + L.tps - 1) / L.tps) * nchunk * (L.mode == 1 ? 2 : 1);
        if (nstage > steps) nstage = steps < min_stages ? min_stages : steps;
        if (nstage > kMaxStages) nstage = kMaxStages;
        if (L.mode == 1) nstage &= ~1u;  // a tile takes two stages
        L.nstage = nstage;
        L.panel = panel;
        L.es = xs_col_stride(panel * cb);
        L.xs_off = kBarBytes + nstage * stage;
        L.xsum_off = (L.xs_off + L.ecols * L.es + 15) & ~15u;
        L.red_off = L.xsum_off + panel * cb * 8 * 2 * 4;
        L.zero_off = (L.red_off + red_bytes + 15) & ~15u;
        L.grid_off = (L.zero_off + kZeroBytes + 15) & ~15u;
        L.smem_bytes = L.grid_off + grid_bytes;
        if (L.smem_bytes <= budget) return true;
    }
    return false;
}

template <int TY, int XDT, bool SEP>
static cudaError_t launch_t(GemvArgs a, cudaStream_t s, int sms, int dev) {
    GemvLayout L;
    const uint32_t ctas = a.tiles < (uint32_t)sms ? a.tiles : (uint32_t)sms;
    if (!gemv_layout(TY, a.nunit, a.n, XDT, SEP, (a.tiles + ctas - 1) / ctas, a, L)) return cudaErrorInvalidConfiguration;
    static bool attr_set[64] = {};  // the opt-in is per device
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<TY, XDT, SEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = L.smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemv_kernel<TY, XDT, SEP>, a, L);
}

template <int TY>
static cudaError_t launch_ty(const GemvArgs &a, int xdt, bool sep, cudaStream_t s, int sms, int dev) {
    if (sep) {
        switch (xdt) {
        case DT_F16: return launch_t<TY, DT_F16, true>(a, s, sms, dev);
        case DT_BF16: return launch_t<TY, DT_BF16, true>(a, s, sms, dev);
        case DT_F32: return launch_t<TY, DT_F32, true>(a, s, sms, dev);
        }
    } else if constexpr (TY == T_Q4_K) {
        switch (xdt) {
        case DT_F16: return launch_t<TY, DT_F16, false>(a, s, sms, dev);
        case DT_BF16: return launch_t<TY, DT_BF16, false>(a, s, sms, dev);
        case DT_F32: return launch_t<TY, DT_F32, false>(a, s, sms, dev);
        }
    }
    return cudaErrorInvalidValue;
}

bool gemv_fast_supported(int ty, uint32_t k, uint32_t m, const void *w, const void *x, int xdt, uint32_t n,
                         int sms) {
    if (ty != T_Q4_K && ty != T_Q8_0 && ty != T_Q2_0 && ty != T_IQ2_XXS) return false;
    if (n == 0 || n > 8 || m == 0) return false;
    if (k % 256) return false;  // Q8_0 / Q2_0 rows that end inside a 256-wide unit take the simple kernel
    if ((uintptr_t)w % 16 || (uintptr_t)x % 16 || (k * (xdt == DT_F32 ? 4 : 2)) % 16) return false;
    GemvArgs a = {};
    GemvLayout L;
    const uint32_t tiles = (m + 15) / 16, ctas = tiles < (uint32_t)sms ? tiles : (uint32_t)sms;
    // the widest pass takes the most shared memory; narrower ones then fit too
    const uint32_t tpc = (tiles + ctas - 1) / ctas;
    if (!gemv_layout(ty, k / 256, xdt == DT_F32 ? 1 : (n < 2 ? n : 2), xdt, true, tpc, a, L)) return false;
    if (ty == T_Q4_K && n > (xdt == DT_F32 ? 1u : 2u)) {
        const uint32_t pre = xdt == DT_F32 ? 4 : 8;
        if (!gemv_layout(ty, k / 256, n < pre ? n : pre, xdt, false, tpc, a, L)) return false;
    }
    return true;
}

// One launch covers one or two effective columns (SEP) or, for Q4_K, up to eight
// (PRE); wider requests are cut into passes over consecutive columns.
cudaError_t launch_gemv_fast(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                             uint32_t n, float *out, int *status, cudaStream_t s, int sms, int dev,
                             uint64_t *launches) {
    GemvArgs a = {};
    a.w = w; a.status = status; a.k = k; a.m = m;
    a.nunit = k / 256;
    a.tiles = (m + 15) / 16;
    a.row_bytes = a.nunit * (ty == T_Q4_K ? 144 : ty == T_Q8_0 ? 272 : ty == T_Q2_0 ? 68 : 66);
    const size_t xsz = xdt == DT_F32 ? 4 : 2;
    const uint32_t sep_cols = xdt == DT_F32 ? 1 : 2;                    // real columns per SEP pass
    const uint32_t pre_cols = ty == T_Q4_K ? (xdt == DT_F32 ? 4 : 8) : 0;  // real columns per PRE pass
    for (uint32_t c0 = 0; c0 < n;) {
        const uint32_t left = n - c0;
        const bool sep = left <= sep_cols || pre_cols == 0;
        const uint32_t cap = sep ? sep_cols : pre_cols;
        const uint32_t take = left < cap ? left : cap;
        a.x = (const uint8_t *)x + (size_t)c0 * k * xsz;
        a.out = out + (size_t)c0 * m;
        a.n = take;
        cudaError_t e;
        switch (ty) {
        case T_Q4_K: e = launch_ty<T_Q4_K>(a, xdt, sep, s, sms, dev); break;
        case T_Q8_0: e = launch_ty<T_Q8_0>(a, xdt, sep, s, sms, dev); break;
        case T_Q2_0: e = launch_ty<T_Q2_0>(a, xdt, sep, s, sms, dev); break;
        case T_IQ2_XXS: e = launch_ty<T_IQ2_XXS>(a, xdt, sep, s, sms, dev); break;
        default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        c0 += take;
    }
    return cudaSuccess;
}

}  // namespace okf
