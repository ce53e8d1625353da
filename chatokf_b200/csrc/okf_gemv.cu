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
// The eight consumer warps deal the units of a stage among themselves, add what
// they computed into their own slots of a partial-sum buffer, and after a group
// of tiles the slots are summed in warp order and stored, so results do not
// depend on timing.
//
// Activations.  Each 256-wide unit of a column of x is reduced to 16-bit integers
// with one fp32 scale, x ~ xs * q, |q| <= 32512 (round to nearest; the step is
// 2^-15 of the unit's largest magnitude), and q is split into two signed bytes,
// q = 256 * hi + lo.  Every kernel here works on these values, so one column
// gives the same result whatever the batch width.
//
// Integer tensor cores.  Weights go into the MMA as the bytes they are stored as
// (nibbles and 2-bit codes after one AND, Q8_0 and the IQ2_XXS codebook
// untouched), x as the hi / lo bytes, mma.sync m16n8k32 with s32 accumulators:
// the sums are exact integers; scales, mins and biases are applied afterwards.
//   One column ("SEP"): MMA column g stands for (quarter g / 2 of the unit, byte
// g % 2 of x).  Thread c of a quad owns the k of quarter c and feeds x only into
// that quarter's columns, so the accumulator a thread reads back is the sum over
// exactly the 64 k whose block scales it decoded.
//   Two to four columns ("WIDE"): MMA column g stands for (activation column g / 2,
// byte g % 2); one MMA per 32-wide block, fed by all four threads of the quad.
// More than four columns are run as passes.
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
    uint32_t ecols;        // byte columns of the x panel in shared memory: hi and lo of every activation column
    uint32_t es;           // bytes between columns of the x panel
    uint32_t panel;        // k-chunks whose slice of x is staged together
    uint32_t xs_off, info_off, red_off, tab_off;  // byte offsets in dynamic shared memory
    uint32_t smem_bytes;
};

constexpr uint32_t kBarBytes = 256;
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kConsumers = kGemvWarps * 32;
// SEP x panel: a unit of a byte column is its 256 bytes in k order, except that
// in quarters 2 and 3 neighbouring 16-byte pieces are swapped; with the second
// byte column 32 (mod 128) bytes after the first, the eight lanes of a load that
// carry data (4 quarters x 2 byte columns) touch eight different bank groups.
constexpr uint32_t kXqUnit = 256;
constexpr float kXqMax = 32512.f;  // 127 * 256: hi stays a signed byte after rounding

__host__ __device__ inline uint32_t xq_col_stride(uint32_t units) {
    const uint32_t raw = units * kXqUnit;
    return raw + ((32u + 128u - raw % 128u) % 128u);
}
__host__ __device__ inline uint32_t xq_piece_offset(uint32_t c, uint32_t piece) {
    return c * 64 + ((piece ^ (c >> 1)) & 3u) * 16;
}

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
// The same for two rows at once: bytes {row a: 2c, 2c+1, row b: 2c, 2c+1}.
__device__ __forceinline__ void q4k_scale_min2(const uint4 &ha, const uint4 &hb, uint32_t c, uint32_t &sc,
                                               uint32_t &mn) {
    const uint32_t sel = (c & 1) ? 0x7632u : 0x5410u;
    const uint32_t a = __byte_perm(ha.y, hb.y, sel), b = __byte_perm(ha.z, hb.z, sel), e = __byte_perm(ha.w, hb.w, sel);
    if (c < 2) {
        sc = a & 0x3F3F3F3Fu;
        mn = b & 0x3F3F3F3Fu;
    } else {
        sc = (e & 0x0F0F0F0Fu) | ((a >> 2) & 0x30303030u);
        mn = ((e >> 4) & 0x0F0F0F0Fu) | ((b >> 2) & 0x30303030u);
    }
}

// ---- integer MMA: D (16 x 8, s32) += A (16 x 32, bytes) * B (32 x 8, signed bytes) ----
// Thread (g = lane / 4, c = lane % 4): a0 / a2 = row g, a1 / a3 = row g + 8, at
// k-slots 4c..4c+3 (a0, a1, b0) and 16+4c..16+4c+3 (a2, a3, b1); b = column g;
// d[0], d[1] = row g, columns 2c, 2c+1; d[2], d[3] = row g + 8.
template <bool SIGNED_A>
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    if constexpr (SIGNED_A)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// first of a chain: D = A * B
template <bool SIGNED_A>
__device__ __forceinline__ void imma0(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                      uint32_t b1) {
    if constexpr (SIGNED_A)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
// IQ2_XXS: byte masks (0xFF = negative) of the eight weights a 7-bit sign index stands
// for; the eighth sign is the parity of the seven (LLM/Quantize/IQ2Grid.swift:73-85).
// n * 0x00204081 puts bit j of a nibble on bit 8j (and on bits that the AND drops; no
// two of its terms meet, so nothing carries); times 0xFF a set bit fills its byte.
// Computed rather than looked up: look-ups at data-dependent addresses collide on
// shared-memory banks, and the multiplies run on the otherwise idle FMA pipe.
__device__ __forceinline__ uint2 iq2_sign_masks(uint32_t idx7) {
    const uint32_t lo = idx7 & 15u, hi = (idx7 >> 4) | ((__popc(idx7) & 1u) << 3);
    uint2 m;
    m.x = ((lo * 0x00204081u) & 0x01010101u) * 0xFFu;
    m.y = ((hi * 0x00204081u) & 0x01010101u) * 0xFFu;
    return m;
}

// sum over the hi and lo bytes of x: columns 2c (hi) and 2c+1 (lo) of one row
__device__ __forceinline__ float join_hi_lo(int hi, int lo) { return (float)(hi * 256 + lo); }

// ---- per-unit arithmetic, SEP -------------------------------------------------
// ua / ub: the unit in rows g and g + 8.  xf: this thread's 64 bytes of x (its
// quarter of the unit, the byte column its MMA column stands for; zeros in the
// lanes that feed nothing).  xi: for the two 32-wide blocks of the quarter,
// {xs of the first, xs of the second, sum of x over the first, over the second}.
// tab: IQ2_XXS codebook (256 x 8 magnitudes).
// acc: rows g and g + 8.
template <int TY>
__device__ __forceinline__ void unit_sep(const uint8_t *ua, const uint8_t *ub, uint32_t c,
                                         const uint32_t (&xf)[16], const float4 &xi, const uint2 *tab,
                                         float (&acc)[2]) {
    if constexpr (TY == T_Q4_K) {
        // {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} (LLM/Quantize/KQuants.swift:104-125).
        // Group c of qs (32 bytes): low nibbles = sub-block 2c, high = 2c+1, both in k order.
        // The high nibbles stay where they are (16 x the value); 1/16 goes into the scale.
        const uint4 ha = lds128(ua), hb = lds128(ub);
        const uint4 a0 = lds128(ua + 16 + 32 * c), a1 = lds128(ua + 32 + 32 * c);
        const uint4 b0 = lds128(ub + 16 + 32 * c), b1 = lds128(ub + 32 + 32 * c);
        const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        const uint32_t ml = 0x0F0F0F0Fu, mh = 0xF0F0F0F0u;
        int lo[4], hi[4];
        imma0<false>(lo, wa[0] & ml, wb[0] & ml, wa[1] & ml, wb[1] & ml, xf[0], xf[1]);
        imma0<false>(hi, wa[0] & mh, wb[0] & mh, wa[1] & mh, wb[1] & mh, xf[8], xf[9]);
#pragma unroll
        for (int i = 1; i < 4; i++) {
            imma<false>(lo, wa[2 * i] & ml, wb[2 * i] & ml, wa[2 * i + 1] & ml, wb[2 * i + 1] & ml, xf[2 * i], xf[2 * i + 1]);
            imma<false>(hi, wa[2 * i] & mh, wb[2 * i] & mh, wa[2 * i + 1] & mh, wb[2 * i + 1] & mh, xf[8 + 2 * i],
                        xf[9 + 2 * i]);
        }
        uint32_t sc, mn;
        q4k_scale_min2(ha, hb, c, sc, mn);
        const float da = f16bits(ha.x & 0xFFFF), dma = f16bits(ha.x >> 16);
        const float db = f16bits(hb.x & 0xFFFF), dmb = f16bits(hb.x >> 16);
        const float x0 = xi.x, x1 = xi.y * 0.0625f;
        acc[0] += da * (byte_to_f32(sc, 0) * (x0 * join_hi_lo(lo[0], lo[1])) + byte_to_f32(sc, 1) * (x1 * join_hi_lo(hi[0], hi[1]))) -
                  dma * (byte_to_f32(mn, 0) * xi.z + byte_to_f32(mn, 1) * xi.w);
        acc[1] += db * (byte_to_f32(sc, 2) * (x0 * join_hi_lo(lo[2], lo[3])) + byte_to_f32(sc, 3) * (x1 * join_hi_lo(hi[2], hi[3]))) -
                  dmb * (byte_to_f32(mn, 2) * xi.z + byte_to_f32(mn, 3) * xi.w);
    } else if constexpr (TY == T_Q8_0) {
        // eight blocks {f16 d; i8 q[32]} (LLM/Gemma/Gemma4Quant.swift:51-69); thread c
        // takes blocks 2c and 2c+1; the quants go into the MMA as they are.
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
        int lo[4], hi[4];
        imma0<true>(lo, qa[0], qb[0], qa[1], qb[1], xf[0], xf[1]);
        imma0<true>(hi, qa[8], qb[8], qa[9], qb[9], xf[8], xf[9]);
#pragma unroll
        for (int i = 1; i < 4; i++) {
            imma<true>(lo, qa[2 * i], qb[2 * i], qa[2 * i + 1], qb[2 * i + 1], xf[2 * i], xf[2 * i + 1]);
            imma<true>(hi, qa[8 + 2 * i], qb[8 + 2 * i], qa[9 + 2 * i], qb[9 + 2 * i], xf[8 + 2 * i], xf[9 + 2 * i]);
        }
        const float da0 = f16bits(wa[0] & 0xFFFF), da1 = f16bits(wa[8] >> 16);
        const float db0 = f16bits(wb[0] & 0xFFFF), db1 = f16bits(wb[8] >> 16);
        acc[0] += da0 * (xi.x * join_hi_lo(lo[0], lo[1])) + da1 * (xi.y * join_hi_lo(hi[0], hi[1]));
        acc[1] += db0 * (xi.x * join_hi_lo(lo[2], lo[3])) + db1 * (xi.y * join_hi_lo(hi[2], hi[3]));
    } else if constexpr (TY == T_Q2_0) {
        // two blocks {f16 d; u8 qs[32]} of 128 ternary codes, weight = (code - 1) * d
        // (LLM/Base/Quant.swift:2-25).  Thread c takes half (c & 1) of block c >> 1:
        // 16 bytes = 64 codes; byte t holds k 4t .. 4t+3.  Masking code s of every
        // byte of a word in place gives 4^s times the codes of k = s, 4+s, 8+s, 12+s
        // (x is staged in that order); the factors are undone on the integer sums.
        const uint8_t *pa = ua + 34 * (c >> 1), *pb = ub + 34 * (c >> 1);
        uint32_t wa[4], wb[4];
        lds_a2<4>(pa + 2 + 16 * (c & 1), wa);
        lds_a2<4>(pb + 2 + 16 * (c & 1), wb);
        const float da = f16bits(ld_u16(pa)), db = f16bits(ld_u16(pb));
        float sum[2][2];  // [32-wide half][row], times 64
#pragma unroll
        for (int sub = 0; sub < 2; sub++) {
            int t[4] = {0, 0, 0, 0};
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const uint32_t m = 0x03030303u << (2 * s);
                int d[4];
                imma0<false>(d, wa[2 * sub] & m, wb[2 * sub] & m, wa[2 * sub + 1] & m, wb[2 * sub + 1] & m,
                             xf[8 * sub + s], xf[8 * sub + 4 + s]);
#pragma unroll
                for (int e = 0; e < 4; e++) t[e] = t[e] + d[e] * (64 >> (2 * s));
            }
            sum[sub][0] = join_hi_lo(t[0], t[1]);
            sum[sub][1] = join_hi_lo(t[2], t[3]);
        }
        const float s = 0.015625f;
        acc[0] += da * (s * (xi.x * sum[0][0] + xi.y * sum[1][0]) - xi.z - xi.w);
        acc[1] += db * (s * (xi.x * sum[0][1] + xi.y * sum[1][1]) - xi.z - xi.w);
    } else {
        // IQ2_XXS {f16 d; 8 x (u32 a0: four codebook indices, u32 a1: four 7-bit sign
        // indices + 4-bit scale)} (LLM/Quantize/IQ2XXS.swift:34-53).  Thread c takes
        // sub-blocks 2c and 2c+1.  A codebook entry is eight magnitude bytes = the two
        // A registers of one row; sum(sign * mag * x) = sum(mag * x) - 2 * sum over the
        // negative positions, the second from the magnitudes ANDed with the sign's byte
        // mask.  db = d * (0.5 + s) * 0.25 is applied in fp32.
        uint32_t wa[4], wb[4];
        lds_a2<4>(ua + 2 + 16 * c, wa);
        lds_a2<4>(ub + 2 + 16 * c, wb);
        const float da = f16bits(ld_u16(ua)), db = f16bits(ld_u16(ub));
        float sum[2][2];
#pragma unroll
        for (int sb = 0; sb < 2; sb++) {
            const uint32_t a0a = wa[2 * sb], a1a = wa[2 * sb + 1], a0b = wb[2 * sb], a1b = wb[2 * sb + 1];
            int pos[4], neg[4];
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint2 ea = tab[(a0a >> (8 * l)) & 0xFF], eb = tab[(a0b >> (8 * l)) & 0xFF];
                const uint2 ma = iq2_sign_masks((a1a >> (7 * l)) & 127u), mb = iq2_sign_masks((a1b >> (7 * l)) & 127u);
                const uint32_t x0 = xf[8 * sb + 2 * l], x1 = xf[8 * sb + 2 * l + 1];
                if (l == 0) {
                    imma0<false>(pos, ea.x, eb.x, ea.y, eb.y, x0, x1);
                    imma0<false>(neg, ea.x & ma.x, eb.x & mb.x, ea.y & ma.y, eb.y & mb.y, x0, x1);
                } else {
                    imma<false>(pos, ea.x, eb.x, ea.y, eb.y, x0, x1);
                    imma<false>(neg, ea.x & ma.x, eb.x & mb.x, ea.y & ma.y, eb.y & mb.y, x0, x1);
                }
            }
            sum[sb][0] = join_hi_lo(pos[0] - 2 * neg[0], pos[1] - 2 * neg[1]);
            sum[sb][1] = join_hi_lo(pos[2] - 2 * neg[2], pos[3] - 2 * neg[3]);
        }
        const float sa0 = da * (0.5f + (float)(wa[1] >> 28)) * 0.25f, sa1 = da * (0.5f + (float)(wa[3] >> 28)) * 0.25f;
        const float sb0 = db * (0.5f + (float)(wb[1] >> 28)) * 0.25f, sb1 = db * (0.5f + (float)(wb[3] >> 28)) * 0.25f;
        acc[0] += sa0 * (xi.x * sum[0][0]) + sa1 * (xi.y * sum[1][0]);
        acc[1] += sb0 * (xi.x * sum[0][1]) + sb1 * (xi.y * sum[1][1]);
    }
}

// ---- per-unit arithmetic, up to four columns ("WIDE") ---------------------------
// MMA column g stands for (activation column g / 2, byte g % 2 of x); all four
// threads of a quad feed every MMA, thread c with the eight k [8c, 8c + 8) of a
// 32-wide block (Q2_0: k = 16w + 4b + c for word w, byte b).  One MMA per block:
// what comes back to thread (g, c) is the block's integer sum for rows g, g + 8
// and activation column c, hi and lo byte.  Block scales multiply these sums as
// integers where they are integers (Q4_K), else in fp32.
// xf: this thread's 64 bytes of x for the unit, block b in xf[2b], xf[2b+1].
// xw: {xs, -, -, -, X0..X7}: the unit's scale for column c and the integer sums
// of x over its eight blocks.  acc: rows g, g + 8 of column c.
__device__ __forceinline__ uint2 lds64(const uint8_t *p) { return *reinterpret_cast<const uint2 *>(p); }
__device__ __forceinline__ int ubyte(uint32_t v, int i) { return (int)__byte_perm(v, 0, 0x4440 + i); }

template <int TY>
__device__ __forceinline__ void unit_wide(const uint8_t *ua, const uint8_t *ub, uint32_t c, const uint32_t (&xf)[16],
                                          const float *xw, const uint2 *tab, float (&acc)[2]) {
    const float xs = xw[0];
    if constexpr (TY == T_Q4_K) {
        const uint4 ha = lds128(ua), hb = lds128(ub);
        // 6-bit scales and mins of the eight sub-blocks, four to a word (get_scale_min_k4)
        const uint32_t sa03 = ha.y & 0x3F3F3F3Fu, ma03 = ha.z & 0x3F3F3F3Fu;
        const uint32_t sa47 = (ha.w & 0x0F0F0F0Fu) | ((ha.y >> 2) & 0x30303030u);
        const uint32_t ma47 = ((ha.w >> 4) & 0x0F0F0F0Fu) | ((ha.z >> 2) & 0x30303030u);
        const uint32_t sb03 = hb.y & 0x3F3F3F3Fu, mb03 = hb.z & 0x3F3F3F3Fu;
        const uint32_t sb47 = (hb.w & 0x0F0F0F0Fu) | ((hb.y >> 2) & 0x30303030u);
        const uint32_t mb47 = ((hb.w >> 4) & 0x0F0F0F0Fu) | ((hb.z >> 2) & 0x30303030u);
        const int4 x03 = *reinterpret_cast<const int4 *>(xw + 4), x47 = *reinterpret_cast<const int4 *>(xw + 8);
        const int xb[8] = {x03.x, x03.y, x03.z, x03.w, x47.x, x47.y, x47.z, x47.w};
        const uint32_t ml = 0x0F0F0F0Fu, mh = 0xF0F0F0F0u;
        int te[4] = {0, 0, 0, 0}, to[4] = {0, 0, 0, 0};  // sum of scale * block sum: low-nibble / high-nibble blocks
        int mina = 0, minb = 0;
#pragma unroll
        for (int p = 0; p < 4; p++) {  // 32 bytes of nibbles: block 2p in the low ones, 2p+1 in the high ones
            const uint2 wa = lds64(ua + 16 + 32 * p + 8 * c), wb = lds64(ub + 16 + 32 * p + 8 * c);
            const int sa0 = ubyte(p < 2 ? sa03 : sa47, (2 * p) & 3), sa1 = ubyte(p < 2 ? sa03 : sa47, (2 * p + 1) & 3);
            const int sb0 = ubyte(p < 2 ? sb03 : sb47, (2 * p) & 3), sb1 = ubyte(p < 2 ? sb03 : sb47, (2 * p + 1) & 3);
            int d[4];
            imma0<false>(d, wa.x & ml, wb.x & ml, wa.y & ml, wb.y & ml, xf[4 * p], xf[4 * p + 1]);
            te[0] += sa0 * d[0]; te[1] += sa0 * d[1]; te[2] += sb0 * d[2]; te[3] += sb0 * d[3];
            imma0<false>(d, wa.x & mh, wb.x & mh, wa.y & mh, wb.y & mh, xf[4 * p + 2], xf[4 * p + 3]);
            to[0] += sa1 * d[0]; to[1] += sa1 * d[1]; to[2] += sb1 * d[2]; to[3] += sb1 * d[3];
            mina += ubyte(p < 2 ? ma03 : ma47, (2 * p) & 3) * xb[2 * p] + ubyte(p < 2 ? ma03 : ma47, (2 * p + 1) & 3) * xb[2 * p + 1];
            minb += ubyte(p < 2 ? mb03 : mb47, (2 * p) & 3) * xb[2 * p] + ubyte(p < 2 ? mb03 : mb47, (2 * p + 1) & 3) * xb[2 * p + 1];
        }
        const float da = f16bits(ha.x & 0xFFFF), dma = f16bits(ha.x >> 16);
        const float db = f16bits(hb.x & 0xFFFF), dmb = f16bits(hb.x >> 16);
        // The scaled sums no longer fit 256 * hi + lo in 32 bits: join them in fp32.  The
        // high-nibble sums are exact multiples of 16, taken out by a shift; everything
        // converted is below 2^24 in magnitude.
        auto join = [](int hi, int lo) { return fmaf((float)hi, 256.f, (float)lo); };
        acc[0] += xs * (da * (join(te[0], te[1]) + join(to[0] >> 4, to[1] >> 4)) - dma * (float)mina);
        acc[1] += xs * (db * (join(te[2], te[3]) + join(to[2] >> 4, to[3] >> 4)) - dmb * (float)minb);
    } else if constexpr (TY == T_Q8_0) {
        float fa = 0.f, fb = 0.f;
#pragma unroll
        for (int b = 0; b < 8; b++) {  // block b: {f16 d; i8 q[32]}, this thread's quants at 2 + 8c
            uint32_t qa[2], qb[2];
            lds_a2<2>(ua + 34 * b + 2 + 8 * c, qa);
            lds_a2<2>(ub + 34 * b + 2 + 8 * c, qb);
            int d[4];
            imma0<true>(d, qa[0], qb[0], qa[1], qb[1], xf[2 * b], xf[2 * b + 1]);
            fa += f16bits(ld_u16(ua + 34 * b)) * join_hi_lo(d[0], d[1]);
            fb += f16bits(ld_u16(ub + 34 * b)) * join_hi_lo(d[2], d[3]);
        }
        acc[0] += xs * fa;
        acc[1] += xs * fb;
    } else if constexpr (TY == T_Q2_0) {
        const int4 x03 = *reinterpret_cast<const int4 *>(xw + 4), x47 = *reinterpret_cast<const int4 *>(xw + 8);
        const int xsum[2] = {x03.x + x03.y + x03.z + x03.w, x47.x + x47.y + x47.z + x47.w};
        float fa = 0.f, fb = 0.f;
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {  // block of 128 codes: {f16 d; u8 qs[32]}
            const uint8_t *pa = ua + 34 * blk, *pb = ub + 34 * blk;
            int t[4] = {0, 0, 0, 0};
#pragma unroll
            for (int sb = 0; sb < 4; sb++) {  // 8 bytes = 32 codes; this thread takes code c of every byte
                uint32_t wa[2], wb[2];
                lds_a2<2>(pa + 2 + 8 * sb, wa);
                lds_a2<2>(pb + 2 + 8 * sb, wb);
                const uint32_t m = 0x03030303u, sh = 2 * c;
                int d[4];
                imma0<false>(d, (wa[0] >> sh) & m, (wb[0] >> sh) & m, (wa[1] >> sh) & m, (wb[1] >> sh) & m,
                             xf[8 * blk + 2 * sb], xf[8 * blk + 2 * sb + 1]);
#pragma unroll
                for (int e = 0; e < 4; e++) t[e] += d[e];
            }
            // (code - 1) * d: the sum of x over the block leaves again
            fa += f16bits(ld_u16(pa)) * (join_hi_lo(t[0], t[1]) - (float)xsum[blk]);
            fb += f16bits(ld_u16(pb)) * (join_hi_lo(t[2], t[3]) - (float)xsum[blk]);
        }
        acc[0] += xs * fa;
        acc[1] += xs * fb;
    } else {
        // IQ2_XXS: codebook entry c of every sub-block is this thread's eight weights
        float fa = 0.f, fb = 0.f;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            uint32_t wa[2], wb[2];  // a0: four codebook indices, a1: four 7-bit sign indices + 4-bit scale
            lds_a2<2>(ua + 2 + 8 * b, wa);
            lds_a2<2>(ub + 2 + 8 * b, wb);
            const uint2 ea = tab[(wa[0] >> (8 * c)) & 0xFF], eb = tab[(wb[0] >> (8 * c)) & 0xFF];
            const uint2 ma = iq2_sign_masks((wa[1] >> (7 * c)) & 127u), mb = iq2_sign_masks((wb[1] >> (7 * c)) & 127u);
            int pos[4], neg[4];
            imma0<false>(pos, ea.x, eb.x, ea.y, eb.y, xf[2 * b], xf[2 * b + 1]);
            imma0<false>(neg, ea.x & ma.x, eb.x & mb.x, ea.y & ma.y, eb.y & mb.y, xf[2 * b], xf[2 * b + 1]);
            fa += (0.5f + (float)(wa[1] >> 28)) * join_hi_lo(pos[0] - 2 * neg[0], pos[1] - 2 * neg[1]);
            fb += (0.5f + (float)(wb[1] >> 28)) * join_hi_lo(pos[2] - 2 * neg[2], pos[3] - 2 * neg[3]);
        }
        acc[0] += xs * 0.25f * f16bits(ld_u16(ua)) * fa;
        acc[1] += xs * 0.25f * f16bits(ld_u16(ub)) * fb;
    }
}

// ---- staging x ------------------------------------------------------------------
// One item is 16 consecutive k of one column; the 16 neighbouring items (lanes) of
// a 256-wide unit agree on its scale, two neighbours make one 32-wide block.
template <int XDT> struct XRaw { uint4 v[XDT == DT_F32 ? 4 : 2]; };

template <int XDT>
__device__ __forceinline__ XRaw<XDT> load16(const void *x, size_t src, bool live) {
    XRaw<XDT> r;
    constexpr int NV = XDT == DT_F32 ? 4 : 2;
    const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(x) + src * (XDT == DT_F32 ? 4 : 2));
#pragma unroll
    for (int j = 0; j < NV; j++) r.v[j] = live ? __ldg(p + j) : make_uint4(0u, 0u, 0u, 0u);
    return r;
}

// The 16 integers, the unit's scale (NaN if the unit holds a NaN, so that it
// spreads to the results as it would in a plain dot product) and the 32-wide
// block's integer sum.
template <int XDT>
__device__ __forceinline__ void quantize16(const XRaw<XDT> &raw, int (&q)[16], float &xs, int &qsum) {
    float v[16];
    if constexpr (XDT == DT_F32) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
            v[4 * j] = __uint_as_float(raw.v[j].x); v[4 * j + 1] = __uint_as_float(raw.v[j].y);
            v[4 * j + 2] = __uint_as_float(raw.v[j].z); v[4 * j + 3] = __uint_as_float(raw.v[j].w);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t w[4] = {raw.v[j].x, raw.v[j].y, raw.v[j].z, raw.v[j].w};
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
    // largest magnitude of the 256-wide unit (16 neighbouring items); a NaN anywhere
    // makes the probe below a NaN
    float m8[8], bad8[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        m8[j] = fmaxf(fabsf(v[j]), fabsf(v[j + 8]));
        bad8[j] = v[j] + v[j + 8];  // NaN if either is (inf - inf cannot matter: infs give NaN results anyway)
    }
#pragma unroll
    for (int w = 4; w >= 1; w >>= 1)
#pragma unroll
        for (int j = 0; j < w; j++) {
            m8[j] = fmaxf(m8[j], m8[j + w]);
            bad8[j] = bad8[j] + bad8[j + w];
        }
    float amax = m8[0], nanprobe = bad8[0];
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        nanprobe += __shfl_xor_sync(0xffffffffu, nanprobe, o);
    }
    const bool bad = nanprobe != nanprobe && !(amax == __int_as_float(0x7F800000));
    // an infinite amax gives 0 and xs = inf; a unit whose largest magnitude is below 1e-30
    // counts as zeros (32512 / amax would overflow, and its products vanish in fp32 anyway)
    const float inv = amax > 1e-30f ? __fdividef(kXqMax, amax) : 0.f;
    xs = bad ? __int_as_float(0x7FC00000) : amax * (1.f / kXqMax);
    int s4[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; j++) {
        q[j] = __float2int_rn(v[j] * inv);
        s4[j & 3] += q[j];
    }
    qsum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
    qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
}

// SEP: one column as hi / lo bytes.  Byte order inside an item:
//   Q4_K / Q8_0 / IQ2_XXS: k order
//   Q2_0: register s = k (s, 4+s, 8+s, 12+s), the order the masked code words come in
// info[unit * 4 + quarter] = {xs of its first block, of its second, sum of x over
// the first, over the second}.
template <int TY, int XDT>
__device__ __forceinline__ void stage_x_bytes(uint8_t *xs, float4 *info, const GemvLayout &L, const void *x,
                                              uint32_t u_first, uint32_t nu, uint32_t tid) {
    const uint32_t items = nu * 16;
    const uint32_t total = (items + 31) & ~31u;  // whole warps, for the shuffles
    constexpr uint32_t kFlight = 3;              // items a thread has in flight: the loads go out first
    for (uint32_t base = tid; base < total; base += kFlight * kConsumers) {
        XRaw<XDT> raw[kFlight];
#pragma unroll
        for (uint32_t r = 0; r < kFlight; r++) {
            const uint32_t i = base + r * kConsumers;
            raw[r] = load16<XDT>(x, (size_t)u_first * 256 + (size_t)i * 16, i < items);
        }
#pragma unroll
        for (uint32_t r = 0; r < kFlight; r++) {
            const uint32_t i = base + r * kConsumers;
            if (i >= total) break;  // the same for the whole warp
            const uint32_t u = i >> 4, c = (i >> 2) & 3, piece = i & 3;  // unit, quarter, 16-k piece of the quarter
            int q[16], qsum;
            float scale;
            quantize16<XDT>(raw[r], q, scale, qsum);
            if (i >= items) continue;
            // q + 128 = 256 * hi + (lo + 128): hi is its byte 1, lo its byte 0 with the top bit flipped
            uint32_t rh[4], rl[4];
#pragma unroll
            for (int w = 0; w < 4; w++) {
                uint32_t t[4];
#pragma unroll
                for (int b = 0; b < 4; b++) t[b] = (uint32_t)(q[TY == T_Q2_0 ? 4 * b + w : 4 * w + b] + 128);
                rh[w] = __byte_perm(__byte_perm(t[0], t[1], 0x0051), __byte_perm(t[2], t[3], 0x0051), 0x5410);
                rl[w] = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410) ^ 0x80808080u;
            }
            uint8_t *dst = xs + u * kXqUnit + xq_piece_offset(c, piece);
            *reinterpret_cast<uint4 *>(dst) = make_uint4(rh[0], rh[1], rh[2], rh[3]);
            *reinterpret_cast<uint4 *>(dst + L.es) = make_uint4(rl[0], rl[1], rl[2], rl[3]);
            if ((piece & 1) == 0) {
                float *f = reinterpret_cast<float *>(info + u * 4 + c);
                f[piece >> 1] = scale;
                f[2 + (piece >> 1)] = scale * (float)qsum;
            }
        }
    }
}

// WIDE: up to four columns, each as a hi and a lo byte column (panel columns 2j and
// 2j + 1).  Inside a unit of a byte column, thread c's 64 bytes start at 64c: eight
// bytes per 32-wide block, block after block, the 16-byte pieces of threads 2 and 3
// swapped in pairs as in the one-column panel.  The eight bytes of a block are its
// k [8c, 8c + 8) in order (Q2_0: k = 16w + 4b + c for word w, byte b).
// xw[(unit * 4 + column) * 12]: {xs, -, -, -, X0 .. X7}.
template <int TY, int XDT>
__device__ __forceinline__ void stage_x_wide(uint8_t *xs, float *xw, const GemvLayout &L, const void *x, uint32_t kdim,
                                             uint32_t u_first, uint32_t nu, uint32_t tid) {
    const uint32_t items_per_col = nu * 16;
    const uint32_t total = (L.nc * items_per_col + 31) & ~31u;
    constexpr uint32_t kFlight = 3;  // items a thread has in flight: the loads go out first
    auto where = [&](uint32_t i, bool &live, uint32_t &col, uint32_t &it) {
        live = i < L.nc * items_per_col;
        col = live ? i / items_per_col : 0;
        it = live ? i % items_per_col : 0;
    };
    for (uint32_t base_i = tid; base_i < total; base_i += kFlight * kConsumers) {
      XRaw<XDT> raw[kFlight];
#pragma unroll
      for (uint32_t r = 0; r < kFlight; r++) {
          bool live; uint32_t col, it;
          where(base_i + r * kConsumers, live, col, it);
          raw[r] = load16<XDT>(x, (size_t)col * kdim + (size_t)(u_first + (it >> 4)) * 256 + (it & 15) * 16, live);
      }
#pragma unroll
      for (uint32_t r = 0; r < kFlight; r++) {
        const uint32_t i = base_i + r * kConsumers;
        if (i >= total) break;  // the same for the whole warp
        bool live; uint32_t col, it;
        where(i, live, col, it);
        const uint32_t u = it >> 4, blk = (it >> 1) & 7, half = it & 1;  // unit, 32-wide block, 16-k half of it
        int q[16], qsum;
        float scale;
        quantize16<XDT>(raw[r], q, scale, qsum);
        if (!live) continue;
        uint8_t *base = xs + (2 * col) * L.es + u * kXqUnit;
        if constexpr (TY == T_Q2_0) {
            // k = 16 * half + 4 * b + c: thread c gets four bytes (b = 0..3) from this item
#pragma unroll
            for (int c = 0; c < 4; c++) {
                uint32_t t[4];
#pragma unroll
                for (int b = 0; b < 4; b++) t[b] = (uint32_t)(q[4 * b + c] + 128);
                const uint32_t h = __byte_perm(__byte_perm(t[0], t[1], 0x0051), __byte_perm(t[2], t[3], 0x0051), 0x5410);
                const uint32_t l = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410) ^ 0x80808080u;
                uint8_t *dst = base + xq_piece_offset(c, blk >> 1) + (blk & 1) * 8 + half * 4;
                *reinterpret_cast<uint32_t *>(dst) = h;
                *reinterpret_cast<uint32_t *>(dst + L.es) = l;
            }
        } else {
            // k = 16 * half + 0..15: threads 2 * half and 2 * half + 1 get eight bytes each
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                uint32_t h[2], l[2];
#pragma unroll
                for (int w = 0; w < 2; w++) {
                    uint32_t t[4];
#pragma unroll
                    for (int b = 0; b < 4; b++) t[b] = (uint32_t)(q[8 * cc + 4 * w + b] + 128);
                    h[w] = __byte_perm(__byte_perm(t[0], t[1], 0x0051), __byte_perm(t[2], t[3], 0x0051), 0x5410);
                    l[w] = __byte_perm(__byte_perm(t[0], t[1], 0x0040), __byte_perm(t[2], t[3], 0x0040), 0x5410) ^ 0x80808080u;
                }
                uint8_t *dst = base + xq_piece_offset(2 * half + cc, blk >> 1) + (blk & 1) * 8;
                *reinterpret_cast<uint2 *>(dst) = make_uint2(h[0], h[1]);
                *reinterpret_cast<uint2 *>(dst + L.es) = make_uint2(l[0], l[1]);
            }
        }
        float *w12 = xw + ((size_t)u * 4 + col) * 12;
        if (half == 0) {
            reinterpret_cast<int *>(w12)[4 + blk] = qsum;
            if (blk == 0) w12[0] = scale;
        }
      }
    }
}

// ---- the kernel ---------------------------------------------------------------------
// Position in the ring of stages; the producer and the consumers step through it
// in the same order, so both keep one of these.
struct RingPos {
    uint32_t s = 0, use = 0;  // slot, and how many times the ring wrapped
    __device__ __forceinline__ void next(uint32_t nstage) {
        if (++s == nstage) { s = 0; use++; }
    }
};

template <int TY, int XDT, bool SEP>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_kernel(GemvArgs p, GemvLayout L, GemvGather G) {
    constexpr uint32_t UB = UnitGeom<TY>::bytes;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kMaxStages);
    uint8_t *stages = smem + kBarBytes;
    uint8_t *xs = smem + L.xs_off;
    float4 *info = reinterpret_cast<float4 *>(smem + L.info_off);  // SEP: [unit][quarter]; WIDE: [unit][column] x 3
    float *red = reinterpret_cast<float *>(smem + L.red_off);      // [tile in group][warp][16][nc]
    const uint2 *tab = reinterpret_cast<const uint2 *>(smem + L.tab_off);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
    const uint32_t t0 = (uint32_t)((uint64_t)p.tiles * blockIdx.x / gridDim.x);
    const uint32_t t1 = (uint32_t)((uint64_t)p.tiles * (blockIdx.x + 1) / gridDim.x);
    const uint32_t ntl = t1 - t0;
    const uint32_t spt = L.mode == 1 ? 2 : 1;  // stages per step (two half-tiles in mode 1)

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
        // the codebook: 256 entries of eight magnitude bytes
        uint64_t *tw = reinterpret_cast<uint64_t *>(smem + L.tab_off);
        for (uint32_t i = threadIdx.x; i < 256; i += kGemvThreads) tw[i] = g_iq2xxs_grid[i];
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
                for (uint32_t tl = gb, tn; tl < gb + gn; tl += tn) {
                    const GemvSeg sg = gemv_segment(p, t0 + tl);
                    tn = min(min(L.tps, gb + gn - tl), sg.tile1 - (t0 + tl));  // a step stays inside one matrix
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
                        const uint32_t row0 = (t0 + tl - sg.tile0) * 16 + half * 8;
                        uint8_t *dst = stages + (size_t)rp.s * L.stage_bytes;
                        if (L.mode != 2) {
                            // whole rows: one copy; the byte count is rounded up to 16, which may
                            // read a few bytes past the last row (weight buffers are padded)
                            const uint32_t want = L.mode == 1 ? 8u : 16u * tn;
                            const uint32_t nrows = row0 < sg.m ? min(want, sg.m - row0) : 0u;
                            const uint32_t bytes = (nrows * p.row_bytes + 15u) & ~15u;
                            mbar_expect_tx(&full[rp.s], bytes);
                            if (bytes) bulk_g2s(dst, sg.w + (size_t)row0 * p.row_bytes, bytes, &full[rp.s]);
                        } else {
                            // one copy per row segment.  A segment may start anywhere (2-byte
                            // aligned layouts): the copy starts at the 16-byte boundary below it
                            // and the consumers skip the same few bytes.
                            const uint32_t seg = nu * UB;
                            uint32_t total = 0;
                            for (uint32_t r = 0; r < 16; r++) {
                                const size_t src = (size_t)min(row0 + r, sg.m - 1) * p.row_bytes + (size_t)u0 * UB;
                                total += ((uint32_t)(src & 15) + seg + 15u) & ~15u;
                            }
                            mbar_expect_tx(&full[rp.s], total);
                            for (uint32_t r = 0; r < 16; r++) {
                                const size_t src = (size_t)min(row0 + r, sg.m - 1) * p.row_bytes + (size_t)u0 * UB;
                                const uint32_t skew = (uint32_t)(src & 15);
                                bulk_g2s(dst + (size_t)r * L.rs, sg.w + (src - skew), (skew + seg + 15u) & ~15u, &full[rp.s]);
                            }
                        }
                        rp.next(L.nstage);
                    }
                }
            }
        }
        return;
    }

    // ---- consumers
    pdl_wait();  // activations come from the previous kernel; outputs may still be read by it

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

    // What this thread feeds into column g of the MMA's B operand.
    //   SEP:  byte column g % 2 of x, and only in the lanes of quarter g / 2.
    //   WIDE: byte column g of the panel (hi, lo of activation column g / 2), every lane
    //         its own 64 bytes; lanes of columns past the last one feed zeros.
    const bool x_active = SEP ? (g >> 1) == c : g < 2 * p.n;
    const uint8_t *xs_mine = xs + (SEP ? (g & 1) : g) * L.es + c * 64;
    const uint32_t xs_ustride = kXqUnit;
    const uint32_t xq_swap = (c >> 1) * 16;
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
                if constexpr (SEP) stage_x_bytes<TY, XDT>(xs, info, L, p.x, pu0, pnu, tid);
                else stage_x_wide<TY, XDT>(xs, reinterpret_cast<float *>(info), L, p.x, p.k, pu0, pnu, tid);
            }
            consumer_sync();
            for (uint32_t j = j0; j < j1; j++) {
                const uint32_t u0 = j * p.cb, nu = min(p.cb, p.nunit - u0);
                const uint32_t pu = u0 - pu0;  // first unit of the chunk inside the panel
                // in whole-row stages a row holds every unit; in segment stages only this chunk's
                const uint32_t ubase = L.mode == 2 ? 0 : u0;
                for (uint32_t tl = gb, tn; tl < gb + gn; tl += tn) {
                    const GemvSeg sg = gemv_segment(p, t0 + tl);
                    tn = min(min(L.tps, gb + gn - tl), sg.tile1 - (t0 + tl));
                    const uint32_t sA = rp.s;
                    wait_full(rp.s, rp.use);
                    rp.next(L.nstage);
                    const uint32_t sB = rp.s;
                    if (spt == 2) {
                        wait_full(rp.s, rp.use);
                        rp.next(L.nstage);
                    }
                    // rows g and g + 8 of the step's first tile
                    const uint8_t *ra = stages + (size_t)sA * L.stage_bytes + (size_t)g * L.rs;
                    const uint8_t *rb = L.mode == 1 ? stages + (size_t)sB * L.stage_bytes + (size_t)g * L.rs
                                                    : ra + (size_t)8 * L.rs;
                    if (L.mode == 2 && L.ragged) {  // skip what the copy fetched below each segment's start
                        const uint32_t row = (t0 + tl - sg.tile0) * 16 + g;
                        ra += ((size_t)min(row, sg.m - 1) * p.row_bytes + (size_t)u0 * UB) & 15;
                        rb += ((size_t)min(row + 8, sg.m - 1) * p.row_bytes + (size_t)u0 * UB) & 15;
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
                        const uint32_t cur = ti;
                        const uint8_t *ta = ra + (size_t)cur * tile_bytes, *tb = rb + (size_t)cur * tile_bytes;
                        // this warp's own slot of the tile's partial sums
                        float *dst = red + ((size_t)(tl - gb + cur) * kGemvWarps + warp) * 16 * L.nc;
                        if constexpr (SEP) {
                            float acc[2] = {0.f, 0.f};
                            do {
                                uint32_t xf[16];
                                const uint8_t *xp = xs_mine + (pu + u) * xs_ustride;
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                                    // quarters 2 and 3 keep their pieces swapped in pairs
                                    if (x_active) w4 = lds128(xp + (q >> 1) * 32 + ((q & 1) ? 16 - xq_swap : xq_swap));
                                    xf[4 * q] = w4.x; xf[4 * q + 1] = w4.y; xf[4 * q + 2] = w4.z; xf[4 * q + 3] = w4.w;
                                }
                                const uint32_t off = (ubase + u) * UB;
                                unit_sep<TY>(ta + off, tb + off, c, xf, info[(pu + u) * 4 + c], tab, acc);
                                v += kGemvWarps;
                                u += kGemvWarps;
                                while (u >= nu && v < total) { u -= nu; ti++; }
                            } while (v < total && ti == cur);
                            // each thread of the quad covered another quarter: add them up
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
                                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
                            }
                            if (c < 2) dst[g + 8 * c] += c ? acc[1] : acc[0];
                        } else {
                            float acc[2] = {0.f, 0.f};
                            do {
                                uint32_t xf[16];
                                const uint8_t *xp = xs_mine + (pu + u) * xs_ustride;
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                                    if (x_active) w4 = lds128(xp + (q >> 1) * 32 + ((q & 1) ? 16 - xq_swap : xq_swap));
                                    xf[4 * q] = w4.x; xf[4 * q + 1] = w4.y; xf[4 * q + 2] = w4.z; xf[4 * q + 3] = w4.w;
                                }
                                const uint32_t off = (ubase + u) * UB;
                                // lanes of columns that do not exist read column 0's record; their sums are dropped
                                const float *xw = reinterpret_cast<const float *>(info) + ((size_t)(pu + u) * 4 + (c < L.nc ? c : 0)) * 12;
                                unit_wide<TY>(ta + off, tb + off, c, xf, xw, tab, acc);
                                v += kGemvWarps;
                                u += kGemvWarps;
                                while (u >= nu && v < total) { u -= nu; ti++; }
                            } while (v < total && ti == cur);
                            // thread (g, c) holds the finished sums of rows g, g + 8 for column c
                            if (c < L.nc) {
                                dst[g * L.nc + c] += acc[0];
                                dst[(g + 8) * L.nc + c] += acc[1];
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(&empty[sA]);
                        if (spt == 2) mbar_arrive(&empty[sB]);
                    }
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
            const GemvSeg sg = gemv_segment(p, t0 + gb + tl);
            const uint32_t row = (t0 + gb + tl - sg.tile0) * 16 + r;
            if (row < sg.m) {
                if (G.nranks == 0) {
                    sg.out[(size_t)col * sg.m + row] = sum;
                } else {
                    const size_t at = (size_t)col * G.m_total[sg.index] + G.row_first[sg.index] + row;
                    for (uint32_t rk = 0; rk < G.nranks; rk++) G.out[sg.index][rk][at] = sum;
                }
            }
        }
        if (gb + L.group < ntl) consumer_sync();  // before the buffer is zeroed again
    }
    if (G.nranks) {
        // The stores above must be visible on every GPU before this CTA counts itself in:
        // the barrier orders them before thread 0, whose system-wide fence then covers them.
        consumer_sync();
        if (tid == 0) {
            __threadfence_system();
            for (uint32_t rk = 0; rk < G.nranks; rk++) atomicAdd_system(G.arrivals[rk], 1u);
            if (blockIdx.x == 0) {
                // one CTA stays until every CTA of every rank has counted in here: when the
                // launch is over, the whole output has arrived.  The wait is bounded.
                const uint32_t e = *G.epoch + 1;
                *G.epoch = e;
                const uint32_t target = e * G.nranks * gridDim.x;
                const long long t_start = clock64();
                for (;;) {
                    uint32_t seen;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(G.arrivals[G.rank]) : "memory");
                    if ((int32_t)(seen - target) >= 0) break;
                    if (clock64() - t_start > kWaitCycles) {
                        if (p.status) atomicExch(p.status, kStatusGatherTimeout);
                        break;
                    }
                    __nanosleep(20);
                }
            }
        }
    }
}

// Shared-memory plan.  Two CTAs share an SM (this launch's and the next one's,
// already prefetching), so each gets at most 112 KB.  (A launch with many tiles
// per CTA gains nothing from taking the SM for itself with a deeper ring: at
// that size the kernel is bound by instruction issue, not by bytes in flight.)
//
// Ring stages.  A bulk copy costs the copy engine about 50 ns however small it
// is, and a stage hand-over costs the consumers a few hundred cycles, so stages
// are large (20 - 46 KB) and filled by as few copies as possible: when whole rows
// fit, a stage is up to four tiles (or half a tile) of consecutive rows and one
// contiguous copy -- which also makes the 2-byte-aligned layouts copyable, since
// 8 rows always start on a 16-byte boundary -- otherwise rows are cut into
// segments of at least 1 KB, one copy per row.  `tiles_per_cta` is the most tiles
// any CTA of the launch gets.
constexpr uint32_t kSharedBudget = 112 * 1024;

static bool gemv_layout(int ty, uint32_t nunit, uint32_t n, bool sep, uint32_t tiles_per_cta, GemvArgs &a,
                        GemvLayout &L) {
    const uint32_t ub = ty == T_Q4_K ? 144 : ty == T_Q8_0 ? 272 : ty == T_Q2_0 ? 68 : 66;
    L.nc = sep ? 1 : n;
    L.ecols = sep ? 2 : 2 * n;
    const uint32_t budget = kSharedBudget;
    const uint32_t per_tile = kGemvWarps * 16 * L.nc * 4;
    L.group = 8192 / per_tile;
    if (L.group < 1) L.group = 1;
    if (L.group > tiles_per_cta) L.group = tiles_per_cta;
    const uint32_t red_bytes = L.group * per_tile;
    const uint32_t tab_bytes = ty == T_IQ2_XXS ? 256 * 8 : 0;
    const uint32_t stage_cap = 46 * 1024;
    const uint32_t row_bytes = nunit * ub;
    const uint32_t xunit = kXqUnit, info_unit = sep ? 64 : 4 * 48;  // per unit: 4 quarters x float4, or 4 columns x 12 words
    // Candidate plans, best first: whole tiles, half tiles, then one copy per row of
    // ever shorter segments (1, 2, ... per row).  Contiguous rows cannot be padded:
    // when the row size is a multiple of 64 bytes the rows a warp reads together
    // sit on the same banks, and per-row copies with a padded stride come first.
    const bool same_banks = row_bytes % 64 == 0;
    GemvArgs fb_a = a;
    GemvLayout fb_L = L;
    bool have_fallback = false;
    for (uint32_t plan = 0; plan < 3 + nunit; plan++) {
        uint32_t nchunk, cb, rs, stage;
        L.tps = 1;
        L.ragged = 0;
        const uint32_t kind = same_banks ? (plan == 0 ? 2 : plan <= 2 ? plan - 1 : 2) : (plan < 2 ? plan : 2);
        if (kind == 0) {
            L.mode = 0; nchunk = 1; cb = nunit; rs = row_bytes;
            // several tiles per stage while they fit and the CTA still gets two steps
            while (L.tps < 4 && (L.tps + 1) * 16 * rs <= stage_cap && (L.tps + 1) * 2 <= tiles_per_cta) L.tps++;
            stage = (L.tps * 16 * rs + 15) & ~15u;
        } else if (kind == 1) { L.mode = 1; nchunk = 1; cb = nunit; rs = row_bytes; stage = (8 * rs + 15) & ~15u; }
        else {
            L.mode = 2;
            nchunk = same_banks ? (plan == 0 ? 1 : plan - 1) : plan - 1;  // 1, 2, 3, ...
            if (same_banks && plan > 0 && nchunk == 1) continue;         // already tried
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
        const uint32_t per_chunk = L.ecols * cb * xunit + cb * info_unit;  // x and what goes with it
        const uint32_t small = kBarBytes + red_bytes + tab_bytes + 64 + L.ecols * 128;
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
        L.es = xq_col_stride(panel * cb);
        L.xs_off = kBarBytes + nstage * stage;
        L.info_off = (L.xs_off + L.ecols * L.es + 15) & ~15u;
        L.red_off = L.info_off + panel * cb * info_unit;
        L.tab_off = (L.red_off + red_bytes + 15) & ~15u;
        L.smem_bytes = L.tab_off + tab_bytes;
        if (L.smem_bytes > budget) continue;
        // A plan that keeps all of x resident stages it once per launch; one that does
        // not stages a slice per k-chunk, every time with all warps waiting.  Prefer
        // the first, as long as its row segments stay above 1 KB.
        if (panel == nchunk) return true;
        if (!have_fallback) { fb_a = a; fb_L = L; have_fallback = true; }
        if ((nunit / (nchunk + 1)) * ub < 1024) break;
    }
    if (have_fallback) { a = fb_a; L = fb_L; }
    return have_fallback;
}

template <int TY, int XDT, bool SEP>
static cudaError_t launch_t(GemvArgs a, const GemvGather &G, cudaStream_t s, int sms, int dev) {
    GemvLayout L;
    const uint32_t ctas = a.tiles < (uint32_t)sms ? a.tiles : (uint32_t)sms;
    if (!gemv_layout(TY, a.nunit, a.n, SEP, (a.tiles + ctas - 1) / ctas, a, L)) return cudaErrorInvalidConfiguration;
    static bool attr_set[64] = {};  // the opt-in is per device
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<TY, XDT, SEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSharedBudget);
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
    return cudaLaunchKernelEx(&cfg, gemv_kernel<TY, XDT, SEP>, a, L, G);
}

template <int TY>
static cudaError_t launch_ty(const GemvArgs &a, const GemvGather &G, int xdt, bool sep, cudaStream_t s, int sms, int dev) {
    if (sep) {
        switch (xdt) {
        case DT_F16: return launch_t<TY, DT_F16, true>(a, G, s, sms, dev);
        case DT_BF16: return launch_t<TY, DT_BF16, true>(a, G, s, sms, dev);
        case DT_F32: return launch_t<TY, DT_F32, true>(a, G, s, sms, dev);
        }
    } else {
        switch (xdt) {
        case DT_F16: return launch_t<TY, DT_F16, false>(a, G, s, sms, dev);
        case DT_BF16: return launch_t<TY, DT_BF16, false>(a, G, s, sms, dev);
        case DT_F32: return launch_t<TY, DT_F32, false>(a, G, s, sms, dev);
        }
    }
    return cudaErrorInvalidValue;
}

bool gemv_group_supported(int ty, uint32_t k, uint32_t nseg, const uint32_t *m, const uint8_t *const *w,
                          const void *x, int xdt, uint32_t n, int sms) {
    if (ty != T_Q4_K && ty != T_Q8_0 && ty != T_Q2_0 && ty != T_IQ2_XXS) return false;
    if (nseg == 0 || nseg > (uint32_t)kGemvSegs || n == 0 || n > 8) return false;
    if (k % 256) return false;  // Q8_0 / Q2_0 rows that end inside a 256-wide unit take the simple kernel
    if ((uintptr_t)x % 16 || (k * (xdt == DT_F32 ? 4 : 2)) % 16) return false;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < nseg; i++) {
        if (m[i] == 0 || (uintptr_t)w[i] % 16) return false;
        tiles += (m[i] + 15) / 16;
    }
    GemvArgs a = {};
    GemvLayout L;
    const uint32_t ctas = tiles < (uint32_t)sms ? tiles : (uint32_t)sms;
    const uint32_t tpc = (tiles + ctas - 1) / ctas;
    if (!gemv_layout(ty, k / 256, 1, true, tpc, a, L)) return false;
    if (n > 1 && !gemv_layout(ty, k / 256, n < 4 ? n : 4, false, tpc, a, L)) return false;
    return true;
}

bool gemv_fast_supported(int ty, uint32_t k, uint32_t m, const void *w, const void *x, int xdt, uint32_t n,
                         int sms) {
    const uint8_t *wp = (const uint8_t *)w;
    return gemv_group_supported(ty, k, 1, &m, &wp, x, xdt, n, sms);
}

// One launch covers one column (SEP) or up to four (WIDE); wider requests are cut
// into passes over consecutive columns.  `nseg` matrices of the
// same type and K share every launch.
cudaError_t launch_gemv_group(int ty, uint32_t nseg, const uint8_t *const *w, const uint32_t *m, float *const *out,
                              uint32_t k, const void *x, int xdt, uint32_t n, int *status, cudaStream_t s,
                              int sms, int dev, uint64_t *launches, const GemvGatherPlan *gather) {
    if (nseg == 0 || nseg > (uint32_t)kGemvSegs) return cudaErrorInvalidValue;
    GemvArgs a = {};
    a.status = status; a.k = k;
    a.nunit = k / 256;
    a.row_bytes = a.nunit * (ty == T_Q4_K ? 144 : ty == T_Q8_0 ? 272 : ty == T_Q2_0 ? 68 : 66);
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < (uint32_t)kGemvSegs; i++) {
        const uint32_t j = i < nseg ? i : nseg - 1;  // unused slots repeat the last one
        a.w[i] = w[j];
        a.m[i] = m[j];
        if (i < nseg) tiles += (m[i] + 15) / 16;
        a.tile_end[i] = tiles;
    }
    a.tiles = tiles;
    GemvGather G = {};
    if (gather) {
        G.nranks = gather->nranks;
        G.rank = gather->rank;
        G.epoch = gather->epoch;
        for (uint32_t r = 0; r < gather->nranks; r++) G.arrivals[r] = gather->arrivals[r];
    }
    const size_t xsz = xdt == DT_F32 ? 4 : 2;
    for (uint32_t c0 = 0; c0 < n;) {
        const uint32_t left = n - c0;
        const bool sep = left == 1;
        const uint32_t take = sep ? 1 : (left < 4 ? left : 4);
        a.x = (const uint8_t *)x + (size_t)c0 * k * xsz;
        for (uint32_t i = 0; i < (uint32_t)kGemvSegs; i++) {
            const uint32_t j = i < nseg ? i : nseg - 1;
            a.out[i] = (out && out[j]) ? out[j] + (size_t)c0 * m[j] : nullptr;
            if (gather) {
                G.m_total[i] = gather->seg[j].m_total;
                G.row_first[i] = gather->seg[j].row_first;
                for (uint32_t r = 0; r < gather->nranks; r++)
                    G.out[i][r] = gather->seg[j].out[r] + (size_t)c0 * gather->seg[j].m_total;
            }
        }
        a.n = take;
        cudaError_t e;
        switch (ty) {
        case T_Q4_K: e = launch_ty<T_Q4_K>(a, G, xdt, sep, s, sms, dev); break;
        case T_Q8_0: e = launch_ty<T_Q8_0>(a, G, xdt, sep, s, sms, dev); break;
        case T_Q2_0: e = launch_ty<T_Q2_0>(a, G, xdt, sep, s, sms, dev); break;
        case T_IQ2_XXS: e = launch_ty<T_IQ2_XXS>(a, G, xdt, sep, s, sms, dev); break;
        default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        c0 += take;
    }
    return cudaSuccess;
}

cudaError_t launch_gemv_fast(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                             uint32_t n, float *out, int *status, cudaStream_t s, int sms, int dev,
                             uint64_t *launches) {
    return launch_gemv_group(ty, 1, &w, &m, &out, k, x, xdt, n, status, s, sms, dev, launches, nullptr);
}

}  // namespace okf
