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
template <> struct UnitGeom<T_Q4_0> { static constexpr uint32_t bytes = 144; };
template <> struct UnitGeom<T_Q6_K> { static constexpr uint32_t bytes = 210; };
template <> struct UnitGeom<T_Q5_K> { static constexpr uint32_t bytes = 176; };
template <> struct UnitGeom<T_IQ4_NL> { static constexpr uint32_t bytes = 144; };
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
    uint32_t tab_copies;   // IQ2_XXS: copies of every codebook entry, side by side (a power of two)
    uint32_t smem_bytes;
};

constexpr uint32_t kBarBytes = 512;   // barriers and the abort flag, then 256 bytes of zeros at kZeroOff
constexpr uint32_t kZeroOff = 256;    // what the lanes that feed nothing into an MMA read instead of x
constexpr uint32_t kMaxStages = 8;
constexpr uint32_t kConsumers = kGemvWarps * 32;
// WIDE x panel: a unit of a byte column is its 256 bytes in k order, except that in
// quarters 2 and 3 neighbouring 16-byte pieces are swapped; with the second byte column
// 32 (mod 128) bytes after the first, the lanes of a load that carry data touch different
// bank groups.
constexpr uint32_t kXqUnit = 256;
constexpr float kXqMax = 32512.f;  // 127 * 256: hi stays a signed byte after rounding
// SEP x panel: per byte column and unit, four quarters of 80 bytes: 64 bytes of x in k
// order, then (first byte column only) the quarter's record {scale, scale * sum of x over
// its first 32-wide block, over its second, -}.  One address register reaches a
// quarter's x and its record with immediate offsets.  80-byte quarters put the four
// quarters of a 16-byte access on different bank groups (0, 80, 32, 112 mod 128) and the
// second byte column, 64 (mod 128) bytes after the first, on the other four.
constexpr uint32_t kSepQuarter = 80, kSepUnit = 4 * kSepQuarter;

__host__ __device__ inline uint32_t xq_col_stride(uint32_t units) {
    const uint32_t raw = units * kXqUnit;
    return raw + ((32u + 128u - raw % 128u) % 128u);
}
__host__ __device__ inline uint32_t sep_col_stride(uint32_t units) {
    const uint32_t raw = units * kSepUnit;
    return raw + ((64u + 128u - raw % 128u) % 128u);
}
__host__ __device__ inline uint32_t xq_piece_offset(uint32_t c, uint32_t piece) {
    return c * 64 + ((piece ^ (c >> 1)) & 3u) * 16;
}

__device__ __forceinline__ uint4 lds128(const uint8_t *p) { return *reinterpret_cast<const uint4 *>(p); }

// Shared-memory loads by 32-bit shared-window address: the one-column path does
// all its address arithmetic in 32 bits.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// 4 * NW bytes from a 2-byte aligned shared address: aligned words and a funnel shift
template <int NW>
__device__ __forceinline__ void lds_a2(uint32_t a, uint32_t (&out)[NW]) {
    const uint32_t base = a & ~3u, sh = (a & 2u) * 8u;
    uint32_t w[NW + 1];
#pragma unroll
    for (int i = 0; i <= NW; i++) w[i] = lds32(base + 4 * i);
#pragma unroll
    for (int i = 0; i < NW; i++) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
}
__device__ __forceinline__ uint2 lds64(const uint8_t *p) { return *reinterpret_cast<const uint2 *>(p); }
__device__ __forceinline__ int ubyte(uint32_t v, int i) { return (int)__byte_perm(v, 0, 0x4440 + i); }
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t x) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(x) : "memory");
}
__device__ __forceinline__ void sts16(uint32_t a, uint32_t x) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "r"(x) : "memory");
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t v;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(a), "r"(b), "r"(sel));
    return v;
}

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
// What a thread works out once per launch for the one-column path.
struct SepConst {
    uint32_t qoff;          // where this thread's share of a unit starts (bytes from the unit's start)
    uint32_t hoff;          // Q2_0: where the block that share lies in starts
    uint32_t sel, m1, m2;   // Q4_K: how to pick this thread's 6-bit scales and mins out of the 12 bytes
    bool low;               // Q4_K: sub-blocks 0..3 (plain 6-bit fields) or 4..7 (split fields)
    uint32_t tab_lane;      // IQ2_XXS: shared address of this lane's copy of codebook entry 0
    uint32_t tab_stride;    // IQ2_XXS: bytes between table entries (copies of one entry lie side by side)
};
template <int TY>
__device__ __forceinline__ SepConst sep_const(uint32_t c, uint32_t lane, uint32_t tab, uint32_t tab_copies) {
    SepConst k = {};
    if constexpr (TY == T_Q4_K || TY == T_Q5_K) {
        k.qoff = (TY == T_Q4_K ? 16 : 48) + 32 * c;
        k.hoff = 2 * c;  // Q5_K: the bit of qh that belongs to sub-block 2c
        k.sel = (c & 1) ? 0x7632u : 0x5410u;
        k.low = c < 2;
        k.m1 = k.low ? 0x3F3F3F3Fu : 0x0F0F0F0Fu;
        k.m2 = k.low ? 0u : 0x30303030u;
    } else if constexpr (TY == T_Q8_0) {
        k.qoff = 68 * c;
    } else if constexpr (TY == T_Q4_0 || TY == T_IQ4_NL) {
        k.qoff = 36 * c;
    } else if constexpr (TY == T_Q6_K) {
        k.qoff = 64 * (c >> 1);         // ql of this half of the block
        k.hoff = 128 + 32 * (c >> 1);   // qh of this half
        k.sel = 4 * (c & 1);            // low or high nibbles of ql; bits 0-3 or 4-7 of qh
        k.m1 = 192 + 4 * c;             // this quarter's four scales
    } else if constexpr (TY == T_Q2_0) {
        k.hoff = 34 * (c >> 1);
        k.qoff = k.hoff + 2 + 16 * (c & 1);
    } else {
        k.qoff = 2 + 16 * c;
        k.tab_lane = tab + (lane & (tab_copies - 1)) * 8;
        k.tab_stride = tab_copies * 8;
    }
    return k;
}

// IQ2_XXS: byte masks (0xFF = negative) of the eight weights a 7-bit sign index stands
// for; the eighth sign is the parity of the seven (LLM/Quantize/IQ2Grid.swift:73-85).
// One multiply puts sign bit j on the top bit of byte j (the shifted copies of a 7-bit
// number do not overlap, so nothing carries), and a byte permute in its
// sign-replicating mode fills each byte with its top bit.
__device__ __forceinline__ void iq2_sign_bytes(uint32_t idx7, uint32_t &lo, uint32_t &hi) {
    const uint32_t par = (uint32_t)__popc(idx7) << 31;
    lo = prmt(idx7 * 0x10204080u, 0u, 0xBA98u);        // signs 0..3: shifts 7, 14, 21, 28
    hi = prmt(idx7 * 0x00020408u + par, 0u, 0xBA98u);  // signs 4..6: shifts 3, 10, 17; parity on bit 31
}

// IQ4_NL: the sixteen codebook values (LLM/Gemma/Gemma4Quant.swift:5-9) for four nibbles (one per
// byte of v, 0..15) as four signed bytes.
__device__ __forceinline__ uint32_t iq4nl_lookup(uint32_t v) {
    // {-127, -104, -83, -65}, {-49, -35, -22, -10}, {1, 13, 25, 38}, {53, 69, 89, 113}
    constexpr uint32_t T0 = 0xBFAD9881u, T1 = 0xF6EADDCFu, T2 = 0x26190D01u, T3 = 0x71594535u;
    const uint32_t s = v & 0x07070707u;
    const uint32_t t = s | (s >> 4);                       // bytes 0 and 2: two selector nibbles each
    const uint32_t sel = (t & 0xFFu) | ((t >> 8) & 0xFF00u);
    const uint32_t lo = prmt(T0, T1, sel), hi = prmt(T2, T3, sel);
    const uint32_t pick = ((v >> 3) & 0x01010101u) * 0xFFu;  // bytes whose nibble is 8..15
    return (lo & ~pick) | (hi & pick);
}

// ua / ub: shared addresses of the unit in rows g and g + 8.  xf: this thread's 64
// bytes of x (its quarter of the unit, the byte column its MMA column stands for; zeros
// in the lanes that feed nothing).  xi: {scale of x in this unit, scale * sum of x over
// the first 32-wide block of the quarter, over the second, -} as float bits.
// acc: rows g and g + 8.
template <int TY>
__device__ __forceinline__ void unit_sep(uint32_t ua, uint32_t ub, const SepConst &K, const uint32_t (&xf)[16],
                                         const uint4 &xi, float (&acc)[2]) {
    const float xs = __uint_as_float(xi.x);
    if constexpr (TY == T_Q4_K) {
        // {f16 d; f16 dmin; u8 scales[12]; u8 qs[128]} (LLM/Quantize/KQuants.swift:104-125).
        // Group c of qs (32 bytes): low nibbles = sub-block 2c, high = 2c+1, both in k order.
        // The high nibbles stay where they are (16 x the value); the sums are shifted back.
        const uint4 ha = lds128(ua), hb = lds128(ub);
        const uint4 a0 = lds128(ua + K.qoff), a1 = lds128(ua + K.qoff + 16);
        const uint4 b0 = lds128(ub + K.qoff), b1 = lds128(ub + K.qoff + 16);
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
        // 6-bit (scale, min) of sub-blocks 2c and 2c+1 of both rows (ggml get_scale_min_k4,
        // LLM/Quantize/KQuants.swift:86-101) as bytes {row a: 2c, 2c+1, row b: 2c, 2c+1},
        // without a branch: the two cases differ in where the low bits come from.
        const uint32_t pa = prmt(ha.y, hb.y, K.sel), pb = prmt(ha.z, hb.z, K.sel), pe = prmt(ha.w, hb.w, K.sel);
        const uint32_t sc = ((K.low ? pa : pe) & K.m1) | ((pa >> 2) & K.m2);
        const uint32_t mn = ((K.low ? pb : (pe >> 4)) & K.m1) | ((pb >> 2) & K.m2);
        // From here on floating point: integer instructions run at half the rate of fp32 ones
        // on this part, and the masks above have used up the integer budget.  A scale byte
        // becomes a float with one byte permute and one subtraction.  The high-nibble sums
        // carry a factor 16 that goes into x's scale.
        const float xs16 = xs * 0.0625f;
        const float la = join_hi_lo(lo[0], lo[1]), ha_ = join_hi_lo(hi[0], hi[1]);
        const float lb = join_hi_lo(lo[2], lo[3]), hb_ = join_hi_lo(hi[2], hi[3]);
        const float x0 = __uint_as_float(xi.y), x1 = __uint_as_float(xi.z);  // scale * sum of x per block
        const float2 fa = __half22float2(*reinterpret_cast<const __half2 *>(&ha.x));
        const float2 fb = __half22float2(*reinterpret_cast<const __half2 *>(&hb.x));
        acc[0] += fa.x * (byte_to_f32(sc, 0) * (xs * la) + byte_to_f32(sc, 1) * (xs16 * ha_)) -
                  fa.y * (byte_to_f32(mn, 0) * x0 + byte_to_f32(mn, 1) * x1);
        acc[1] += fb.x * (byte_to_f32(sc, 2) * (xs * lb) + byte_to_f32(sc, 3) * (xs16 * hb_)) -
                  fb.y * (byte_to_f32(mn, 2) * x0 + byte_to_f32(mn, 3) * x1);
    } else if constexpr (TY == T_Q4_0) {
        // eight blocks {f16 d; u8 qs[16]}, byte j = weights j (low nibble) and j + 16 (high), value
        // (q - 8) * d (LLM/Gemma/Gemma4Quant.swift:30-49).  Thread c takes blocks 2c and 2c+1:
        // {d0, qs0[16], d1, qs1[16]} = 9 words (units start on 16-byte boundaries, 36c is a
        // multiple of 4).  Nibbles are masked in place; the high ones stay 16 x the value.
        uint32_t wa[9], wb[9];
#pragma unroll
        for (int i = 0; i < 9; i++) {
            wa[i] = lds32(ua + K.qoff + 4 * i);
            wb[i] = lds32(ub + K.qoff + 4 * i);
        }
        uint32_t qa[8], qb[8];  // block 0's bytes start two bytes into word 0, block 1's on word 5
#pragma unroll
        for (int i = 0; i < 4; i++) {
            qa[i] = __funnelshift_r(wa[i], wa[i + 1], 16);
            qb[i] = __funnelshift_r(wb[i], wb[i + 1], 16);
            qa[4 + i] = wa[5 + i];
            qb[4 + i] = wb[5 + i];
        }
        const uint32_t ml = 0x0F0F0F0Fu, mh = 0xF0F0F0F0u;
        float part[2][2];  // [block][row]: sum of q * x in units of x's scale
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
            const uint32_t *a = qa + 4 * blk, *b = qb + 4 * blk;
            const uint32_t *xb = xf + 8 * blk;  // bytes of k 0..15 (low nibbles), then 16..31 (high)
            int lo[4], hi[4];
            imma0<false>(lo, a[0] & ml, b[0] & ml, a[1] & ml, b[1] & ml, xb[0], xb[1]);
            imma0<false>(hi, a[0] & mh, b[0] & mh, a[1] & mh, b[1] & mh, xb[4], xb[5]);
            imma<false>(lo, a[2] & ml, b[2] & ml, a[3] & ml, b[3] & ml, xb[2], xb[3]);
            imma<false>(hi, a[2] & mh, b[2] & mh, a[3] & mh, b[3] & mh, xb[6], xb[7]);
            part[blk][0] = fmaf(join_hi_lo(hi[0], hi[1]), 0.0625f, join_hi_lo(lo[0], lo[1]));
            part[blk][1] = fmaf(join_hi_lo(hi[2], hi[3]), 0.0625f, join_hi_lo(lo[2], lo[3]));
        }
        const float x0 = __uint_as_float(xi.y), x1 = __uint_as_float(xi.z);  // scale * sum of x per block
        const float da0 = f16bits(wa[0] & 0xFFFF), da1 = f16bits(wa[4] >> 16);
        const float db0 = f16bits(wb[0] & 0xFFFF), db1 = f16bits(wb[4] >> 16);
        acc[0] += da0 * fmaf(xs, part[0][0], -8.f * x0) + da1 * fmaf(xs, part[1][0], -8.f * x1);
        acc[1] += db0 * fmaf(xs, part[0][1], -8.f * x0) + db1 * fmaf(xs, part[1][1], -8.f * x1);
    } else if constexpr (TY == T_IQ4_NL) {
        // Q4_0's layout with a codebook: weight = kvalues[nibble] * d (LLM/Gemma/Gemma4Quant.swift:5-29).
        // The sixteen signed bytes sit in four registers; a byte permute looks four nibbles up in
        // the low or the high eight, bit 3 of each nibble picks between the two.
        uint32_t wa[9], wb[9];
#pragma unroll
        for (int i = 0; i < 9; i++) {
            wa[i] = lds32(ua + K.qoff + 4 * i);
            wb[i] = lds32(ub + K.qoff + 4 * i);
        }
        uint32_t qa[8], qb[8];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            qa[i] = __funnelshift_r(wa[i], wa[i + 1], 16);
            qb[i] = __funnelshift_r(wb[i], wb[i + 1], 16);
            qa[4 + i] = wa[5 + i];
            qb[4 + i] = wb[5 + i];
        }
        float part[2][2];
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
            const uint32_t *a = qa + 4 * blk, *b = qb + 4 * blk;
            const uint32_t *xb = xf + 8 * blk;  // bytes of k 0..15 (low nibbles), then 16..31 (high)
            int d[4];
            imma0<true>(d, iq4nl_lookup(a[0] & 0x0F0F0F0Fu), iq4nl_lookup(b[0] & 0x0F0F0F0Fu), iq4nl_lookup(a[1] & 0x0F0F0F0Fu),
                        iq4nl_lookup(b[1] & 0x0F0F0F0Fu), xb[0], xb[1]);
            imma<true>(d, iq4nl_lookup(a[2] & 0x0F0F0F0Fu), iq4nl_lookup(b[2] & 0x0F0F0F0Fu), iq4nl_lookup(a[3] & 0x0F0F0F0Fu),
                       iq4nl_lookup(b[3] & 0x0F0F0F0Fu), xb[2], xb[3]);
            imma<true>(d, iq4nl_lookup((a[0] >> 4) & 0x0F0F0F0Fu), iq4nl_lookup((b[0] >> 4) & 0x0F0F0F0Fu),
                       iq4nl_lookup((a[1] >> 4) & 0x0F0F0F0Fu), iq4nl_lookup((b[1] >> 4) & 0x0F0F0F0Fu), xb[4], xb[5]);
            imma<true>(d, iq4nl_lookup((a[2] >> 4) & 0x0F0F0F0Fu), iq4nl_lookup((b[2] >> 4) & 0x0F0F0F0Fu),
                       iq4nl_lookup((a[3] >> 4) & 0x0F0F0F0Fu), iq4nl_lookup((b[3] >> 4) & 0x0F0F0F0Fu), xb[6], xb[7]);
            part[blk][0] = join_hi_lo(d[0], d[1]);
            part[blk][1] = join_hi_lo(d[2], d[3]);
        }
        const float da0 = f16bits(wa[0] & 0xFFFF), da1 = f16bits(wa[4] >> 16);
        const float db0 = f16bits(wb[0] & 0xFFFF), db1 = f16bits(wb[4] >> 16);
        acc[0] += xs * (da0 * part[0][0] + da1 * part[1][0]);
        acc[1] += xs * (db0 * part[0][1] + db1 * part[1][1]);
    } else if constexpr (TY == T_Q5_K) {
        // {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} (LLM/Quantize/KQuants.swift:127-158):
        // Q4_K's header and nibbles, plus a fifth bit: bit j of qh[l] for sub-block j.  The five
        // bits are joined into unsigned bytes (0..31) for both sub-blocks of the quarter.
        const uint4 ha = lds128(ua), hb = lds128(ub);
        int lo[4], hi[4];
#pragma unroll
        for (int half = 0; half < 2; half++) {  // 16 bytes of qs and of qh at a time
            const uint4 a = lds128(ua + K.qoff + 16 * half), b = lds128(ub + K.qoff + 16 * half);
            const uint4 ga = lds128(ua + 16 + 16 * half), gb = lds128(ub + 16 + 16 * half);
            const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
            const uint32_t fa[4] = {ga.x >> K.hoff, ga.y >> K.hoff, ga.z >> K.hoff, ga.w >> K.hoff};
            const uint32_t fb[4] = {gb.x >> K.hoff, gb.y >> K.hoff, gb.z >> K.hoff, gb.w >> K.hoff};
            uint32_t la[4], lb[4], ua5[4], ub5[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                la[i] = (wa[i] & 0x0F0F0F0Fu) | ((fa[i] & 0x01010101u) << 4);
                lb[i] = (wb[i] & 0x0F0F0F0Fu) | ((fb[i] & 0x01010101u) << 4);
                ua5[i] = ((wa[i] >> 4) & 0x0F0F0F0Fu) | ((fa[i] & 0x02020202u) << 3);
                ub5[i] = ((wb[i] >> 4) & 0x0F0F0F0Fu) | ((fb[i] & 0x02020202u) << 3);
            }
            if (half == 0) {
                imma0<false>(lo, la[0], lb[0], la[1], lb[1], xf[0], xf[1]);
                imma0<false>(hi, ua5[0], ub5[0], ua5[1], ub5[1], xf[8], xf[9]);
                imma<false>(lo, la[2], lb[2], la[3], lb[3], xf[2], xf[3]);
                imma<false>(hi, ua5[2], ub5[2], ua5[3], ub5[3], xf[10], xf[11]);
            } else {
                imma<false>(lo, la[0], lb[0], la[1], lb[1], xf[4], xf[5]);
                imma<false>(hi, ua5[0], ub5[0], ua5[1], ub5[1], xf[12], xf[13]);
                imma<false>(lo, la[2], lb[2], la[3], lb[3], xf[6], xf[7]);
                imma<false>(hi, ua5[2], ub5[2], ua5[3], ub5[3], xf[14], xf[15]);
            }
        }
        const uint32_t pa = prmt(ha.y, hb.y, K.sel), pb = prmt(ha.z, hb.z, K.sel), pe = prmt(ha.w, hb.w, K.sel);
        const uint32_t sc = ((K.low ? pa : pe) & K.m1) | ((pa >> 2) & K.m2);
        const uint32_t mn = ((K.low ? pb : (pe >> 4)) & K.m1) | ((pb >> 2) & K.m2);
        const float la_ = join_hi_lo(lo[0], lo[1]), ha_ = join_hi_lo(hi[0], hi[1]);
        const float lb_ = join_hi_lo(lo[2], lo[3]), hb_ = join_hi_lo(hi[2], hi[3]);
        const float x0 = __uint_as_float(xi.y), x1 = __uint_as_float(xi.z);  // scale * sum of x per block
        const float2 fa2 = __half22float2(*reinterpret_cast<const __half2 *>(&ha.x));
        const float2 fb2 = __half22float2(*reinterpret_cast<const __half2 *>(&hb.x));
        acc[0] += fa2.x * xs * (byte_to_f32(sc, 0) * la_ + byte_to_f32(sc, 1) * ha_) -
                  fa2.y * (byte_to_f32(mn, 0) * x0 + byte_to_f32(mn, 1) * x1);
        acc[1] += fb2.x * xs * (byte_to_f32(sc, 2) * lb_ + byte_to_f32(sc, 3) * hb_) -
                  fb2.y * (byte_to_f32(mn, 2) * x0 + byte_to_f32(mn, 3) * x1);
    } else if constexpr (TY == T_Q6_K) {
        // {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d} (LLM/Quantize/KQuants.swift:160-177): weight =
        // d * scale[group of 16] * (q - 32), q = four bits of ql and two of qh.  Quarter c is
        // elements 64c .. 64c + 63 = the low (c even) or high (c odd) nibbles of the 64 ql bytes of
        // half c / 2, with qh bits 4(c & 1) .. +1 for its first 32 elements and the next two bits
        // for the other 32, and scales 4c .. 4c + 3.  q - 32 is made a signed byte in place
        // (flip bit 5, then copy it into bits 6 and 7: 0x20 * 6 = 0xC0 stays inside the byte), so
        // the signed MMA needs no correction; one accumulator per 16-wide scale group.
        // Units are only 2-byte aligned.
        uint32_t sa[1], sb[1];
        lds_a2<1>(ua + K.m1, sa);
        lds_a2<1>(ub + K.m1, sb);
        const float da = f16bits(lds16(ua + 208)), db = f16bits(lds16(ub + 208));
        const uint32_t sh = K.sel;
        float suma = 0.f, sumb = 0.f;
#pragma unroll
        for (int grp = 0; grp < 4; grp++) {  // 16 elements: 16 bytes of ql, 16 of qh (groups 2, 3 reuse those of 0, 1)
            uint32_t la[4], lb[4], ha[4], hb[4];
            lds_a2<4>(ua + K.qoff + 16 * grp, la);
            lds_a2<4>(ub + K.qoff + 16 * grp, lb);
            lds_a2<4>(ua + K.hoff + 16 * (grp & 1), ha);
            lds_a2<4>(ub + K.hoff + 16 * (grp & 1), hb);
            const uint32_t hs = sh + 2 * (grp >> 1);
            uint32_t qa[4], qb[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t va = (((la[i] >> sh) & 0x0F0F0F0Fu) | (((ha[i] >> hs) & 0x03030303u) << 4)) ^ 0x20202020u;
                const uint32_t vb = (((lb[i] >> sh) & 0x0F0F0F0Fu) | (((hb[i] >> hs) & 0x03030303u) << 4)) ^ 0x20202020u;
                qa[i] = va | ((va & 0x20202020u) * 6u);
                qb[i] = vb | ((vb & 0x20202020u) * 6u);
            }
            int d[4];
            imma0<true>(d, qa[0], qb[0], qa[1], qb[1], xf[4 * grp], xf[4 * grp + 1]);
            imma<true>(d, qa[2], qb[2], qa[3], qb[3], xf[4 * grp + 2], xf[4 * grp + 3]);
            const float fa = (float)((int)(sa[0] << (24 - 8 * grp)) >> 24), fb = (float)((int)(sb[0] << (24 - 8 * grp)) >> 24);
            suma = fmaf(fa, join_hi_lo(d[0], d[1]), suma);
            sumb = fmaf(fb, join_hi_lo(d[2], d[3]), sumb);
        }
        acc[0] += (da * xs) * suma;
        acc[1] += (db * xs) * sumb;
    } else if constexpr (TY == T_Q8_0) {
        // eight blocks {f16 d; i8 q[32]} (LLM/Gemma/Gemma4Quant.swift:51-69); thread c
        // takes blocks 2c and 2c+1: {d0, q0[32], d1, q1[32]} = 17 words (units start on
        // 16-byte boundaries, 68c is a multiple of 4); the quants go into the MMA as they are.
        uint32_t wa[17], wb[17];
#pragma unroll
        for (int i = 0; i < 17; i++) {
            wa[i] = lds32(ua + K.qoff + 4 * i);
            wb[i] = lds32(ub + K.qoff + 4 * i);
        }
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
        acc[0] += xs * (da0 * join_hi_lo(lo[0], lo[1]) + da1 * join_hi_lo(hi[0], hi[1]));
        acc[1] += xs * (db0 * join_hi_lo(lo[2], lo[3]) + db1 * join_hi_lo(hi[2], hi[3]));
    } else if constexpr (TY == T_Q2_0) {
        // two blocks {f16 d; u8 qs[32]} of 128 ternary codes, weight = (code - 1) * d
        // (LLM/Base/Quant.swift:2-25).  Thread c takes half (c & 1) of block c >> 1:
        // 16 bytes = 64 codes; byte t holds k 4t .. 4t+3.  Masking code s of every
        // byte of a word in place gives 4^s times the codes of k = s, 4+s, 8+s, 12+s
        // (x is staged in that order); the factors are undone on the integer sums.
        uint32_t wa[4], wb[4];
        lds_a2<4>(ua + K.qoff, wa);
        lds_a2<4>(ub + K.qoff, wb);
        const float da = f16bits(lds16(ua + K.hoff)), db = f16bits(lds16(ub + K.hoff));
        int t[4] = {0, 0, 0, 0};  // both 32-wide halves together, times 64
#pragma unroll
        for (int sub = 0; sub < 2; sub++) {
#pragma unroll
            for (int s = 0; s < 4; s++) {
                const uint32_t m = 0x03030303u << (2 * s);
                int d[4];
                imma0<false>(d, wa[2 * sub] & m, wb[2 * sub] & m, wa[2 * sub + 1] & m, wb[2 * sub + 1] & m,
                             xf[8 * sub + s], xf[8 * sub + 4 + s]);
#pragma unroll
                for (int e = 0; e < 4; e++) t[e] = t[e] + d[e] * (64 >> (2 * s));
            }
        }
        const float xsum = __uint_as_float(xi.y) + __uint_as_float(xi.z);  // scale * sum of x over the quarter
        acc[0] += da * (xs * 0.015625f * join_hi_lo(t[0], t[1]) - xsum);
        acc[1] += db * (xs * 0.015625f * join_hi_lo(t[2], t[3]) - xsum);
    } else {
        // IQ2_XXS {f16 d; 8 x (u32 a0: four codebook indices, u32 a1: four 7-bit sign
        // indices + 4-bit scale)} (LLM/Quantize/IQ2XXS.swift:34-53).  Thread c takes
        // sub-blocks 2c and 2c+1.  A codebook entry is eight magnitude bytes = the two
        // A registers of one row; the byte masks of a sign index (0xFF = negative) are
        // computed (a table of them, tried, gained 2 % at K = 5120 and cost 8 % at K = 17408,
        // where it crowds the ring out of shared memory).  Signs: XOR with the mask turns a
        // magnitude m into the signed byte -(m + 1); a second MMA on the masks themselves
        // (255 per negative weight) gives 255 x the sum of x over the negative weights, which
        // puts the missing 1 back: sum(sign * m * x) = D1 + D2 / 255.
        uint32_t wa[4], wb[4];
        lds_a2<4>(ua + K.qoff, wa);
        lds_a2<4>(ub + K.qoff, wb);
        const float da = f16bits(lds16(ua)), db = f16bits(lds16(ub));
        float sum[2][2];
#pragma unroll
        for (int sb = 0; sb < 2; sb++) {
            const uint32_t a0a = wa[2 * sb], a1a = wa[2 * sb + 1], a0b = wb[2 * sb], a1b = wb[2 * sb + 1];
            int d1[4], d2[4];
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint2 ea = lds64(K.tab_lane + prmt(a0a, 0u, 0x4440u + l) * K.tab_stride);
                const uint2 eb = lds64(K.tab_lane + prmt(a0b, 0u, 0x4440u + l) * K.tab_stride);
                uint2 ma, mb;
                iq2_sign_bytes((a1a >> (7 * l)) & 127u, ma.x, ma.y);
                iq2_sign_bytes((a1b >> (7 * l)) & 127u, mb.x, mb.y);
                const uint32_t x0 = xf[8 * sb + 2 * l], x1 = xf[8 * sb + 2 * l + 1];
                if (l == 0) {
                    imma0<true>(d1, ea.x ^ ma.x, eb.x ^ mb.x, ea.y ^ ma.y, eb.y ^ mb.y, x0, x1);
                    imma0<false>(d2, ma.x, mb.x, ma.y, mb.y, x0, x1);
                } else {
                    imma<true>(d1, ea.x ^ ma.x, eb.x ^ mb.x, ea.y ^ ma.y, eb.y ^ mb.y, x0, x1);
                    imma<false>(d2, ma.x, mb.x, ma.y, mb.y, x0, x1);
                }
            }
            sum[sb][0] = fmaf(join_hi_lo(d2[0], d2[1]), 1.f / 255.f, join_hi_lo(d1[0], d1[1]));
            sum[sb][1] = fmaf(join_hi_lo(d2[2], d2[3]), 1.f / 255.f, join_hi_lo(d1[2], d1[3]));
        }
        const float sa0 = 0.5f + (float)(wa[1] >> 28), sa1 = 0.5f + (float)(wa[3] >> 28);
        const float sb0 = 0.5f + (float)(wb[1] >> 28), sb1 = 0.5f + (float)(wb[3] >> 28);
        acc[0] += (0.25f * xs * da) * (sa0 * sum[0][0] + sa1 * sum[1][0]);
        acc[1] += (0.25f * xs * db) * (sb0 * sum[0][1] + sb1 * sum[1][1]);
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

template <int TY>
__device__ __forceinline__ void unit_wide(const uint8_t *ua, const uint8_t *ub, uint32_t c, const uint32_t (&xf)[16],
                                          const float *xw, const uint2 *tab, uint32_t tab_copies, float (&acc)[2]) {
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
    } else if constexpr (TY == T_Q5_K) {
        // Q4_K's layout with qh[32] after the header and a fifth bit per weight: bit j of qh[l]
        // for sub-block j (LLM/Quantize/KQuants.swift:127-158); this thread's l are 8c .. 8c + 7
        const uint2 ga = lds64(ua + 16 + 8 * c), gb = lds64(ub + 16 + 8 * c);
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
        const uint32_t ml = 0x0F0F0F0Fu;
        int te[4] = {0, 0, 0, 0}, to[4] = {0, 0, 0, 0};  // sum of scale * block sum: low-nibble / high-nibble blocks
        int mina = 0, minb = 0;
#pragma unroll
        for (int p = 0; p < 4; p++) {  // 32 bytes of nibbles: block 2p in the low ones, 2p+1 in the high ones
            const uint2 wa = lds64(ua + 48 + 32 * p + 8 * c), wb = lds64(ub + 48 + 32 * p + 8 * c);
            const uint32_t b1 = 0x01010101u;
            const uint32_t la0 = (wa.x & ml) | (((ga.x >> (2 * p)) & b1) << 4), la1 = (wa.y & ml) | (((ga.y >> (2 * p)) & b1) << 4);
            const uint32_t lb0 = (wb.x & ml) | (((gb.x >> (2 * p)) & b1) << 4), lb1 = (wb.y & ml) | (((gb.y >> (2 * p)) & b1) << 4);
            const uint32_t ha0 = ((wa.x >> 4) & ml) | (((ga.x >> (2 * p + 1)) & b1) << 4), ha1 = ((wa.y >> 4) & ml) | (((ga.y >> (2 * p + 1)) & b1) << 4);
            const uint32_t hb0 = ((wb.x >> 4) & ml) | (((gb.x >> (2 * p + 1)) & b1) << 4), hb1 = ((wb.y >> 4) & ml) | (((gb.y >> (2 * p + 1)) & b1) << 4);
            const int sa0 = ubyte(p < 2 ? sa03 : sa47, (2 * p) & 3), sa1 = ubyte(p < 2 ? sa03 : sa47, (2 * p + 1) & 3);
            const int sb0 = ubyte(p < 2 ? sb03 : sb47, (2 * p) & 3), sb1 = ubyte(p < 2 ? sb03 : sb47, (2 * p + 1) & 3);
            int d[4];
            imma0<false>(d, la0, lb0, la1, lb1, xf[4 * p], xf[4 * p + 1]);
            te[0] += sa0 * d[0]; te[1] += sa0 * d[1]; te[2] += sb0 * d[2]; te[3] += sb0 * d[3];
            imma0<false>(d, ha0, hb0, ha1, hb1, xf[4 * p + 2], xf[4 * p + 3]);
            to[0] += sa1 * d[0]; to[1] += sa1 * d[1]; to[2] += sb1 * d[2]; to[3] += sb1 * d[3];
            mina += ubyte(p < 2 ? ma03 : ma47, (2 * p) & 3) * xb[2 * p] + ubyte(p < 2 ? ma03 : ma47, (2 * p + 1) & 3) * xb[2 * p + 1];
            minb += ubyte(p < 2 ? mb03 : mb47, (2 * p) & 3) * xb[2 * p] + ubyte(p < 2 ? mb03 : mb47, (2 * p + 1) & 3) * xb[2 * p + 1];
        }
        const float da = f16bits(ha.x & 0xFFFF), dma = f16bits(ha.x >> 16);
        const float db = f16bits(hb.x & 0xFFFF), dmb = f16bits(hb.x >> 16);
        // The scaled sums no longer fit 256 * hi + lo in 32 bits: join them in fp32.
        auto join = [](int hi, int lo) { return fmaf((float)hi, 256.f, (float)lo); };
        acc[0] += xs * (da * (join(te[0], te[1]) + join(to[0], to[1])) - dma * (float)mina);
        acc[1] += xs * (db * (join(te[2], te[3]) + join(to[2], to[3])) - dmb * (float)minb);
    } else if constexpr (TY == T_IQ4_NL) {
        float fa = 0.f, fb = 0.f;
        const uint32_t sh = 4 * (c >> 1);  // threads 0, 1: low nibbles (k 0..15); 2, 3: high (k 16..31)
#pragma unroll
        for (int b = 0; b < 8; b++) {  // block b: {f16 d; u8 qs[16]}, this thread's eight bytes at 2 + 8 (c & 1)
            uint32_t qa[2], qb[2];
            lds_a2<2>(ua + 18 * b + 2 + 8 * (c & 1), qa);
            lds_a2<2>(ub + 18 * b + 2 + 8 * (c & 1), qb);
            int d[4];
            imma0<true>(d, iq4nl_lookup((qa[0] >> sh) & 0x0F0F0F0Fu), iq4nl_lookup((qb[0] >> sh) & 0x0F0F0F0Fu),
                        iq4nl_lookup((qa[1] >> sh) & 0x0F0F0F0Fu), iq4nl_lookup((qb[1] >> sh) & 0x0F0F0F0Fu), xf[2 * b], xf[2 * b + 1]);
            fa += f16bits(ld_u16(ua + 18 * b)) * join_hi_lo(d[0], d[1]);
            fb += f16bits(ld_u16(ub + 18 * b)) * join_hi_lo(d[2], d[3]);
        }
        acc[0] += xs * fa;
        acc[1] += xs * fb;
    } else if constexpr (TY == T_Q6_K) {
        // Block b = half n = b / 4 of the unit, granule r = b % 4 (see the one-column path).  This
        // thread's eight weights l = 8c .. 8c + 7 share one of the block's two 16-wide scales,
        // threads 0, 1 the first and 2, 3 the second: two MMAs per block, each fed by the two
        // threads of one scale (the others pass zeros), so that each sum meets its own scale.
        float fa = 0.f, fb = 0.f;
        const bool first = c < 2;
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const int n = b >> 2, r = b & 3;
            uint32_t la[2], lb[2], ha[2], hb[2];
            lds_a2<2>(ua + 64 * n + 32 * (r & 1) + 8 * c, la);
            lds_a2<2>(ub + 64 * n + 32 * (r & 1) + 8 * c, lb);
            lds_a2<2>(ua + 128 + 32 * n + 8 * c, ha);
            lds_a2<2>(ub + 128 + 32 * n + 8 * c, hb);
            uint32_t qa[2], qb[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint32_t va = (((la[i] >> (r >= 2 ? 4 : 0)) & 0x0F0F0F0Fu) | (((ha[i] >> (2 * r)) & 0x03030303u) << 4)) ^ 0x20202020u;
                const uint32_t vb = (((lb[i] >> (r >= 2 ? 4 : 0)) & 0x0F0F0F0Fu) | (((hb[i] >> (2 * r)) & 0x03030303u) << 4)) ^ 0x20202020u;
                qa[i] = va | ((va & 0x20202020u) * 6u);  // q - 32 as a signed byte
                qb[i] = vb | ((vb & 0x20202020u) * 6u);
            }
            const uint32_t sca = ld_u16(ua + 192 + 8 * n + 2 * r), scb = ld_u16(ub + 192 + 8 * n + 2 * r);
            int d0[4], d1[4];
            imma0<true>(d0, first ? qa[0] : 0u, first ? qb[0] : 0u, first ? qa[1] : 0u, first ? qb[1] : 0u, xf[2 * b], xf[2 * b + 1]);
            imma0<true>(d1, first ? 0u : qa[0], first ? 0u : qb[0], first ? 0u : qa[1], first ? 0u : qb[1], xf[2 * b], xf[2 * b + 1]);
            fa += (float)(int)(int8_t)(sca & 0xFF) * join_hi_lo(d0[0], d0[1]) + (float)(int)(int8_t)(sca >> 8) * join_hi_lo(d1[0], d1[1]);
            fb += (float)(int)(int8_t)(scb & 0xFF) * join_hi_lo(d0[2], d0[3]) + (float)(int)(int8_t)(scb >> 8) * join_hi_lo(d1[2], d1[3]);
        }
        acc[0] += xs * f16bits(ld_u16(ua + 208)) * fa;
        acc[1] += xs * f16bits(ld_u16(ub + 208)) * fb;
    } else if constexpr (TY == T_Q4_0) {
        const int4 x03 = *reinterpret_cast<const int4 *>(xw + 4), x47 = *reinterpret_cast<const int4 *>(xw + 8);
        const int xb[8] = {x03.x, x03.y, x03.z, x03.w, x47.x, x47.y, x47.z, x47.w};
        float fa = 0.f, fb = 0.f;
        const uint32_t sh = 4 * (c >> 1);  // threads 0, 1: low nibbles (k 0..15); 2, 3: high (k 16..31)
#pragma unroll
        for (int b = 0; b < 8; b++) {  // block b: {f16 d; u8 qs[16]}, this thread's eight bytes at 2 + 8 (c & 1)
            uint32_t qa[2], qb[2];
            lds_a2<2>(ua + 18 * b + 2 + 8 * (c & 1), qa);
            lds_a2<2>(ub + 18 * b + 2 + 8 * (c & 1), qb);
            int d[4];
            imma0<false>(d, (qa[0] >> sh) & 0x0F0F0F0Fu, (qb[0] >> sh) & 0x0F0F0F0Fu, (qa[1] >> sh) & 0x0F0F0F0Fu,
                         (qb[1] >> sh) & 0x0F0F0F0Fu, xf[2 * b], xf[2 * b + 1]);
            // (q - 8) * d: eight times the block's sum of x leaves again
            fa += f16bits(ld_u16(ua + 18 * b)) * (float)(d[0] * 256 + d[1] - 8 * xb[b]);
            fb += f16bits(ld_u16(ub + 18 * b)) * (float)(d[2] * 256 + d[3] - 8 * xb[b]);
        }
        acc[0] += xs * fa;
        acc[1] += xs * fb;
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
            const uint2 ea = tab[((wa[0] >> (8 * c)) & 0xFF) * tab_copies], eb = tab[((wb[0] >> (8 * c)) & 0xFF) * tab_copies];
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

// SEP: one column as a hi and a lo byte column.  An item is 8 consecutive k; the
// 32 items of a 256-wide unit are the 32 lanes of one warp, so the unit's largest
// magnitude is one warp reduction.  Magnitudes are compared as integers (the bit
// patterns of non-negative floats order like the floats, and every NaN pattern lies
// above infinity, so a NaN anywhere in the unit comes out on top and is seen).
// Rounding: v * inv + (1.5 * 2^23 + 128) lands where the float's low mantissa bits are
// the integer q + 128 = 256 * hi + (lo + 128): hi is byte 1, lo is byte 0 with its top
// bit flipped.  Byte order inside a quarter: k order (Q2_0: inside each 16, byte 4s + b
// holds k = s + 4b, the order the masked code words come in).  The quarter's record
// {scale, scale * sum of x over its first 32-wide block, over its second} follows its 64
// bytes in the first byte column.
template <int XDT> struct XRaw8 { uint4 v[XDT == DT_F32 ? 2 : 1]; };

template <int TY, int XDT>
__device__ __forceinline__ void stage_x_bytes(uint32_t xs32, uint32_t es, const void *x, uint32_t u_first, uint32_t nu,
                                              uint32_t tid) {
    const uint32_t items = nu * 32;
    constexpr uint32_t kFlight = 4;  // items a thread has in flight: the loads go out first
    constexpr uint32_t kMagicBits = 0x4B400080u;  // 1.5 * 2^23 + 128 as a float
    const uint32_t e8 = tid & 31;  // this lane's item inside its unit, the same in every pass
    const uint32_t c = e8 >> 3;
    const uint32_t item_off = c * kSepQuarter + (e8 & 7) * 8;  // 8 bytes of the quarter's 64
    for (uint32_t base = tid; base < items; base += kFlight * kConsumers) {
        XRaw8<XDT> raw[kFlight];
#pragma unroll
        for (uint32_t r = 0; r < kFlight; r++) {
            const uint32_t i = base + r * kConsumers;
            const uint4 *src = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint8_t *>(x) +
                                                              ((size_t)u_first * 256 + (size_t)i * 8) * (XDT == DT_F32 ? 4 : 2));
#pragma unroll
            for (int j = 0; j < (XDT == DT_F32 ? 2 : 1); j++)
                raw[r].v[j] = i < items ? __ldg(src + j) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (uint32_t r = 0; r < kFlight; r++) {
            const uint32_t i = base + r * kConsumers;
            if (i >= items) break;  // the same for the whole warp: a warp holds one unit
            float v[8];
            if constexpr (XDT == DT_F32) {
                v[0] = __uint_as_float(raw[r].v[0].x); v[1] = __uint_as_float(raw[r].v[0].y);
                v[2] = __uint_as_float(raw[r].v[0].z); v[3] = __uint_as_float(raw[r].v[0].w);
                v[4] = __uint_as_float(raw[r].v[1].x); v[5] = __uint_as_float(raw[r].v[1].y);
                v[6] = __uint_as_float(raw[r].v[1].z); v[7] = __uint_as_float(raw[r].v[1].w);
            } else {
                const uint32_t w[4] = {raw[r].v[0].x, raw[r].v[0].y, raw[r].v[0].z, raw[r].v[0].w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    if constexpr (XDT == DT_F16) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e]));
                        v[2 * e] = f.x; v[2 * e + 1] = f.y;
                    } else {
                        v[2 * e] = __uint_as_float(w[e] << 16);
                        v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
                    }
                }
            }
            uint32_t mb = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) mb = max(mb, __float_as_uint(v[j]) & 0x7FFFFFFFu);
            mb = __reduce_max_sync(0xffffffffu, mb);
            const float amax = __uint_as_float(mb);
            // amax below 1e-30: the unit counts as zeros (32512 / amax would overflow, and its
            // products vanish in fp32 anyway); amax infinite: inv = 0, scale = inf; amax a NaN:
            // both comparisons fail, inv = 0, and the scale is that NaN
            const float inv = amax > 1e-30f ? __fdividef(kXqMax, amax) : 0.f;
            const float scale = amax * (1.f / kXqMax);
            uint32_t t[8], tsum = 0;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                t[j] = __float_as_uint(fmaf(v[j], inv, __uint_as_float(kMagicBits)));
                tsum += t[j];
            }
            int qsum = (int)(tsum - 8u * kMagicBits);  // sum of the eight q
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
            qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
            const uint32_t u = i >> 5;
            const uint32_t dst = xs32 + u * kSepUnit + item_off;
            if constexpr (TY == T_Q2_0) {
                // this item is half (e8 & 1) of a 16: bytes 2h, 2h + 1 of each of its four words
                const uint32_t at16 = dst - (e8 & 1) * 8;
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    const uint32_t at = at16 + 4 * w + 2 * (e8 & 1);
                    sts16(at, prmt(t[w], t[w + 4], 0x0051u) & 0xFFFFu);
                    sts16(at + es, (prmt(t[w], t[w + 4], 0x0040u) & 0xFFFFu) ^ 0x8080u);
                }
            } else {
                sts64(dst, prmt(prmt(t[0], t[1], 0x0051u), prmt(t[2], t[3], 0x0051u), 0x5410u),
                      prmt(prmt(t[4], t[5], 0x0051u), prmt(t[6], t[7], 0x0051u), 0x5410u));
                sts64(dst + es, prmt(prmt(t[0], t[1], 0x0040u), prmt(t[2], t[3], 0x0040u), 0x5410u) ^ 0x80808080u,
                      prmt(prmt(t[4], t[5], 0x0040u), prmt(t[6], t[7], 0x0040u), 0x5410u) ^ 0x80808080u);
            }
            // the quarter's record, behind its 64 bytes in the first byte column
            const uint32_t rec = xs32 + u * kSepUnit + c * kSepQuarter + 64;
            if ((e8 & 7) == 0) sts32(rec, __float_as_uint(scale));
            if ((e8 & 3) == 0) sts32(rec + 4 + ((e8 >> 2) & 1) * 4, __float_as_uint(scale * (float)qsum));
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
    if constexpr (TY != T_Q2_0) {
        // An item is 8 consecutive k = the eight bytes thread c = item % 4 of a quad feeds into block
        // item / 4; the 32 items of a (column, unit) pair are the lanes of one warp, so the unit's
        // largest magnitude is one warp reduction and a block's sum two shuffles, as in the
        // one-column panel.  The loads of four pairs go out before the first is worked on.
        const uint32_t warp = tid >> 5, e8 = tid & 31, blk = e8 >> 2, c = e8 & 3;
        const uint32_t pairs = L.nc * nu;
        constexpr uint32_t kFlight = 4;
        constexpr uint32_t kMagicBits = 0x4B400080u;  // 1.5 * 2^23 + 128 as a float
        const uint32_t piece = xq_piece_offset(c, blk >> 1) + (blk & 1) * 8;
        for (uint32_t base = warp; base < pairs; base += kFlight * kGemvWarps) {
            XRaw8<XDT> raw[kFlight];
            uint32_t col_of[kFlight], u_of[kFlight];
#pragma unroll
            for (uint32_t r = 0; r < kFlight; r++) {
                const uint32_t pr = base + r * kGemvWarps;
                const bool live = pr < pairs;
                col_of[r] = live ? pr / nu : 0;
                u_of[r] = live ? pr - col_of[r] * nu : 0;
                const uint4 *src = reinterpret_cast<const uint4 *>(
                    reinterpret_cast<const uint8_t *>(x) +
                    ((size_t)col_of[r] * kdim + (size_t)(u_first + u_of[r]) * 256 + e8 * 8) * (XDT == DT_F32 ? 4 : 2));
#pragma unroll
                for (int j = 0; j < (XDT == DT_F32 ? 2 : 1); j++)
                    raw[r].v[j] = live ? __ldg(src + j) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (uint32_t r = 0; r < kFlight; r++) {
                if (base + r * kGemvWarps >= pairs) break;  // the same for the whole warp
                float v[8];
                if constexpr (XDT == DT_F32) {
                    v[0] = __uint_as_float(raw[r].v[0].x); v[1] = __uint_as_float(raw[r].v[0].y);
                    v[2] = __uint_as_float(raw[r].v[0].z); v[3] = __uint_as_float(raw[r].v[0].w);
                    v[4] = __uint_as_float(raw[r].v[1].x); v[5] = __uint_as_float(raw[r].v[1].y);
                    v[6] = __uint_as_float(raw[r].v[1].z); v[7] = __uint_as_float(raw[r].v[1].w);
                } else {
                    const uint32_t w[4] = {raw[r].v[0].x, raw[r].v[0].y, raw[r].v[0].z, raw[r].v[0].w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        if constexpr (XDT == DT_F16) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[e]));
                            v[2 * e] = f.x; v[2 * e + 1] = f.y;
                        } else {
                            v[2 * e] = __uint_as_float(w[e] << 16);
                            v[2 * e + 1] = __uint_as_float(w[e] & 0xFFFF0000u);
                        }
                    }
                }
                uint32_t mb = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) mb = max(mb, __float_as_uint(v[j]) & 0x7FFFFFFFu);
                mb = __reduce_max_sync(0xffffffffu, mb);
                const float amax = __uint_as_float(mb);
                // as in the one-column panel: below 1e-30 the unit counts as zeros, an infinite
                // amax gives inv = 0 and an infinite scale, a NaN gives inv = 0 and a NaN scale
                const float inv = amax > 1e-30f ? __fdividef(kXqMax, amax) : 0.f;
                const float scale = amax * (1.f / kXqMax);
                uint32_t t[8], tsum = 0;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    t[j] = __float_as_uint(fmaf(v[j], inv, __uint_as_float(kMagicBits)));
                    tsum += t[j];
                }
                int qsum = (int)(tsum - 8u * kMagicBits);
                qsum += __shfl_xor_sync(0xffffffffu, qsum, 1);
                qsum += __shfl_xor_sync(0xffffffffu, qsum, 2);
                uint8_t *dst = xs + (2 * col_of[r]) * L.es + u_of[r] * kXqUnit + piece;
                *reinterpret_cast<uint2 *>(dst) =
                    make_uint2(prmt(prmt(t[0], t[1], 0x0051u), prmt(t[2], t[3], 0x0051u), 0x5410u),
                               prmt(prmt(t[4], t[5], 0x0051u), prmt(t[6], t[7], 0x0051u), 0x5410u));
                *reinterpret_cast<uint2 *>(dst + L.es) =
                    make_uint2(prmt(prmt(t[0], t[1], 0x0040u), prmt(t[2], t[3], 0x0040u), 0x5410u) ^ 0x80808080u,
                               prmt(prmt(t[4], t[5], 0x0040u), prmt(t[6], t[7], 0x0040u), 0x5410u) ^ 0x80808080u);
                float *w12 = xw + ((size_t)u_of[r] * 4 + col_of[r]) * 12;
                if (c == 0) reinterpret_cast<int *>(w12)[4 + blk] = qsum;
                if (e8 == 0) w12[0] = scale;
            }
        }
        return;
    }
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

#ifndef OKF_GEMV_MINB
#define OKF_GEMV_MINB 2
#endif
template <int TY, int XDT, bool SEP>
__global__ void __launch_bounds__(kGemvThreadsMax, OKF_GEMV_MINB) gemv_kernel(GemvArgs p, GemvLayout L, GemvGather G) {
    constexpr uint32_t UB = UnitGeom<TY>::bytes;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kMaxStages);
    uint8_t *stages = smem + kBarBytes;
    uint8_t *xs = smem + L.xs_off;
    float4 *info = reinterpret_cast<float4 *>(smem + L.info_off);  // SEP: [unit][quarter]; WIDE: [unit][column] x 3
    float *red = reinterpret_cast<float *>(smem + L.red_off);      // [tile in group][warp][16][nc]
    const uint32_t smem32 = smem_u32(smem);

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
    if (threadIdx.x < 64) reinterpret_cast<uint32_t *>(smem + kZeroOff)[threadIdx.x] = 0u;
    if constexpr (TY == T_IQ2_XXS) {
        // The codebook, 256 entries of eight magnitude bytes, every entry `tab_copies`
        // times side by side: a lane reads copy (lane mod copies), so with 16 copies the
        // 16 lanes of a 64-bit access hit 16 different bank pairs whatever they look up.
        uint64_t *tw = reinterpret_cast<uint64_t *>(smem + L.tab_off);
        const uint32_t sh = 31 - __clz(L.tab_copies);
        for (uint32_t i = threadIdx.x; i < 256 * L.tab_copies; i += blockDim.x) tw[i] = g_iq2xxs_grid[i >> sh];
    }
    __syncthreads();

    // Steps are visited in the same order by the producer and the consumers: group
    // by group, inside a group k-chunk by k-chunk, inside that `tps` tiles at a time.
    if (warp == kGemvWarps + 1) {
        // ---- present in row-shard launches only: announce the exchange of the launch before
        if (lane == 0 && blockIdx.x == 0 && G.sig_nranks) {
            pdl_wait();
            gather_signal(G.sig_arrivals, G.sig_nranks);
        }
        return;
    }
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
                            !mbar_wait_relaxed(&empty[rp.s], (rp.use - 1) & 1, abort_flag, p.status, kStatusEmptyTimeout)) {
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
    const uint32_t tid = threadIdx.x;  // 0 .. kConsumers - 1
    // A wait that gives up marks the warp dead; a dead warp skips further waits but
    // keeps walking the loops, so the barriers among the consumer warps still match.
    bool alive = true;
    // `seen`: lane 0 already found the stage complete when it looked ahead during the step before
    auto wait_full = [&](uint32_t s, uint32_t use, bool seen) {
        bool ok = true;
        if (alive && lane == 0 && !seen) ok = mbar_wait(&full[s], use & 1, abort_flag, p.status, kStatusFullTimeout);
        alive = alive && __shfl_sync(0xffffffffu, ok, 0);
    };
    // has the stage at ring position `q` landed?  (lane 0 asks, before a step's arithmetic,
    // about the next step's stages, so that the answer is there when the step is over)
    auto peek_full = [&](const RingPos &q) { return lane == 0 && mbar_test_wait(&full[q.s], q.use & 1); };
    auto consumer_sync = [&]() { named_bar_sync(1, kConsumers); };

    // What this thread feeds into column g of the MMA's B operand.
    //   SEP:  byte column g % 2 of x, and only in the lanes of quarter g / 2.
    //   WIDE: byte column g of the panel (hi, lo of activation column g / 2), every lane
    //         its own 64 bytes; lanes of columns past the last one feed zeros.
    const bool x_active = SEP ? (g >> 1) == c : g < 2 * p.n;
    const uint8_t *xs_mine = xs + (SEP ? (g & 1) : g) * L.es + c * 64;
    const uint32_t xs_ustride = kXqUnit;
    const uint32_t xq_swap = (c >> 1) * 16;
    // The same in shared-window addresses for the one-column path.  Lanes that feed nothing
    // read zeros (stride 0) instead of predicating every load; their zeros sit on a bank
    // group that the two lanes carrying data in the same 8-lane phase do not touch.
    const SepConst KC = sep_const<TY>(c, lane, smem32 + L.tab_off, L.tab_copies);
    const uint32_t stages32 = smem32 + kBarBytes;
    const uint32_t xbase32 = SEP && x_active ? smem32 + L.xs_off + (g & 1) * L.es + c * kSepQuarter
                                             : smem32 + kZeroOff + ((5 * (g >> 1) + 1) & 7) * 16;
    const uint32_t xstride32 = SEP && x_active ? kSepUnit : 0u;
    const uint32_t rec32 = smem32 + L.xs_off + c * kSepQuarter + 64;  // this quarter's record of unit 0
    const uint32_t red32 = smem32 + L.red_off + (warp * 16 + g + 8 * (c & 1)) * 4;  // this thread's slot of tile 0
    // WIDE: this lane's copy of the IQ2_XXS codebook
    const uint2 *tab = reinterpret_cast<const uint2 *>(smem + L.tab_off) + (lane & (L.tab_copies - 1));
    RingPos rp;
    uint32_t rot = 0;  // the deal of units to warps rotates from step to step
    bool seen_a = false, seen_b = false;
    // Everything up to here, and clearing the first group's partial sums, needs nothing from
    // the kernel before this one.
    for (uint32_t i = tid; i < min(L.group, ntl) * kGemvWarps * 16 * L.nc; i += kConsumers) red[i] = 0.f;
    pdl_wait();  // activations come from the previous kernel; outputs may still be read by it
    if (G.wait_arrivals) {
        // x may hold, or derive from, rows other GPUs stored during the exchange launched
        // before this one: it has to be complete on this GPU before anybody reads x.  The
        // weights of this launch are already streaming in meanwhile.
        if (tid == 0) gather_wait(G.wait_arrivals, G.wait_epoch, p.status);
        named_bar_sync(1, kConsumers);
    }
    for (uint32_t gb = 0; gb < ntl; gb += L.group) {
        const uint32_t gn = min(L.group, ntl - gb);
        if (gb > 0)
            for (uint32_t i = tid; i < gn * kGemvWarps * 16 * L.nc; i += kConsumers) red[i] = 0.f;
        for (uint32_t j0 = 0; j0 < p.nchunk; j0 += L.panel) {
            const uint32_t j1 = min(j0 + L.panel, p.nchunk);
            const uint32_t pu0 = j0 * p.cb, pnu = min(j1 * p.cb, p.nunit) - pu0;
            if (gb == 0 || L.panel < p.nchunk) {
                // the previous panel is still being read until every warp gets here
                if (gb > 0 || j0 > 0) consumer_sync();
                if constexpr (SEP) stage_x_bytes<TY, XDT>(smem32 + L.xs_off, L.es, p.x, pu0, pnu, tid);
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
                    wait_full(rp.s, rp.use, seen_a);
                    rp.next(L.nstage);
                    const uint32_t sB = rp.s;
                    if (spt == 2) {
                        wait_full(rp.s, rp.use, seen_b);
                        rp.next(L.nstage);
                    }
                    {   // look ahead at the next step's stage(s)
                        RingPos q = rp;
                        seen_a = peek_full(q);
                        q.next(L.nstage);
                        seen_b = spt == 2 && peek_full(q);
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
                    // Integer instructions run at half the rate of the others on this part and the
                    // unit bodies are full of them, so a warp takes a run of consecutive units of the
                    // step's tn * nu (unit v being unit v % nu of tile v / nu): the loop over a run
                    // within one tile is a counter and a few addresses moved by constants, and the
                    // sums are put away once per run.  The warps that get one unit more than the
                    // others rotate from step to step.
                    const uint32_t total = tn * nu;
                    const uint32_t wr = warp >= rot ? warp - rot : warp + kGemvWarps - rot;
                    const uint32_t share = total / kGemvWarps, extra = total % kGemvWarps;
                    rot = (rot + extra) % kGemvWarps;
                    uint32_t left = share + (wr < extra ? 1u : 0u);
                    uint32_t ti = 0, u = wr * share + min(wr, extra);
                    while (u >= nu && ti + 1 < tn) { u -= nu; ti++; }
                    if constexpr (SEP) {
                        uint32_t wa = stages32 + (uint32_t)(ra - stages) + ti * tile_bytes + (ubase + u) * UB;  // row g
                        const uint32_t wdelta = (uint32_t)(rb - ra);                                            // to row g + 8
                        uint32_t xa = xbase32 + (pu + u) * xstride32;
                        uint32_t ia = rec32 + (pu + u) * kSepUnit;
                        uint32_t da = red32 + (tl - gb + ti) * (kGemvWarps * 16 * 4);
                        while (left) {
                            const uint32_t run = min(left, nu - u);  // the rest of this tile, or of the share
                            left -= run;
                            float acc[2] = {0.f, 0.f};
#pragma unroll 1
                            for (uint32_t i = run; i; i--) {
                                const uint4 q0 = lds128(xa), q1 = lds128(xa + 16), q2 = lds128(xa + 32), q3 = lds128(xa + 48);
                                const uint32_t xf[16] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w,
                                                         q2.x, q2.y, q2.z, q2.w, q3.x, q3.y, q3.z, q3.w};
                                const uint4 xi = lds128(ia);
                                unit_sep<TY>(wa, wa + wdelta, KC, xf, xi, acc);
                                wa += UB;
                                xa += xstride32;
                                ia += kSepUnit;
                            }
                            // each thread of a quad covered another quarter: add them up and put the
                            // sums into the warp's slot of the tile
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
                                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
                            }
                            if (c < 2) sts32(da, __float_as_uint(__uint_as_float(lds32(da)) + (c ? acc[1] : acc[0])));
                            // on to the first unit of the next tile
                            u = 0;
                            wa += tile_bytes - nu * UB;
                            xa -= nu * xstride32;
                            ia -= nu * kSepUnit;
                            da += kGemvWarps * 16 * 4;
                        }
                    } else {
                        // lanes of columns that do not exist read column 0's record; their sums are dropped
                        const float *xw0 = reinterpret_cast<const float *>(info) + (c < L.nc ? c : 0) * 12;
                        while (left) {
                            const uint32_t run = min(left, nu - u);
                            left -= run;
                            const uint8_t *ta = ra + (size_t)ti * tile_bytes + (size_t)(ubase + u) * UB;
                            const uint32_t tdelta = (uint32_t)(rb - ra);
                            const uint8_t *xp = xs_mine + (pu + u) * xs_ustride;
                            const float *xw = xw0 + (size_t)(pu + u) * 48;
                            float acc[2] = {0.f, 0.f};
#pragma unroll 1
                            for (uint32_t i = run; i; i--) {
                                uint32_t xf[16];
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                                    if (x_active) w4 = lds128(xp + (q >> 1) * 32 + ((q & 1) ? 16 - xq_swap : xq_swap));
                                    xf[4 * q] = w4.x; xf[4 * q + 1] = w4.y; xf[4 * q + 2] = w4.z; xf[4 * q + 3] = w4.w;
                                }
                                unit_wide<TY>(ta, ta + tdelta, c, xf, xw, tab, L.tab_copies, acc);
                                ta += UB;
                                xp += xs_ustride;
                                xw += 48;
                            }
                            // thread (g, c) holds the sums of rows g, g + 8 for column c: into this
                            // warp's own slot of the tile's partial sums
                            if (c < L.nc) {
                                float *dst = red + ((size_t)(tl - gb + ti) * kGemvWarps + warp) * 16 * L.nc;
                                dst[g * L.nc + c] += acc[0];
                                dst[(g + 8) * L.nc + c] += acc[1];
                            }
                            u = 0;
                            ti++;
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
        if (G.nranks == 0) {
            for (uint32_t i = tid; i < gn * per_tile; i += kConsumers) {
                const uint32_t tl = i / per_tile, r = (i % per_tile) / L.nc, col = i % L.nc;
                const float *src = red + (size_t)tl * kGemvWarps * per_tile + r * L.nc + col;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < kGemvWarps; w++) sum += src[(size_t)w * per_tile];
                const GemvSeg sg = gemv_segment(p, t0 + gb + tl);
                const uint32_t row = (t0 + gb + tl - sg.tile0) * 16 + r;
                if (row < sg.m) sg.out[(size_t)col * sg.m + row] = sum;
            }
        } else {
            // Row shards: an item is four consecutive rows of one column for one rank, stored
            // as one 16-byte word into that rank's copy of the whole output; the ranks of a
            // run of rows are taken by different threads so that their stores go out side by side.
            const uint32_t runs = gn * 4 * L.nc;  // (tile, four-row run, column)
            for (uint32_t i = tid; i < runs * G.nranks; i += kConsumers) {
                const uint32_t rk = i / runs, j = i % runs;
                const uint32_t tl = j / (4 * L.nc), r0 = (j / L.nc) % 4 * 4, col = j % L.nc;
                const float *src = red + (size_t)tl * kGemvWarps * per_tile + r0 * L.nc + col;
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int w = 0; w < kGemvWarps; w++)
#pragma unroll
                    for (int e = 0; e < 4; e++) sum[e] += src[(size_t)w * per_tile + e * L.nc];
                const GemvSeg sg = gemv_segment(p, t0 + gb + tl);
                const uint32_t row = (t0 + gb + tl - sg.tile0) * 16 + r0;
                if (row >= sg.m) continue;
                float *dst = G.out[sg.index][rk] + (size_t)col * G.m_total[sg.index] + G.row_first[sg.index] + row;
                if (row + 4 <= sg.m && ((uintptr_t)dst & 15) == 0) {
                    *reinterpret_cast<float4 *>(dst) = make_float4(sum[0], sum[1], sum[2], sum[3]);
                } else {
                    for (uint32_t e = 0; e < 4 && row + e < sg.m; e++) dst[e] = sum[e];
                }
            }
        }
        if (gb + L.group < ntl) consumer_sync();  // before the buffer is zeroed again
    }
    // Row shards: nobody fences or waits here.  The count the local counter has to reach for
    // the exchanges launched so far goes up by one per rank; whoever waits next reads it after
    // this kernel is complete.
    if (G.nranks && blockIdx.x == 0 && tid == 0) G.epoch[0] += G.nranks;
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

static bool gemv_layout_with(int ty, uint32_t nunit, uint32_t n, bool sep, uint32_t tiles_per_cta, uint32_t tab_copies,
                             uint32_t budget, GemvArgs &a, GemvLayout &L) {
    const uint32_t ub = (ty == T_Q4_K || ty == T_Q4_0 || ty == T_IQ4_NL) ? 144 : ty == T_Q8_0 ? 272 : ty == T_Q2_0 ? 68 : ty == T_Q6_K ? 210 : ty == T_Q5_K ? 176 : 66;
    L.nc = sep ? 1 : n;
    L.ecols = sep ? 2 : 2 * n;
    const uint32_t per_tile = kGemvWarps * 16 * L.nc * 4;
    L.group = 8192 / per_tile;
    if (L.group < 1) L.group = 1;
    if (L.group > tiles_per_cta) L.group = tiles_per_cta;
    const uint32_t red_bytes = L.group * per_tile;
    const uint32_t tab_bytes = ty == T_IQ2_XXS ? 256 * 8 * tab_copies : 0;
    L.tab_copies = tab_copies;
    const uint32_t stage_cap = 46 * 1024;
    const uint32_t row_bytes = nunit * ub;
    // per unit: SEP 320 bytes per byte column, records included; WIDE 256 per byte column + 4 columns x 12 words
    const uint32_t xunit = sep ? kSepUnit : kXqUnit, info_unit = sep ? 0 : 4 * 48;
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
            if (L.ragged && ty != T_IQ2_XXS && ty != T_Q2_0 && ty != T_Q6_K) continue;
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
        const uint32_t small = kBarBytes + red_bytes + tab_bytes + 64 + 128 + L.ecols * 128;
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
        L.es = sep ? sep_col_stride(panel * cb) : xq_col_stride(panel * cb);
        L.xs_off = (kBarBytes + nstage * stage + 127) & ~127u;  // the bank arithmetic of the panel counts from 128
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

// IQ2_XXS: as many side-by-side copies of the codebook as leave room for a plan that
// keeps all of x resident (16 copies make every look-up free of bank conflicts).
static bool gemv_layout_in(int ty, uint32_t nunit, uint32_t n, bool sep, uint32_t tiles_per_cta, uint32_t budget,
                           GemvArgs &a, GemvLayout &L) {
    if (ty != T_IQ2_XXS) return gemv_layout_with(ty, nunit, n, sep, tiles_per_cta, 1, budget, a, L);
    GemvArgs fa = a;
    GemvLayout fl = L;
    bool have = false;
    for (uint32_t copies = 16; copies >= 1; copies /= 2) {
        GemvArgs ta = a;
        GemvLayout tl = L;
        if (!gemv_layout_with(ty, nunit, n, sep, tiles_per_cta, copies, budget, ta, tl)) continue;
        if (tl.panel == ta.nchunk) { a = ta; L = tl; return true; }
        if (!have) { fa = ta; fl = tl; have = true; }
    }
    if (have) { a = fa; L = fl; }
    return have;
}

static bool gemv_layout(int ty, uint32_t nunit, uint32_t n, bool sep, uint32_t tiles_per_cta, GemvArgs &a,
                        GemvLayout &L) {
    // (Tried for several columns of long rows, whose panel of x does not fit beside the ring in
    // half an SM's shared memory: taking the SM alone with the whole panel resident.  Slower:
    // the next kernel can then not prefetch under this one.)
    return gemv_layout_in(ty, nunit, n, sep, tiles_per_cta, kSharedBudget, a, L);
}

// CTAs of a launch: one per SM, each with its share of the tiles -- except when there are only
// a few more tiles than SMs (160 on 148): then two tiles in a row on a dozen SMs would set the
// launch's time, and one CTA per tile is used instead; an SM has room for two of them side by
// side, and they do not slow each other down much (a CTA alone issues on a third of the cycles).
// (One column only: with several columns two CTAs on an SM, each staging its slices of x at
// barriers, were 16 % slower than two tiles in a row.)
static uint32_t gemv_ctas(uint32_t tiles, int sms, bool sep) {
    const uint32_t n = (uint32_t)sms;
    if (tiles <= n) return tiles;
    return sep && tiles <= n + n / 4 ? tiles : n;
}

template <int TY, int XDT, bool SEP>
static cudaError_t launch_t(GemvArgs a, const GemvGather &G, cudaStream_t s, int sms, int dev) {
    GemvLayout L;
    const uint32_t ctas = gemv_ctas(a.tiles, sms, SEP);
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
    cfg.blockDim = dim3(G.nranks ? kGemvThreadsMax : kGemvThreads);
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
    if (!has_fast_kernels(ty)) return false;
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
    const uint32_t ctas = gemv_ctas(tiles, sms, true), ctas_wide = gemv_ctas(tiles, sms, false);
    if (!gemv_layout(ty, k / 256, 1, true, (tiles + ctas - 1) / ctas, a, L)) return false;
    if (n > 1 && !gemv_layout(ty, k / 256, n < 4 ? n : 4, false, (tiles + ctas_wide - 1) / ctas_wide, a, L)) return false;
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
    a.row_bytes = a.nunit * ((ty == T_Q4_K || ty == T_Q4_0 || ty == T_IQ4_NL) ? 144 : ty == T_Q8_0 ? 272 : ty == T_Q2_0 ? 68 : ty == T_Q6_K ? 210 : ty == T_Q5_K ? 176 : 66);
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
        G.wait_arrivals = gather->wait_arrivals;
        G.sig_nranks = gather->sig_nranks;
        for (uint32_t r = 0; r < gather->sig_nranks; r++) G.sig_arrivals[r] = gather->sig_arrivals[r];
        G.wait_epoch = gather->wait_epoch;
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
        case T_Q4_0: e = launch_ty<T_Q4_0>(a, G, xdt, sep, s, sms, dev); break;
        case T_Q6_K: e = launch_ty<T_Q6_K>(a, G, xdt, sep, s, sms, dev); break;
        case T_Q5_K: e = launch_ty<T_Q5_K>(a, G, xdt, sep, s, sms, dev); break;
        case T_IQ4_NL: e = launch_ty<T_IQ4_NL>(a, G, xdt, sep, s, sms, dev); break;
        case T_Q2_0: e = launch_ty<T_Q2_0>(a, G, xdt, sep, s, sms, dev); break;
        case T_IQ2_XXS: e = launch_ty<T_IQ2_XXS>(a, G, xdt, sep, s, sms, dev); break;
        default: e = cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
        if (launches) ++*launches;
        if (gather) {  // a further pass over columns announces this pass's exchange and waits for it
            G.wait_arrivals = gather->arrivals[gather->rank];
            G.wait_epoch = gather->epoch;
            G.sig_nranks = gather->nranks;
            for (uint32_t r = 0; r < gather->nranks; r++) G.sig_arrivals[r] = gather->arrivals[r];
        }
        c0 += take;
    }
    return cudaSuccess;
}

__global__ void gather_wait_kernel(GemvGather G, int *status) {
    pdl_wait();
    if (G.sig_nranks) gather_signal(G.sig_arrivals, G.sig_nranks);
    if (G.wait_arrivals) gather_wait(G.wait_arrivals, G.wait_epoch, status);
}

cudaError_t launch_gather_wait(const GemvGatherPlan &plan, int *status, cudaStream_t s) {
    GemvGather G = {};
    G.wait_arrivals = plan.wait_arrivals;
    G.wait_epoch = plan.wait_epoch;
    G.sig_nranks = plan.sig_nranks;
    for (uint32_t r = 0; r < plan.sig_nranks; r++) G.sig_arrivals[r] = plan.sig_arrivals[r];
    gather_wait_kernel<<<1, 1, 0, s>>>(G, status);
    return cudaGetLastError();
}

cudaError_t launch_gemv_fast(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                             uint32_t n, float *out, int *status, cudaStream_t s, int sms, int dev,
                             uint64_t *launches) {
    return launch_gemv_group(ty, 1, &w, &m, &out, k, x, xdt, n, status, s, sms, dev, launches, nullptr);
}

}  // namespace okf
