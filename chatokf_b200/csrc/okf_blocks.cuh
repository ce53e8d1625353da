// Block geometry and bit-exact device decoders for Q8_0, Q4_K, IQ2_XXS, Q2_0 and, for the
// plain kernels only, Q4_0, IQ4_NL, Q5_K and Q6_K.
//
// Every decoder works on a "granule" of 32 consecutive weights of one row (one
// Q8_0 block, one Q4_K / IQ2_XXS sub-block, a quarter of a Q2_0 block) and
// produces exactly the fp32 values of the reference's block decoders
// (LLM/Gemma/Gemma4Quant.swift:51-69, LLM/Quantize/KQuants.swift:86-125,
// LLM/Quantize/IQ2XXS.swift:34-53, LLM/Base/Quant.swift:10-25; Q4_0 and IQ4_NL
// LLM/Gemma/Gemma4Quant.swift:5-49, Q5_K and Q6_K LLM/Quantize/KQuants.swift:127-177).  The reference
// rounds after every multiply and subtract, so the decoders use __fmul_rn /
// __fsub_rn, which the compiler never contracts into a fused multiply-add.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "iq2xxs_tables.h"

namespace okf {

enum : int { T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ4_NL = 20, T_Q2_0 = 42 };
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };

template <int TY> struct Geom;
template <> struct Geom<T_Q8_0> { static constexpr int per = 32, bytes = 34; };
template <> struct Geom<T_Q4_K> { static constexpr int per = 256, bytes = 144; };
template <> struct Geom<T_IQ2_XXS> { static constexpr int per = 256, bytes = 66; };
template <> struct Geom<T_Q2_0> { static constexpr int per = 128, bytes = 34; };
template <> struct Geom<T_Q4_0> { static constexpr int per = 32, bytes = 18; };
template <> struct Geom<T_IQ4_NL> { static constexpr int per = 32, bytes = 18; };
template <> struct Geom<T_Q5_K> { static constexpr int per = 256, bytes = 176; };
template <> struct Geom<T_Q6_K> { static constexpr int per = 256, bytes = 210; };

__host__ __device__ inline int block_elems(int ty) {
    return ty == T_Q8_0 ? 32 : ty == T_Q4_K ? 256 : ty == T_IQ2_XXS ? 256 : ty == T_Q2_0 ? 128
         : (ty == T_Q4_0 || ty == T_IQ4_NL) ? 32 : (ty == T_Q5_K || ty == T_Q6_K) ? 256 : 0;
}
__host__ __device__ inline int block_bytes(int ty) {
    return ty == T_Q8_0 ? 34 : ty == T_Q4_K ? 144 : ty == T_IQ2_XXS ? 66 : ty == T_Q2_0 ? 34
         : (ty == T_Q4_0 || ty == T_IQ4_NL) ? 18 : ty == T_Q5_K ? 176 : ty == T_Q6_K ? 210 : 0;
}
// the types the streaming matvec and the tensor-core matmul take; the rest run on the plain kernels
__host__ __device__ inline bool has_fast_kernels(int ty) {
    return ty == T_Q8_0 || ty == T_Q4_K || ty == T_IQ2_XXS || ty == T_Q2_0 || ty == T_Q4_0 || ty == T_Q6_K || ty == T_Q5_K || ty == T_IQ4_NL;
}

// IQ2_XXS codebook in device memory: 256 x u64 magnitudes, one copy per
// translation unit (2 KB); kernels copy it to shared memory before use.
static __device__ const uint64_t g_iq2xxs_grid[256] = {OKF_IQ2XXS_GRID_VALUES};

__device__ __forceinline__ float f16bits(uint32_t b) {
    return __half2float(__ushort_as_half((unsigned short)b));
}
__device__ __forceinline__ uint32_t ld_u16(const uint8_t *p) {  // 2-byte aligned
    return *reinterpret_cast<const uint16_t *>(p);
}
__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t *p) {  // 2-byte aligned
    return ld_u16(p) | (ld_u16(p + 2) << 16);
}

// bit j of the result set = element j negative.  The reference's sign table
// (LLM/Quantize/IQ2Grid.swift:73-85) holds i | (parity(i) << 7) for every one of
// its 128 entries (checked against the table in the tests), so it is computed.
__device__ __forceinline__ uint32_t iq2_signs(uint32_t idx7) {
    return idx7 | ((__popc(idx7) & 1u) << 7);
}

// Decode the 32 weights [32*gran, 32*gran + 32) of the row starting at `row`
// into w[0..31].  `grid` points at the 256-entry IQ2_XXS grid (shared or global).
template <int TY>
__device__ __forceinline__ void decode32(const uint8_t *row, uint32_t gran, float *w,
                                         const uint64_t *grid) {
    if constexpr (TY == T_Q8_0) {
        const uint8_t *b = row + (size_t)gran * 34;
        const float d = f16bits(ld_u16(b));
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
            uint32_t v = ld_u16(b + 2 + j);
            w[j] = __fmul_rn((float)(int8_t)(v & 0xFF), d);
            w[j + 1] = __fmul_rn((float)(int8_t)(v >> 8), d);
        }
    } else if constexpr (TY == T_Q2_0) {
        const uint8_t *b = row + (size_t)(gran >> 2) * 34;
        const float d = f16bits(ld_u16(b));
        const uint8_t *qs = b + 2 + (gran & 3) * 8;
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            uint32_t v = ld_u16(qs + j);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                int code = (int)((v >> (2 * e)) & 3u);
                w[j * 4 + e] = __fmul_rn((float)(code - 1), d);
            }
        }
    } else if constexpr (TY == T_Q4_K) {
        const uint8_t *b = row + (size_t)(gran >> 3) * 144;  // 16-byte aligned
        const uint32_t j = gran & 7;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(b);
        const float d = f16bits(dd & 0xFFFF), dmin = f16bits(dd >> 16);
        const uint8_t *s = b + 4;
        uint32_t sc, mn;
        if (j < 4) {
            sc = s[j] & 63u;
            mn = s[j + 4] & 63u;
        } else {
            sc = (s[j + 4] & 0xFu) | ((uint32_t)(s[j - 4] >> 6) << 4);
            mn = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
        }
        const float d1 = __fmul_rn(d, (float)sc), o1 = __fmul_rn(dmin, (float)mn);
        const uint32_t *q = reinterpret_cast<const uint32_t *>(b + 16 + (j >> 1) * 32);
        const uint32_t sh = (j & 1) * 4;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t v = q[i] >> sh;
#pragma unroll
            for (int e = 0; e < 4; e++)
                w[i * 4 + e] = __fsub_rn(__fmul_rn(d1, (float)((v >> (8 * e)) & 0xFu)), o1);
        }
    } else if constexpr (TY == T_Q4_0 || TY == T_IQ4_NL) {
        // {f16 d; u8 qs[16]}: byte j holds element j (low nibble) and j + 16 (high).
        // Q4_0: (q - 8) * d; IQ4_NL: kvalues[q] * d (LLM/Gemma/Gemma4Quant.swift:5-49)
        const uint8_t *b = row + (size_t)gran * 18;
        const float d = f16bits(ld_u16(b));
        const float kv[16] = {-127.f, -104.f, -83.f, -65.f, -49.f, -35.f, -22.f, -10.f,
                              1.f, 13.f, 25.f, 38.f, 53.f, 69.f, 89.f, 113.f};
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
            const uint32_t v = ld_u16(b + 2 + j);
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const uint32_t lo = (v >> (8 * e)) & 0xFu, hi = (v >> (8 * e + 4)) & 0xFu;
                if constexpr (TY == T_Q4_0) {
                    w[j + e] = __fmul_rn((float)lo - 8.f, d);
                    w[j + e + 16] = __fmul_rn((float)hi - 8.f, d);
                } else {
                    w[j + e] = __fmul_rn(kv[lo], d);
                    w[j + e + 16] = __fmul_rn(kv[hi], d);
                }
            }
        }
    } else if constexpr (TY == T_Q5_K) {
        // {f16 d; f16 dmin; u8 scales[12]; u8 qh[32]; u8 qs[128]} (KQuants.swift:127-158):
        // sub-block j: nibbles as in Q4_K, fifth bit = bit j of qh[l]; d1 * q - o1
        const uint8_t *b = row + (size_t)(gran >> 3) * 176;
        const uint32_t j = gran & 7;
        const float d = f16bits(ld_u16(b)), dmin = f16bits(ld_u16(b + 2));
        const uint8_t *s = b + 4;
        uint32_t sc, mn;
        if (j < 4) {
            sc = s[j] & 63u;
            mn = s[j + 4] & 63u;
        } else {
            sc = (s[j + 4] & 0xFu) | ((uint32_t)(s[j - 4] >> 6) << 4);
            mn = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
        }
        const float d1 = __fmul_rn(d, (float)sc), o1 = __fmul_rn(dmin, (float)mn);
        const uint8_t *qh = b + 16, *qs = b + 48 + (j >> 1) * 32;
        const uint32_t sh = (j & 1) * 4;
#pragma unroll
        for (int l = 0; l < 32; l++) {
            const uint32_t q = ((qs[l] >> sh) & 0xFu) + (((qh[l] >> j) & 1u) << 4);
            w[l] = __fsub_rn(__fmul_rn(d1, (float)q), o1);
        }
    } else if constexpr (TY == T_Q6_K) {
        // {u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d} (KQuants.swift:160-177): granule
        // (n = half of the block, r = which 32 of its 128): low four bits from ql, two more
        // from qh, d * scale * (q - 32) multiplied left to right
        const uint8_t *b = row + (size_t)(gran >> 3) * 210;
        const uint32_t n = (gran >> 2) & 1, r = gran & 3;
        const float d = f16bits(ld_u16(b + 208));
        const uint8_t *ql = b + n * 64 + (r & 1) * 32, *qh = b + 128 + n * 32;
        const int8_t *sc = reinterpret_cast<const int8_t *>(b + 192 + n * 8 + 2 * r);
#pragma unroll
        for (int l = 0; l < 32; l++) {
            const uint32_t nib = r < 2 ? (ql[l] & 0xFu) : (uint32_t)(ql[l] >> 4);
            const int q = (int)(nib | (((qh[l] >> (2 * r)) & 3u) << 4)) - 32;
            w[l] = __fmul_rn(__fmul_rn(d, (float)sc[l >> 4]), (float)q);
        }
    } else {  // IQ2_XXS
        const uint8_t *b = row + (size_t)(gran >> 3) * 66;
        const float d = f16bits(ld_u16(b));
        const uint8_t *p = b + 2 + (gran & 7) * 8;
        const uint32_t a0 = ld_u32_a2(p), a1 = ld_u32_a2(p + 4);
        const float db = __fmul_rn(__fmul_rn(d, 0.5f + (float)(a1 >> 28)), 0.25f);
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const uint64_t e = grid[(a0 >> (8 * l)) & 0xFF];
            const uint32_t sg = iq2_signs((a1 >> (7 * l)) & 127u);
#pragma unroll
            for (int j = 0; j < 8; j++) {
                float g = __fmul_rn(db, (float)(uint32_t)((e >> (8 * j)) & 0xFF));
                w[l * 8 + j] = (sg >> j) & 1u ? -g : g;
            }
        }
    }
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

}  // namespace okf
