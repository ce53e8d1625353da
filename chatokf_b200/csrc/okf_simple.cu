// Straightforward kernels: exact dequant, warp-per-row matvec, fp32 tile matmul.
//
// dequant is the bit-exactness probe (the reference demands maxAbs == 0 from its
// dequant-row kernels, LLM/LLMTests/GemmaMetalKernelTests.swift:111-140) and the
// embedding-row unpacker.  The matvec / matmul here accumulate exact fp32
// products of the exactly decoded weights; they are the on-device yardstick for
// the streaming and tensor-core kernels and take any shape those decline.
#include "okf_blocks.cuh"
#include "okf_kernels.h"

namespace okf {

// ---- dequant ---------------------------------------------------------------
// One thread unpacks one granule of 32 weights and stores eight float4s.
template <int TY>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t *__restrict__ w,
                                                      uint64_t granules, float *__restrict__ out) {
    __shared__ uint64_t grid_s[256];
    if constexpr (TY == T_IQ2_XXS) {
        grid_s[threadIdx.x] = g_iq2xxs_grid[threadIdx.x];
        __syncthreads();
    }
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < granules; g += stride) {
        // decode32 indexes granules from a row start; here the "row" is the
        // whole span, split so the 32-bit granule index never overflows.
        const uint64_t gpb = Geom<TY>::per / 32;  // granules per block
        const uint64_t blk = g / gpb;
        float v[32];
        decode32<TY>(w + blk * Geom<TY>::bytes, (uint32_t)(g % gpb), v, grid_s);
        float4 *o = reinterpret_cast<float4 *>(out + g * 32);
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
}

template <int TY>
static cudaError_t dequant_t(const uint8_t *w, uint64_t count, float *out, cudaStream_t s) {
    const uint64_t granules = count / 32;
    if (granules == 0) return cudaSuccess;
    uint64_t blocks = (granules + 255) / 256;
    if (blocks > 148ull * 64) blocks = 148ull * 64;
    dequant_kernel<TY><<<(unsigned)blocks, 256, 0, s>>>(w, granules, out);
    return cudaGetLastError();
}

cudaError_t launch_dequant(int ty, const uint8_t *w, uint64_t count, float *out, cudaStream_t s) {
    switch (ty) {
    case T_Q8_0: return dequant_t<T_Q8_0>(w, count, out, s);
    case T_Q4_K: return dequant_t<T_Q4_K>(w, count, out, s);
    case T_IQ2_XXS: return dequant_t<T_IQ2_XXS>(w, count, out, s);
    case T_Q2_0: return dequant_t<T_Q2_0>(w, count, out, s);
    case T_Q4_0: return dequant_t<T_Q4_0>(w, count, out, s);
    case T_IQ4_NL: return dequant_t<T_IQ4_NL>(w, count, out, s);
    case T_Q5_K: return dequant_t<T_Q5_K>(w, count, out, s);
    case T_Q6_K: return dequant_t<T_Q6_K>(w, count, out, s);
    default: return cudaErrorInvalidValue;
    }
}

// ---- matvec, N <= 8 columns --------------------------------------------------
// One warp per output row; lane l takes granules l, l+32, ...; fp32 FMAs; the
// 32 lane partials are combined with shuffles.
template <int TY, typename XT>
__global__ void __launch_bounds__(128) gemv_simple_kernel(const uint8_t *__restrict__ w, uint32_t k,
                                                          uint32_t m, const XT *__restrict__ x,
                                                          uint32_t n, float *__restrict__ out) {
    __shared__ uint64_t grid_s[256];
    if constexpr (TY == T_IQ2_XXS) {
        for (int i = threadIdx.x; i < 256; i += blockDim.x) grid_s[i] = g_iq2xxs_grid[i];
        __syncthreads();
    }
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= m) return;
    const size_t row_bytes = (size_t)(k / Geom<TY>::per) * Geom<TY>::bytes;
    const uint8_t *rp = w + (size_t)row * row_bytes;
    float acc[8];
#pragma unroll
    for (int c = 0; c < 8; c++) acc[c] = 0.f;
    for (uint32_t g = lane; g < k / 32; g += 32) {
        float v[32];
        decode32<TY>(rp, g, v, grid_s);
#pragma unroll
        for (int c = 0; c < 8; c++) {
            if (c < (int)n) {
                const XT *xp = x + (size_t)c * k + (size_t)g * 32;
#pragma unroll
                for (int j = 0; j < 32; j++) acc[c] = fmaf(v[j], to_f32<XT>(xp[j]), acc[c]);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 8; c++) {
        float a = acc[c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && c < (int)n) out[(size_t)c * m + row] = a;
    }
}

template <int TY>
static cudaError_t gemv_simple_t(const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                                 uint32_t n, float *out, cudaStream_t s) {
    const unsigned blocks = (m + 3) / 4;
    switch (xdt) {
    case DT_F32:
        gemv_simple_kernel<TY, float><<<blocks, 128, 0, s>>>(w, k, m, (const float *)x, n, out);
        break;
    case DT_F16:
        gemv_simple_kernel<TY, __half><<<blocks, 128, 0, s>>>(w, k, m, (const __half *)x, n, out);
        break;
    case DT_BF16:
        gemv_simple_kernel<TY, __nv_bfloat16><<<blocks, 128, 0, s>>>(w, k, m, (const __nv_bfloat16 *)x, n, out);
        break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_gemv_simple(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x,
                               int xdt, uint32_t n, float *out, cudaStream_t s) {
    if (n == 0 || n > 8) return cudaErrorInvalidValue;
    switch (ty) {
    case T_Q8_0: return gemv_simple_t<T_Q8_0>(w, k, m, x, xdt, n, out, s);
    case T_Q4_K: return gemv_simple_t<T_Q4_K>(w, k, m, x, xdt, n, out, s);
    case T_IQ2_XXS: return gemv_simple_t<T_IQ2_XXS>(w, k, m, x, xdt, n, out, s);
    case T_Q2_0: return gemv_simple_t<T_Q2_0>(w, k, m, x, xdt, n, out, s);
    case T_Q4_0: return gemv_simple_t<T_Q4_0>(w, k, m, x, xdt, n, out, s);
    case T_IQ4_NL: return gemv_simple_t<T_IQ4_NL>(w, k, m, x, xdt, n, out, s);
    case T_Q5_K: return gemv_simple_t<T_Q5_K>(w, k, m, x, xdt, n, out, s);
    case T_Q6_K: return gemv_simple_t<T_Q6_K>(w, k, m, x, xdt, n, out, s);
    default: return cudaErrorInvalidValue;
    }
}

// ---- matmul, any N -----------------------------------------------------------
// 64 (rows) x 64 (tokens) output tile per CTA, 32 deep per step, 256 threads
// with a 4 x 4 register tile each.  Weights are decoded exactly to fp32 in
// shared memory; activations are widened to fp32.
template <int TY, typename XT, typename OT>
__global__ void __launch_bounds__(256) gemm_simple_kernel(const uint8_t *__restrict__ w, uint32_t k,
                                                          uint32_t m, const XT *__restrict__ x,
                                                          uint32_t n, OT *__restrict__ out) {
    __shared__ uint64_t grid_s[256];
    __shared__ float ws[32][65];
    __shared__ float xs[32][65];
    if constexpr (TY == T_IQ2_XXS) grid_s[threadIdx.x] = g_iq2xxs_grid[threadIdx.x];
    const uint32_t m0 = blockIdx.x * 64, n0 = blockIdx.y * 64;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t row_bytes = (size_t)(k / Geom<TY>::per) * Geom<TY>::bytes;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (uint32_t g = 0; g < k / 32; g++) {
        __syncthreads();
        if (threadIdx.x < 64) {
            const uint32_t r = m0 + threadIdx.x;
            float v[32];
            if (r < m) {
                decode32<TY>(w + (size_t)r * row_bytes, g, v, grid_s);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = 0.f;
            }
#pragma unroll
            for (int j = 0; j < 32; j++) ws[j][threadIdx.x] = v[j];
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t e = threadIdx.x + 256 * i;
            const uint32_t nl = e >> 5, kk = e & 31;
            const uint32_t col = n0 + nl;
            xs[kk][nl] = col < n ? to_f32<XT>(x[(size_t)col * k + (size_t)g * 32 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = ws[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = xs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const uint32_t col = n0 + tx * 4 + j;
        if (col >= n) continue;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t r = m0 + ty * 4 + i;
            if (r < m) {
                if constexpr (sizeof(OT) == 4) out[(size_t)col * m + r] = acc[i][j];
                else out[(size_t)col * m + r] = __float2bfloat16_rn(acc[i][j]);
            }
        }
    }
}

template <int TY, typename XT>
static cudaError_t gemm_simple_x(const uint8_t *w, uint32_t k, uint32_t m, const XT *x, uint32_t n,
                                 void *out, int odt, cudaStream_t s) {
    dim3 grid((m + 63) / 64, (n + 63) / 64);
    if (odt == DT_F32) gemm_simple_kernel<TY, XT, float><<<grid, 256, 0, s>>>(w, k, m, x, n, (float *)out);
    else if (odt == DT_BF16)
        gemm_simple_kernel<TY, XT, __nv_bfloat16><<<grid, 256, 0, s>>>(w, k, m, x, n, (__nv_bfloat16 *)out);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

template <int TY>
static cudaError_t gemm_simple_t(const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                                 uint32_t n, void *out, int odt, cudaStream_t s) {
    switch (xdt) {
    case DT_F32: return gemm_simple_x<TY, float>(w, k, m, (const float *)x, n, out, odt, s);
    case DT_F16: return gemm_simple_x<TY, __half>(w, k, m, (const __half *)x, n, out, odt, s);
    case DT_BF16: return gemm_simple_x<TY, __nv_bfloat16>(w, k, m, (const __nv_bfloat16 *)x, n, out, odt, s);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemm_simple(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x,
                               int xdt, uint32_t n, void *out, int odt, cudaStream_t s) {
    switch (ty) {
    case T_Q8_0: return gemm_simple_t<T_Q8_0>(w, k, m, x, xdt, n, out, odt, s);
    case T_Q4_K: return gemm_simple_t<T_Q4_K>(w, k, m, x, xdt, n, out, odt, s);
    case T_IQ2_XXS: return gemm_simple_t<T_IQ2_XXS>(w, k, m, x, xdt, n, out, odt, s);
    case T_Q2_0: return gemm_simple_t<T_Q2_0>(w, k, m, x, xdt, n, out, odt, s);
    case T_Q4_0: return gemm_simple_t<T_Q4_0>(w, k, m, x, xdt, n, out, odt, s);
    case T_IQ4_NL: return gemm_simple_t<T_IQ4_NL>(w, k, m, x, xdt, n, out, odt, s);
    case T_Q5_K: return gemm_simple_t<T_Q5_K>(w, k, m, x, xdt, n, out, odt, s);
    case T_Q6_K: return gemm_simple_t<T_Q6_K>(w, k, m, x, xdt, n, out, odt, s);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace okf
