// The small operators that sit right beside the quantized linears in the engines'
// command streams: embedding-row gather, arg-max over logits rows, residual add +
// RMS norm, SiLU gating, and the clamp / fake-quant around gemma's linears.
//
// Replaces MetalEnc.embedBatch (LLM/Base/MetalEnc.swift:1096-1147; kernels embed_batch,
// q4_0_embed_batch, ... LLM/metal/Kernels.metal:3687-3760), argmax_rows
// (Kernels.metal:2756-2794), add_rmsnorm_batch / rmsnorm_batch (Kernels.metal:2811-2864),
// silu_mul (Kernels.metal:3280-3285) and srq_to / srq_inplace (Kernels.metal:4743-4767).
// All of them are bound by memory, not arithmetic: one pass over their operands with
// 16-byte accesses where the shapes allow it.
#include "okf_internal.h"
#include "okf_kernels.h"

namespace okf {

// ---- embedding rows ---------------------------------------------------------------
// out[n][k] = dequant(row ids[n])[k], bit for bit what the block decoders give.  One
// thread unpacks one granule of 32 weights; an id outside [0, rows) gives a row of zeros
// and code 8 in the device status word.
constexpr int kStatusBadId = 8;
template <int TY>
__global__ void __launch_bounds__(256) embed_kernel(const uint8_t *__restrict__ w, const int *__restrict__ ids,
                                                    uint32_t k, uint32_t n, uint32_t rows, float *__restrict__ out,
                                                    int *bad) {
    __shared__ uint64_t grid_s[256];
    if constexpr (TY == T_IQ2_XXS) {
        grid_s[threadIdx.x] = g_iq2xxs_grid[threadIdx.x];
        __syncthreads();
    }
    const uint32_t gpr = k / 32;  // granules per row
    const size_t row_bytes = (size_t)(k / Geom<TY>::per) * Geom<TY>::bytes;
    const uint64_t total = (uint64_t)n * gpr, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total; g += stride) {
        const uint32_t tok = (uint32_t)(g / gpr), gran = (uint32_t)(g % gpr);
        const int id = ids[tok];
        float v[32];
        if (id >= 0 && (uint32_t)id < rows) {
            decode32<TY>(w + (size_t)id * row_bytes, gran, v, grid_s);
        } else {
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = 0.f;
            if (bad && gran == 0) atomicExch(bad, kStatusBadId);
        }
        float4 *o = reinterpret_cast<float4 *>(out + (size_t)tok * k + (size_t)gran * 32);
#pragma unroll
        for (int i = 0; i < 8; i++) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
}

template <int TY>
static cudaError_t embed_t(const uint8_t *w, const int *ids, uint32_t k, uint32_t n, uint32_t rows, float *out, int *bad,
                           cudaStream_t s) {
    const uint64_t total = (uint64_t)n * (k / 32);
    if (total == 0) return cudaSuccess;
    uint64_t blocks = (total + 255) / 256;
    if (blocks > 148ull * 32) blocks = 148ull * 32;
    embed_kernel<TY><<<(unsigned)blocks, 256, 0, s>>>(w, ids, k, n, rows, out, bad);
    return cudaGetLastError();
}

static cudaError_t launch_embed(int ty, const uint8_t *w, const int *ids, uint32_t k, uint32_t n, uint32_t rows, float *out,
                                int *bad, cudaStream_t s) {
    switch (ty) {
    case T_Q8_0: return embed_t<T_Q8_0>(w, ids, k, n, rows, out, bad, s);
    case T_Q4_K: return embed_t<T_Q4_K>(w, ids, k, n, rows, out, bad, s);
    case T_IQ2_XXS: return embed_t<T_IQ2_XXS>(w, ids, k, n, rows, out, bad, s);
    case T_Q2_0: return embed_t<T_Q2_0>(w, ids, k, n, rows, out, bad, s);
    case T_Q4_0: return embed_t<T_Q4_0>(w, ids, k, n, rows, out, bad, s);
    case T_IQ4_NL: return embed_t<T_IQ4_NL>(w, ids, k, n, rows, out, bad, s);
    case T_Q5_K: return embed_t<T_Q5_K>(w, ids, k, n, rows, out, bad, s);
    case T_Q6_K: return embed_t<T_Q6_K>(w, ids, k, n, rows, out, bad, s);
    default: return cudaErrorInvalidValue;
    }
}

// ---- arg-max over rows --------------------------------------------------------------
// One CTA per row.  The largest value wins, ties go to the lower index, NaNs never win
// (an all-NaN row gives 0): what the host arg-max it replaces does.
__device__ __forceinline__ void argmax_take(float &bv, int &bi, float ov, int oi) {
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

__global__ void __launch_bounds__(512) argmax_rows_kernel(const float *__restrict__ x, int *__restrict__ out, uint32_t n) {
    __shared__ float bestv[16];
    __shared__ int besti[16];
    const float *row = x + (size_t)blockIdx.x * n;
    float bv = -INFINITY;
    int bi = 0;
    // 16-byte loads where the row allows them; each thread walks its indices in rising
    // order, so a strict > keeps the lowest index among its equals
    const bool vec = (n & 3u) == 0 && ((uintptr_t)row & 15u) == 0;
    if (vec) {
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
        for (uint32_t i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const float4 v = __ldg(r4 + i);
            if (v.x > bv) { bv = v.x; bi = (int)(4 * i); }
            if (v.y > bv) { bv = v.y; bi = (int)(4 * i + 1); }
            if (v.z > bv) { bv = v.z; bi = (int)(4 * i + 2); }
            if (v.w > bv) { bv = v.w; bi = (int)(4 * i + 3); }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = row[i];
            if (v > bv) { bv = v; bi = (int)i; }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        argmax_take(bv, bi, __shfl_down_sync(0xffffffffu, bv, off), __shfl_down_sync(0xffffffffu, bi, off));
    if ((threadIdx.x & 31) == 0) {
        bestv[threadIdx.x >> 5] = bv;
        besti[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < blockDim.x / 32; w++) argmax_take(bv, bi, bestv[w], besti[w]);
        out[blockIdx.x] = bi;
    }
}

// ---- residual add + RMS norm ----------------------------------------------------------
// x[row] += r[row] (skipped when r is null); y[row] = x[row] * scale * w with
// scale = 1 / sqrt(mean(x^2) + eps).  One CTA per row; the row is read from HBM once
// (the second sweep hits L1 / L2).
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(float *x, const float *__restrict__ r,
                                                          const float *__restrict__ w, float *y, uint32_t n,
                                                          float eps, uint32_t x_stride, uint32_t y_stride) {
    __shared__ float part[8];
    float *xr = x + (size_t)blockIdx.x * x_stride;
    const float *rr = r ? r + (size_t)blockIdx.x * x_stride : nullptr;
    float *yr = y + (size_t)blockIdx.x * y_stride;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float v = xr[i];
        if (rr) {
            v += rr[i];
            xr[i] = v;
        }
        ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += part[i];
    const float scale = 1.f / sqrtf(tot / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = xr[i] * scale * w[i];
}

// ---- SiLU gating: a = silu(a) * b ------------------------------------------------------
__global__ void __launch_bounds__(256) silu_mul_kernel(float *a, const float *__restrict__ b, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = a[i];
        a[i] = v / (1.f + expf(-v)) * b[i];
    }
}

// ---- clamp / fake-quant around a linear -------------------------------------------------
// scale != 0: clamp(round_half_even(x * (1 / scale)), -128, 127) * scale; else clamp to
// [lo, hi] without rounding (SRQ.apply, LLM/Gemma/Gemma4Quant.swift:413-427).  Every step
// rounds once, as the Swift code does, so the result is bit-exact.
__global__ void __launch_bounds__(256) srq_kernel(const float *src, float *dst, size_t n, float scale, float lo, float hi) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const float inv = scale != 0.f ? __fdiv_rn(1.f, scale) : 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = src[i];
        if (scale != 0.f) {
            const float q = rintf(__fmul_rn(v, inv));
            dst[i] = __fmul_rn(fminf(fmaxf(q, -128.f), 127.f), scale);
        } else {
            dst[i] = fminf(fmaxf(v, lo), hi);
        }
    }
}

static unsigned flat_blocks(size_t n) {
    size_t b = (n + 255) / 256;
    return (unsigned)(b > 148ull * 16 ? 148ull * 16 : (b ? b : 1));
}

}  // namespace okf

using namespace okf;

static bool srq_active(const okf_srq_side *s) { return s && (s->scale != 0.f || s->lo < s->hi); }

extern "C" {

int okf_embed_batch(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t rows,
                    const int32_t *ids, uint32_t n, float *out, okf_stream stream) {
    int rc = check_tensor(ctx, type, w, woff, k, rows);
    if (rc) return rc;
    if (!ids || !out) return OKF_E_ARG;
    if (k % 32 || (uintptr_t)out % 16 || (uintptr_t)ids % 4) return OKF_E_ALIGN;
    if (n == 0) return OKF_OK;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    cudaError_t e = launch_embed(type, w->dptr + woff, ids, k, n, rows, out, ctx->dev_status, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

int okf_argmax_rows(okf_ctx *ctx, const float *x, uint32_t n, uint32_t rows, int32_t *out, okf_stream stream) {
    if (!ctx || !x || !out) return OKF_E_ARG;
    if (n == 0) return OKF_E_SHAPE;
    if (rows == 0) return OKF_OK;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    argmax_rows_kernel<<<rows, 512, 0, (cudaStream_t)stream>>>(x, out, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

int okf_add_rmsnorm(okf_ctx *ctx, float *x, const float *r, const float *weight, float *y, uint32_t n, uint32_t rows,
                    float eps, uint32_t x_stride, uint32_t y_stride, okf_stream stream) {
    if (!ctx || !x || !weight || !y) return OKF_E_ARG;
    if (n == 0 || x_stride < n || y_stride < n) return OKF_E_SHAPE;
    if (rows == 0) return OKF_OK;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    add_rmsnorm_kernel<<<rows, 256, 0, (cudaStream_t)stream>>>(x, r, weight, y, n, eps, x_stride, y_stride);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

int okf_silu_mul(okf_ctx *ctx, float *a, const float *b, size_t n, okf_stream stream) {
    if (!ctx || !a || !b) return OKF_E_ARG;
    if (n == 0) return OKF_OK;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    silu_mul_kernel<<<flat_blocks(n), 256, 0, (cudaStream_t)stream>>>(a, b, n);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

int okf_srq(okf_ctx *ctx, const float *src, float *dst, size_t n, const okf_srq_side *side, okf_stream stream) {
    if (!ctx || !src || !dst || !side) return OKF_E_ARG;
    if (n == 0) return OKF_OK;
    if (!srq_active(side)) {
        if (src == dst) return OKF_OK;
        DeviceGuard g0(ctx->device);
        cudaError_t e0 = cudaMemcpyAsync(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice, (cudaStream_t)stream);
        return e0 == cudaSuccess ? OKF_OK : cuda_fail(ctx, e0);
    }
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    srq_kernel<<<flat_blocks(n), 256, 0, (cudaStream_t)stream>>>(src, dst, n, side->scale, side->lo, side->hi);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

int okf_linear(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m, const float *x,
               uint32_t n, float *out, const okf_srq_side *in, const okf_srq_side *outs, float *scratch,
               okf_stream stream) {
    if (!ctx || !x || !out) return OKF_E_ARG;
    if (ctx->par_open) return OKF_E_ARG;  // three dependent launches: not inside a parallel region
    const float *input = x;
    if (srq_active(in)) {
        if (!scratch) return OKF_E_ARG;
        int rc = okf_srq(ctx, x, scratch, (size_t)n * k, in, stream);
        if (rc) return rc;
        input = scratch;
    }
    int rc = okf_gemm(ctx, type, w, woff, k, m, input, OKF_F32, n, out, OKF_F32, stream);
    if (rc) return rc;
    if (srq_active(outs)) rc = okf_srq(ctx, out, out, (size_t)n * m, outs, stream);
    return rc;
}

}  // extern "C"
