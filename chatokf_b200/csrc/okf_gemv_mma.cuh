// Building blocks of the decode matvec (1..8 activation columns): mbarrier /
// bulk-copy pipeline primitives, the warp MMA, activation fragments.
//
// Data path.  Weights stream from HBM into a shared-memory ring with bulk
// asynchronous copies (cp.async.bulk, completion counted on an mbarrier) issued
// by one producer thread, so a CTA has its whole share of a small matrix in
// flight at once.  Consumer warps unpack the blocks from shared memory into
// exact small integers held in fp16 and multiply them with the activations on
// the tensor cores (mma.sync m16n8k16, fp32 accumulate); block scales are
// applied to fp32 partial sums.
//
// MMA operand layout (A = weights 16 rows x 16 k, B = activations 16 k x 8
// columns): thread (g = lane / 4, c = lane % 4) holds A rows g and g + 8 and B
// column g, both at k-slots {2c, 2c+1, 2c+8, 2c+9}.  A dot product does not care
// which real k a slot stands for as long as A and B agree, so thread c simply
// owns k in [64c, 64c + 64) of every 256-wide unit of a row.
//
// Every wait on an mbarrier is bounded: after about a second without progress
// the thread records a code in the status word, raises the CTA's abort flag and
// leaves; the other threads see the flag in their own waits and leave too.
#pragma once
#include "okf_blocks.cuh"

namespace okf {

// Up to kGemvSegs matrices of the same type and K that multiply the same x share
// one launch: their tiles are numbered through, segment after segment.
constexpr int kGemvSegs = 4;
struct GemvArgs {
    const uint8_t *w[kGemvSegs];
    float *out[kGemvSegs];
    uint32_t m[kGemvSegs];
    uint32_t tile_end[kGemvSegs];  // running total of ceil(m / 16)
    const void *x;
    int *status;     // device status word: 0 = ok, else a wait gave up (see kStatus*)
    uint32_t k, n;
    uint32_t nunit;  // 256-wide units per row
    uint32_t tiles;  // all segments together
    uint32_t cb;     // units per chunk (one ring stage holds 16 rows x cb units)
    uint32_t nchunk; // chunks per tile
    uint32_t row_bytes;
};

// The segment a tile belongs to.
struct GemvSeg {
    const uint8_t *w;
    float *out;
    uint32_t m, tile0, tile1;
};
__device__ __forceinline__ GemvSeg gemv_segment(const GemvArgs &p, uint32_t tile) {
    GemvSeg s = {p.w[0], p.out[0], p.m[0], 0u, p.tile_end[0]};
#pragma unroll
    for (int i = 1; i < kGemvSegs; i++)
        if (tile >= p.tile_end[i - 1]) s = {p.w[i], p.out[i], p.m[i], p.tile_end[i - 1], p.tile_end[i]};
    return s;
}

constexpr int kGemvWarps = 8;                      // consumer warps
constexpr int kGemvThreads = (kGemvWarps + 1) * 32;  // + one producer warp
constexpr long long kWaitCycles = 2000000000LL;  // about one second of SM clock
constexpr uint32_t kSpinLimit = 1u << 16;          // polls when draining on the way out
constexpr int kStatusFullTimeout = 1, kStatusEmptyTimeout = 2;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if it gave up or the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *status, int code) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) break;
    }
    *abort_flag = 1;
    if (status) atomicExch(status, code);
    return false;
}

// One-dimensional bulk copy global -> shared; both addresses and the size are
// multiples of 16 bytes.  Completion is reported to `bar` in bytes.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t h2_bcast(float v) { return pack_h2(v, v); }

// Programmatic dependent launch: let the next kernel in the stream start its
// weight prefetch while this one drains, and wait for the previous kernel's
// results before touching activations or outputs.  Both are no-ops when the
// launch does not carry the attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- activations in shared memory -----------------------------------------------
// A slice of x (all effective columns, `nu` units of 256 k) is converted to fp16
// once and kept in shared memory in the order the MMA wants it: the 64 values
// that thread c of a quad owns in unit u of effective column e start at
//     e * es + u * kXsUnit + c * 144          (es % 128 == 64)
// so the eight lanes that read together (two columns or rows x four c) hit
// eight different 16-byte bank groups.
//
// Effective columns: fp16 / bf16 activations have one per real column; fp32
// activations have two, x = hi + lo with hi = fp16(x) (22 significant bits in
// all): column e is hi of x[e], column lo_off + e is lo.  Magnitudes are
// clamped to the fp16 range first.
constexpr uint32_t kXsUnit = 4 * 144;

__host__ __device__ inline uint32_t xs_col_stride(uint32_t cb) {
    const uint32_t raw = cb * kXsUnit;
    return raw + ((64u + 128u - raw % 128u) % 128u);
}

template <int XDT>
__device__ __forceinline__ float load_x_as_f32(const void *x, size_t idx) {
    if constexpr (XDT == DT_F16) return __half2float(__ldg(reinterpret_cast<const __half *>(x) + idx));
    else if constexpr (XDT == DT_BF16) return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(x) + idx));
    else return __ldg(reinterpret_cast<const float *>(x) + idx);
}

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// Cooperative load of the panel of units [u_first, u_first + nu) by `nthreads`
// threads.  fp16 activations that are 16-byte aligned go global -> shared with
// asynchronous 16-byte copies; everything else is converted in registers.
// The caller waits with cp_async_wait_all() and a barrier.
template <int XDT>
__device__ __forceinline__ void stage_x_panel(uint8_t *xs, uint32_t es, const void *x, uint32_t kdim,
                                              uint32_t n, uint32_t lo_off, uint32_t u_first, uint32_t nu,
                                              uint32_t tid, uint32_t nthreads) {
    const uint32_t k0 = u_first * 256;
    if constexpr (XDT == DT_F16) {
        if (((uintptr_t)x % 16) == 0) {
            const uint32_t pieces_per_col = nu * 32;  // 16-byte pieces of eight k
            for (uint32_t i = tid; i < n * pieces_per_col; i += nthreads) {
                const uint32_t col = i / pieces_per_col, pc = i % pieces_per_col;
                const uint32_t u = pc >> 5, c = (pc >> 3) & 3, q = pc & 7;
                cp_async16(xs + col * es + u * kXsUnit + c * 144 + q * 16,
                           reinterpret_cast<const __half *>(x) + (size_t)col * kdim + k0 + pc * 8);
            }
            return;
        }
    }
    const uint32_t pairs_per_col = nu * 128;  // two k per item
    for (uint32_t i = tid; i < n * pairs_per_col; i += nthreads) {
        const uint32_t col = i / pairs_per_col, kk = (i % pairs_per_col) * 2;
        const uint32_t u = kk >> 8, c = (kk >> 6) & 3, r = kk & 63;
        const uint32_t off = u * kXsUnit + c * 144 + r * 2;
        const size_t src = (size_t)col * kdim + k0 + kk;
        float a = load_x_as_f32<XDT>(x, src), b = load_x_as_f32<XDT>(x, src + 1);
        a = fminf(fmaxf(a, -65504.f), 65504.f);
        b = fminf(fmaxf(b, -65504.f), 65504.f);
        const uint32_t hi = pack_h2(a, b);
        *reinterpret_cast<uint32_t *>(xs + col * es + off) = hi;
        if constexpr (XDT == DT_F32) {
            const __half2 h = *reinterpret_cast<const __half2 *>(&hi);
            *reinterpret_cast<uint32_t *>(xs + (lo_off + col) * es + off) =
                pack_h2(a - __low2float(h), b - __high2float(h));
        }
    }
}

// byte b (0..255) of `v` as a float, without the slow int-to-float unit
__device__ __forceinline__ float byte_to_f32(uint32_t v, int which) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 | which)) - 8388608.f;
}

}  // namespace okf
