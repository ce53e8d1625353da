// Prefill matmul on the 5th-generation tensor cores: out[n][m] = sum_k X[n][k] W[m][k]
// for N >= 9 tokens.  Replaces the reference's gemm_mm_impl tile
// (LLM/metal/Kernels.metal:226-294), which stages fp16 copies of a 64 x 32
// weight tile and a 32 x 32 activation tile for simdgroup matrices.
//
// Shape of the computation.  One CTA owns a 128-row slab of W and walks the
// tokens in blocks of 256.  Per k-block of 64:
//   - eight producer warps unpack 128 rows x 64 weights to 16-bit floats and copy
//     (or convert) 256 tokens x 64 activations, both written K-major into shared
//     memory in the 128-byte-swizzled layout the tensor core reads;
//   - one thread issues four tcgen05.mma (M = 128, N = 256, K = 16) that
//     accumulate in fp32 in tensor memory: lane = weight row, column = token;
//   - tcgen05.commit hands the stage back to the producers when the MMAs that
//     read it are done.
// Two 256-column accumulators alternate so the epilogue of one token block
// (tcgen05.ld, convert, coalesced stores along m) overlaps the next block's
// main loop.  Operands are fp16 when the activations are fp16, bf16 otherwise
// (fp32 activations are rounded to bf16); weights are decoded exactly to fp32
// first and rounded once.
//
// Every mbarrier wait is bounded (about a second); a wait that gives up records
// a code in the status word, the CTA frees its tensor memory and returns.
#include "okf_gemv_mma.cuh"
#include "okf_kernels.h"

namespace okf {

namespace tc {

constexpr uint32_t kBM = 128;           // weight rows per CTA tile (UMMA M)
constexpr uint32_t kBN = 256;           // tokens per accumulator (UMMA N)
constexpr uint32_t kBK = 64;            // k per stage: 64 x 2 bytes = one 128-byte swizzle row
constexpr uint32_t kStages = 4;
constexpr uint32_t kABytes = kBM * kBK * 2;  // 16 KB
constexpr uint32_t kBBytes = kBN * kBK * 2;  // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kProducerWarps = 8;
constexpr uint32_t kProducers = kProducerWarps * 32;
constexpr uint32_t kMmaWarp = kProducerWarps;          // warp 8
constexpr uint32_t kEpiWarp0 = kProducerWarps + 1;     // warps 9..12
constexpr uint32_t kThreads = (kProducerWarps + 1 + 4) * 32;
constexpr uint32_t kSmemBytes = 1024 /*align*/ + kStages * kStageBytes + 2048 /*grid*/ + 256 /*barriers*/;
constexpr int kStatusGemmTimeout = 3;

struct Args {
    const uint8_t *w;
    const void *x;
    void *out;
    int *status;
    uint32_t k, m, n;
    uint32_t row_bytes;
};

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows of 128
// bytes, groups of eight rows 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);        // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset: 8 rows x 128 bytes
    d |= (uint64_t)1 << 46;                          // descriptor version for this architecture
    d |= (uint64_t)2 << 61;                          // layout: 128-byte swizzle
    return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A and B of the same
// 16-bit float type (0 = fp16, 1 = bf16), both K-major, M x N as given.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t mm, uint32_t nn) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((nn >> 3) << 17) | ((mm >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <bool F16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
    if constexpr (F16) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
}

// byte offset of 16-byte chunk j of row r in a 128-byte-swizzled K-major tile
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t j) { return r * 128 + ((j ^ (r & 7)) << 4); }

template <int TY, int XDT, typename OT>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(Args p) {
    constexpr bool F16 = XDT == DT_F16;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *stage0 = smem;
    uint64_t *grid = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * kStageBytes + 2048);
    uint64_t *full = bars;                     // producers -> MMA, one per stage
    uint64_t *empty = bars + kStages;          // MMA -> producers
    uint64_t *acc_full = bars + 2 * kStages;   // MMA -> epilogue, one per accumulator
    uint64_t *acc_empty = acc_full + 2;        // epilogue -> MMA
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (p.m + kBM - 1) / kBM, n_blocks = (p.n + kBN - 1) / kBN;
    const uint32_t kblocks = p.k / kBK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) {
            mbar_init(&full[s], kProducerWarps);
            mbar_init(&empty[s], 1);
        }
        for (uint32_t a = 0; a < 2; a++) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (TY == T_IQ2_XXS) {
        for (uint32_t i = threadIdx.x; i < 256; i += kThreads) grid[i] = g_iq2xxs_grid[i];
    }
    if (warp == kMmaWarp) {
        // the whole tensor memory of the SM: two 256-column accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // work items: (m tile, token block) pairs, token block fastest so a CTA keeps its slab of W
    const uint32_t items = m_tiles * n_blocks;

    if (warp < kProducerWarps) {
        // ---------------- producers: unpack W, copy X, both into swizzled shared memory
        const uint32_t t = threadIdx.x;
        uint32_t it = 0;  // running stage counter
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x) {
            const uint32_t mt = item / n_blocks, nb = item % n_blocks;
            const uint32_t m0 = mt * kBM, n0 = nb * kBN;
            const uint32_t arow = t >> 1, ahalf = t & 1;  // thread t unpacks 32 weights of row arow
            const uint32_t wrow = min(m0 + arow, p.m - 1);
            const uint8_t *wp = p.w + (size_t)wrow * p.row_bytes;
            const bool arow_live = m0 + arow < p.m;
            for (uint32_t kb = 0; kb < kblocks; kb++, it++) {
                const uint32_t s = it % kStages, use = it / kStages;
                if (use > 0 && !mbar_wait(&empty[s], (use - 1) & 1, abort_flag, p.status, kStatusGemmTimeout)) goto done;
                uint8_t *sa = stage0 + (size_t)s * kStageBytes, *sb = sa + kABytes;
                {   // A: 32 weights -> four 16-byte chunks of row arow
                    float v[32];
                    decode32<TY>(wp, kb * 2 + ahalf, v, grid);
#pragma unroll
                    for (int c4 = 0; c4 < 4; c4++) {
                        uint4 q;
                        q.x = arow_live ? pack16<F16>(v[8 * c4], v[8 * c4 + 1]) : 0u;
                        q.y = arow_live ? pack16<F16>(v[8 * c4 + 2], v[8 * c4 + 3]) : 0u;
                        q.z = arow_live ? pack16<F16>(v[8 * c4 + 4], v[8 * c4 + 5]) : 0u;
                        q.w = arow_live ? pack16<F16>(v[8 * c4 + 6], v[8 * c4 + 7]) : 0u;
                        *reinterpret_cast<uint4 *>(sa + swz(arow, ahalf * 4 + c4)) = q;
                    }
                }
                // B: 256 tokens x 8 chunks, eight chunks per thread
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint32_t q = t + kProducers * i;
                    const uint32_t row = q >> 3, j = q & 7;
                    const uint32_t tok = n0 + row;
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (tok < p.n) {
                        const size_t e = (size_t)tok * p.k + (size_t)kb * kBK + j * 8;
                        if constexpr (XDT == DT_F32) {
                            const float4 f0 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + e));
                            const float4 f1 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + e) + 1);
                            v.x = pack16<false>(f0.x, f0.y); v.y = pack16<false>(f0.z, f0.w);
                            v.z = pack16<false>(f1.x, f1.y); v.w = pack16<false>(f1.z, f1.w);
                        } else {
                            v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.x) + e));
                        }
                    }
                    *reinterpret_cast<uint4 *>(sb + swz(row, j)) = v;
                }
                fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[s]);
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer: one thread
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(F16 ? 0u : 1u, kBM, kBN);
            uint32_t it = 0, tile = 0;
            for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, tile++) {
                const uint32_t acc = tile & 1, acc_use = tile >> 1;
                if (acc_use > 0 && !mbar_wait(&acc_empty[acc], (acc_use - 1) & 1, abort_flag, p.status, kStatusGemmTimeout)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                bool ok = true;
                for (uint32_t kb = 0; kb < kblocks; kb++, it++) {
                    const uint32_t s = it % kStages, use = it / kStages;
                    if (!mbar_wait(&full[s], use & 1, abort_flag, p.status, kStatusGemmTimeout)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(stage0 + (size_t)s * kStageBytes), sb = sa + kABytes;
                    const uint64_t da = smem_desc(sa), db = smem_desc(sb);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < kBK / 16; k4++) {
                        // 16 k = 32 bytes further along the swizzled 128-byte row
                        umma(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb | k4) != 0 ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[acc]);
            }
        }
    } else {
        // ---------------- epilogue: four warps, warp q reads tensor-memory lanes 32q .. 32q + 31
        const uint32_t q = warp & 3;  // a warp may only touch the lane quarter given by warp id % 4
        uint32_t tile = 0;
        for (uint32_t item = blockIdx.x; item < items; item += gridDim.x, tile++) {
            const uint32_t mt = item / n_blocks, nb = item % n_blocks;
            const uint32_t acc = tile & 1, acc_use = tile >> 1;
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&acc_full[acc], acc_use & 1, abort_flag, p.status, kStatusGemmTimeout);
            if (!__shfl_sync(0xffffffffu, ok, 0)) break;
            tc_fence_after();
            const uint32_t row = mt * kBM + q * 32 + lane;
            OT *out = reinterpret_cast<OT *>(p.out);
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < kBN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((q * 32) << 16) + acc * kBN + c0, r);
                tmem_ld_wait();
                if (row < p.m) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const uint32_t tok = nb * kBN + c0 + j;
                        if (tok < p.n) {
                            const float f = __uint_as_float(r[j]);
                            if constexpr (sizeof(OT) == 4) out[(size_t)tok * p.m + row] = f;
                            else out[(size_t)tok * p.m + row] = __float2bfloat16_rn(f);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
    }
done:
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

template <int TY, int XDT, typename OT>
static cudaError_t launch(const Args &a, cudaStream_t s, int sms, int dev) {
    static bool attr_set[64] = {};  // the opt-in is per device
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TY, XDT, OT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const uint32_t items = ((a.m + kBM - 1) / kBM) * ((a.n + kBN - 1) / kBN);
    const uint32_t grid = items < (uint32_t)sms ? items : (uint32_t)sms;
    gemm_tc_kernel<TY, XDT, OT><<<grid, kThreads, kSmemBytes, s>>>(a);
    return cudaGetLastError();
}

template <int TY, int XDT>
static cudaError_t launch_o(const Args &a, int odt, cudaStream_t s, int sms, int dev) {
    if (odt == DT_F32) return launch<TY, XDT, float>(a, s, sms, dev);
    if (odt == DT_BF16) return launch<TY, XDT, __nv_bfloat16>(a, s, sms, dev);
    return cudaErrorInvalidValue;
}

template <int TY>
static cudaError_t launch_x(const Args &a, int xdt, int odt, cudaStream_t s, int sms, int dev) {
    switch (xdt) {
    case DT_F16: return launch_o<TY, DT_F16>(a, odt, s, sms, dev);
    case DT_BF16: return launch_o<TY, DT_BF16>(a, odt, s, sms, dev);
    case DT_F32: return launch_o<TY, DT_F32>(a, odt, s, sms, dev);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace tc

bool gemm_tc_supported(int ty, uint32_t k, uint32_t m, const void *w, const void *x, int xdt, uint32_t n) {
    if (ty != T_Q4_K && ty != T_Q8_0 && ty != T_Q2_0 && ty != T_IQ2_XXS) return false;
    if (k % 64 || m == 0 || n == 0) return false;
    if ((uintptr_t)x % 16 || (k * (xdt == DT_F32 ? 4 : 2)) % 16) return false;
    if (ty == T_Q4_K && (uintptr_t)w % 16) return false;
    return true;
}

cudaError_t launch_gemm_tc(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                           uint32_t n, void *out, int odt, int *status, cudaStream_t s, int sms, int dev) {
    tc::Args a;
    a.w = w; a.x = x; a.out = out; a.status = status; a.k = k; a.m = m; a.n = n;
    a.row_bytes = (k / block_elems(ty)) * block_bytes(ty);
    switch (ty) {
    case T_Q4_K: return tc::launch_x<T_Q4_K>(a, xdt, odt, s, sms, dev);
    case T_Q8_0: return tc::launch_x<T_Q8_0>(a, xdt, odt, s, sms, dev);
    case T_Q2_0: return tc::launch_x<T_Q2_0>(a, xdt, odt, s, sms, dev);
    case T_IQ2_XXS: return tc::launch_x<T_IQ2_XXS>(a, xdt, odt, s, sms, dev);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace okf
