// Building blocks of the decode matvec (1..8 activation columns): mbarrier /
// bulk-copy pipeline primitives, launch arguments.
//
// Data path.  Weights stream from HBM into a shared-memory ring with bulk
// asynchronous copies (cp.async.bulk, completion counted on an mbarrier) issued
// by one producer thread, so a CTA has its whole share of a small matrix in
// flight at once.  Consumer warps feed the blocks from shared memory to the
// integer tensor cores (mma.sync m16n8k32 on bytes, s32 sums); block scales are
// applied to the sums afterwards.
//
// MMA operand layout (A = weights, 16 rows; B = activations, 8 columns): thread
// (g = lane / 4, c = lane % 4) holds A rows g and g + 8 and B column g, both at
// the k-slots that belong to c.  A dot product does not care which real k a slot
// stands for as long as A and B agree, so the kernels hand every thread the k
// that are contiguous in memory for it.
//
// Every wait on an mbarrier is bounded: after about a second without progress
// the thread records a code in the status word and raises the CTA's abort flag;
// the other waits see the flag and give up too, and the warps walk through the
// rest of their loops without waiting, so every barrier among them still matches.
#pragma once
#include "okf_blocks.cuh"

namespace okf {

// Up to kGemvSegs matrices of the same type and K that multiply the same x share
// one launch: their tiles are numbered through, segment after segment.
constexpr int kGemvSegs = 4;
constexpr int kMaxRanks = 8;
#ifndef OKF_GEMV_WARPS
#define OKF_GEMV_WARPS 8
#endif
constexpr int kGemvWarps = OKF_GEMV_WARPS;         // consumer warps
constexpr int kGemvThreads = (kGemvWarps + 1) * 32;  // + one producer warp
constexpr int kGemvThreadsMax = kGemvThreads + 32;    // + one warp that announces the previous exchange (row shards only)
constexpr long long kWaitCycles = 2000000000LL;  // about one second of SM clock
constexpr uint32_t kSpinLimit = 1u << 16;          // polls when draining on the way out
constexpr int kStatusFullTimeout = 1, kStatusEmptyTimeout = 2, kStatusGatherTimeout = 4;
// Row-sharded matrices on several GPUs: every rank stores its rows straight into
// every rank's copy of the whole output (peer-mapped pointers), counts itself in on
// every rank, and the launch ends on a rank only when all ranks have counted in.
struct GemvGather {
    uint32_t nranks;                       // 0: single GPU, `out` below is used
    uint32_t m_total[kGemvSegs];           // rows of the whole matrix
    uint32_t row_first[kGemvSegs];         // this rank's first row in it
    float *out[kGemvSegs][kMaxRanks];      // rank r's [n][m_total] buffer as mapped here
    uint32_t *arrivals[kMaxRanks];         // rank r's arrival counter, as mapped here: one count per rank and exchange
    uint32_t *epoch;                       // local, two words: {count the local counter reaches when the exchanges
                                           // launched so far are complete, reserved}
    uint32_t rank;
    // The exchange launched before this one (null: none): its local counter and epoch
    // words.  The consumers wait for it to complete before they read x.
    const uint32_t *wait_arrivals;
    const uint32_t *wait_epoch;
    // The exchange launched before this one whose rows have not been announced yet
    // (sig_nranks = 0: none): the counters to add 1 to, on every rank.  A system-wide
    // fence takes microseconds on this part, so the kernel that stores the rows does not
    // fence; a spare warp of the NEXT launch does, once that kernel is complete and while
    // the consumers of this launch are already at work.
    uint32_t *sig_arrivals[kMaxRanks];
    uint32_t sig_nranks;
};

// Announce a complete exchange: every store of the kernel that ran it happens before
// this thread's fence (the kernel is complete), the fence orders them before the counts.
__device__ __forceinline__ void gather_signal(uint32_t *const *arrivals, uint32_t nranks) {
    __threadfence_system();
    for (uint32_t rk = 0; rk < nranks; rk++)
        asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;" ::"l"(arrivals[rk]) : "memory");
}

// Wait, bounded, until the local arrival counter has reached the count published
// for the exchanges launched so far.  One thread calls it; returns false on a timeout.
__device__ __forceinline__ bool gather_wait(const uint32_t *arrivals, const uint32_t *epoch, int *status) {
    const uint32_t target = *reinterpret_cast<const volatile uint32_t *>(epoch);
    const long long t_start = clock64();
    for (;;) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(arrivals) : "memory");
        if ((int32_t)(seen - target) >= 0) return true;
        if (clock64() - t_start > kWaitCycles) {
            if (status) atomicExch(status, kStatusGatherTimeout);
            return false;
        }
        __nanosleep(20);
    }
}
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
    uint32_t m, tile0, tile1, index;
};
__device__ __forceinline__ GemvSeg gemv_segment(const GemvArgs &p, uint32_t tile) {
    GemvSeg s = {p.w[0], p.out[0], p.m[0], 0u, p.tile_end[0], 0u};
#pragma unroll
    for (int i = 1; i < kGemvSegs; i++)
        if (tile >= p.tile_end[i - 1]) s = {p.w[i], p.out[i], p.m[i], p.tile_end[i - 1], p.tile_end[i], (uint32_t)i};
    return s;
}


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
// The same question without ever blocking.
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if it gave up or the CTA is aborting.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *status, int code) {
    if (mbar_try_wait(bar, parity)) return true;  // the usual case: the phase is over
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

// The same for the producer thread, which is in no hurry: between polls it sleeps, so that
// its spinning does not take issue slots from the two consumer warps that share its
// scheduler.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                                  int *status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        __nanosleep(200);
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

// Programmatic dependent launch: let the next kernel in the stream start its
// weight prefetch while this one drains, and wait for the previous kernel's
// results before touching activations or outputs.  Both are no-ops when the
// launch does not carry the attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

// byte b (0..255) of `v` as a float, without the slow int-to-float unit
__device__ __forceinline__ float byte_to_f32(uint32_t v, int which) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 | which)) - 8388608.f;
}

}  // namespace okf
