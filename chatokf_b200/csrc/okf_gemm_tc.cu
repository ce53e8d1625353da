// Prefill matmul on the 5th-generation tensor cores: out[n][m] = sum_k X[n][k] W[m][k]
// for N >= 9 tokens.  Replaces the reference's gemm_mm_impl tile
// (LLM/metal/Kernels.metal:226-294), which stages fp16 copies of a 64 x 32
// weight tile and a 32 x 32 activation tile for simdgroup matrices.
//
// Shape of the computation.  One work item is a 128-row slab of W against one
// block of 256 tokens or two such blocks at once, so that every unpacked weight
// tile feeds two accumulators.  Per k-block of 64:
//   - the activation tile(s), 256 tokens x 64 k each, come by TMA through a tensor
//     map of X, already in the 128-byte-swizzled K-major layout the tensor core
//     reads (fp32 activations are converted by eight warps instead);
//   - two groups of eight warps, taking the k-blocks in turn, unpack 128 rows x 64
//     weights to 16-bit floats into the same layout; weight bytes are fetched one
//     or two turns ahead.  (Bringing Q4_K slabs in by TMA as stored, 128 rows x one
//     144-byte block per copy into a ring of their own, was tried and was slower.)
//   - one thread issues four tcgen05.mma (M = 128, N = 256, K = 16) per token block
//     that accumulate in fp32 in tensor memory: lane = weight row, column = token;
//   - tcgen05.commit hands the stage back to the producers when the MMAs that
//     read it are done.
// The two 256-column accumulators of tensor memory either serve the two token
// blocks of one item or alternate between items, so an epilogue (tcgen05.ld,
// convert, coalesced stores along m) overlaps the next main loop.  Operands are
// fp16 when the activations are fp16, bf16 otherwise (fp32 activations are
// rounded to bf16); weights are decoded exactly to fp32 first and rounded once.
//
// Every mbarrier wait is bounded (about a second); a wait that gives up records
// a code in the status word, the CTA frees its tensor memory and returns.
#include <type_traits>
#include <cuda.h>

#include <cstring>
#include "okf_gemv_mma.cuh"
#include "okf_internal.h"
#include "okf_kernels.h"

namespace okf {

namespace tc {

constexpr uint32_t kBM = 128;           // weight rows per CTA tile (UMMA M)
constexpr uint32_t kBN = 256;           // tokens per accumulator (UMMA N)
constexpr uint32_t kBK = 64;            // k per stage: 64 x 2 bytes = one 128-byte swizzle row
constexpr uint32_t kABytes = kBM * kBK * 2;  // 16 KB
constexpr uint32_t kBBytes = kBN * kBK * 2;  // 32 KB per 256 tokens
// Two rings.  With one token block per item: four stages of A (16 KB) and of B (32 KB).  With
// two blocks a B stage is 64 KB: three of them and two of A, so that a B tile has two MMA
// periods to arrive while the next A tile only has to be stored (IQ2_XXS, which also keeps its
// codebook in shared memory, stays with two B stages).
constexpr uint32_t kAWarps = 8;                        // warps 0..7 unpack weights (A tile)
constexpr uint32_t kBWarps = 8;                        // warps 8..15: fp32 activations: convert the B tile;
                                                       // 16-bit activations: a second unpacking group
constexpr uint32_t kProducerWarps = kAWarps + kBWarps;
constexpr uint32_t kTmaWarp = kProducerWarps;          // warp 16: one thread hands B tiles to the copy engine
constexpr uint32_t kMmaWarp = kProducerWarps + 1;      // warp 17
constexpr uint32_t kThreads = (kProducerWarps + 2 + 4) * 32;  // + four epilogue warps
constexpr uint32_t kMaxRing = 4;                                      // stages a ring may have
constexpr uint32_t kBarRegion = 256;                                  // barriers, tensor-memory slot, abort flag
template <int TY, int NACC> struct Rings {
    static constexpr uint32_t a_stages = NACC == 2 ? 2 : 4;
    static constexpr uint32_t b_stages = NACC == 2 ? (TY == T_IQ2_XXS ? 2 : 3) : 4;
    static constexpr uint32_t a_bytes = a_stages * kABytes, b_stage = NACC * kBBytes, b_bytes = b_stages * b_stage;
    static constexpr uint32_t grid_bytes = TY == T_IQ2_XXS ? 2048 : 0;
    static constexpr uint32_t smem = 1024 /*align*/ + a_bytes + b_bytes + grid_bytes + kBarRegion;
};
constexpr int kStatusGemmTimeout = 3;

// Output element type that stands for "fp32, stored into every rank's whole output" (row shards).
struct GatherF32 { float v; };
template <typename OT> constexpr bool kIsGather = false;
template <> constexpr bool kIsGather<GatherF32> = true;

struct Args {
    const uint8_t *w;
    const void *x;
    void *out;
    int *status;
    uint32_t k, m, n;
    uint32_t row_bytes;
    uint32_t ksplit;   // work items per (slab, token group): each takes a range of k-blocks
    float *partial;    // ksplit > 1: fp32 partial results [ksplit][n][m], summed by a second kernel
    // ksplit == 1: the last tail_items (slab, token block) items -- what is left after
    // the full waves -- are cut into tail_parts runs of tail_tok tokens, one per CTA
    uint32_t tail_items, tail_tok, tail_parts;
};
// Row shards: where results go instead of Args::out.  `nout` buffers (every rank's copy of
// the whole output as mapped here), element (token, row) at [token * out_ld + out_row0 + row].
// A parameter of its own: the main loops compile to slower code (fewer registers, 12 % less
// throughput measured) when Args grows.
struct Outs {
    uint32_t nout, out_ld, out_row0;
    void *outs[8];
    uint32_t *epoch;      // the local count the exchange is complete at goes up by epoch_inc
    uint32_t epoch_inc;
};

// One piece of work of a CTA: rows [mt * 128, +128) x tokens [n0, n0 + ntok) x k-blocks [kb0, kb1).
struct Work {
    uint32_t mt, n0, ntok, kb0, kb1, part;
};

// The j-th piece of work of this CTA; false when there is none.  Whole items go
// round-robin over the CTAs; with a tail split every CTA then takes one run of
// tokens of one of the left-over items (NACC == 1 only).
template <int NACC>
__device__ __forceinline__ bool next_work(const Args &p, uint32_t j, Work &w) {
    const uint32_t m_tiles = (p.m + kBM - 1) / kBM;
    const uint32_t n_groups = (p.n + NACC * kBN - 1) / (NACC * kBN);
    const uint32_t kblocks = p.k / kBK;
    const uint32_t base = m_tiles * n_groups;
    const uint32_t item = blockIdx.x + j * gridDim.x;
    if (p.ksplit > 1) {  // k-range fastest, then token group, then slab
        if (item >= base * p.ksplit) return false;
        w.mt = item / (n_groups * p.ksplit);
        w.n0 = ((item / p.ksplit) % n_groups) * (NACC * kBN);
        w.ntok = NACC * kBN;
        w.part = item % p.ksplit;
        w.kb0 = (uint32_t)((uint64_t)kblocks * w.part / p.ksplit);
        w.kb1 = (uint32_t)((uint64_t)kblocks * (w.part + 1) / p.ksplit);
        return true;
    }
    w.part = 0; w.kb0 = 0; w.kb1 = kblocks;
    const uint32_t whole = p.tail_tok ? base - p.tail_items : base;  // a multiple of the grid when there is a tail
    if (item < whole) {
        w.mt = item / n_groups;
        w.n0 = (item % n_groups) * (NACC * kBN);
        w.ntok = NACC * kBN;
        return true;
    }
    if (!p.tail_tok || j != whole / gridDim.x || blockIdx.x >= p.tail_items * p.tail_parts) return false;
    const uint32_t t_item = whole + blockIdx.x / p.tail_parts;
    w.mt = t_item / n_groups;
    w.n0 = (t_item % n_groups) * (NACC * kBN) + (blockIdx.x % p.tail_parts) * p.tail_tok;
    w.ntok = p.tail_tok;
    return true;
}

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

// ---- weights for the A tile -------------------------------------------------------
// ARaw<TY> holds, in registers, the bytes one thread needs to unpack 32 weights
// (half h of k-block kb of its row); load() is issued one k-block ahead of
// decode() so the memory latency hides behind the previous block's work.
// Q4_K and Q2_0 (the prefill shapes that are benchmarked) have register
// forms; the other types unpack straight from memory with decode32.
// Which 16-byte chunk of the row's 128 bytes (64 k) the thread's c4-th group of eight values is.
__device__ __forceinline__ uint32_t chunk_in_order(uint32_t h, uint32_t c4) { return h * 4 + c4; }

template <int TY> struct ARaw {
    static constexpr int kAhead = 1;  // k-blocks of this thread in flight beside the one being unpacked
    __device__ static __forceinline__ uint32_t chunk(uint32_t h, uint32_t c4) { return chunk_in_order(h, c4); }
    const uint8_t *wp; uint32_t gran;
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t kb, uint32_t h) { wp = row; gran = kb * 2 + h; }
    __device__ __forceinline__ void decode(float (&v)[32], const uint64_t *grid) const { decode32<TY>(wp, gran, v, grid); }
};
// Q4_K: a k-block is 32 bytes of a 144-byte block: low nibbles = its first 32 weights (sub-block
// 2p), high nibbles = the other 32 (sub-block 2p + 1).  The two threads of a row take 16 bytes
// each and unpack both nibbles, so a thread fetches 32 bytes per k-block, header included, and
// can afford to fetch two k-blocks ahead: one turn ahead does not cover the latency of L2.
template <> struct ARaw<T_Q4_K> {
    static constexpr int kAhead = 2;
    // values 0..15 are k = 16h + 0..15 (chunks 2h, 2h + 1), values 16..31 the same positions 32 further on
    __device__ static __forceinline__ uint32_t chunk(uint32_t h, uint32_t c4) { return (c4 >> 1) * 4 + 2 * h + (c4 & 1); }
    uint4 hdr, q; uint32_t p;  // p: which 32 bytes of the block's 128
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t kb, uint32_t h) {
        const uint8_t *b = row + (size_t)(kb >> 2) * 144;
        hdr = __ldg(reinterpret_cast<const uint4 *>(b));
        q = __ldg(reinterpret_cast<const uint4 *>(b + 16 + 32 * (kb & 3) + 16 * h));
        p = kb & 3;
    }
    // w = (d * sc) * q - dmin * m (LLM/Quantize/KQuants.swift:104-125), here with one
    // fused multiply-add: the result is rounded to a 16-bit float anyway
    __device__ __forceinline__ void decode(float (&v)[32], const uint64_t *) const {
        // 6-bit scales and mins of sub-blocks 2p and 2p + 1 (get_scale_min_k4): bytes 2p, 2p + 1 of
        // the scale field for p < 2, split fields above
        const uint32_t sh = (p & 1) * 16;
        const uint32_t a = hdr.y >> sh, b = hdr.z >> sh, e = hdr.w >> sh;
        uint32_t sc, mn;  // two bytes each: sub-block 2p, 2p + 1
        if (p < 2) { sc = a & 0x3F3Fu; mn = b & 0x3F3Fu; }
        else { sc = (e & 0x0F0Fu) | ((a >> 2) & 0x3030u); mn = ((e >> 4) & 0x0F0Fu) | ((b >> 2) & 0x3030u); }
        const float d = f16bits(hdr.x & 0xFFFF), dm = f16bits(hdr.x >> 16);
        const float d0 = d * byte_to_f32(sc, 0), d1 = d * byte_to_f32(sc, 1);
        const float o0 = dm * byte_to_f32(mn, 0), o1 = dm * byte_to_f32(mn, 1);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t lo = w[i] & 0x0F0F0F0Fu, hi = (w[i] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
            for (int e4 = 0; e4 < 4; e4++) {
                v[4 * i + e4] = fmaf(d0, byte_to_f32(lo, e4), -o0);
                v[16 + 4 * i + e4] = fmaf(d1, byte_to_f32(hi, e4), -o1);
            }
        }
    }
};
template <> struct ARaw<T_Q8_0> {
    static constexpr int kAhead = 1;
    __device__ static __forceinline__ uint32_t chunk(uint32_t h, uint32_t c4) { return chunk_in_order(h, c4); }
    uint32_t w[10], sh;  // the 34-byte block {f16 d; i8 q[32]} and what precedes it in its first word
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t kb, uint32_t h) {
        const uint8_t *b = row + (size_t)(kb * 2 + h) * 34;  // 2-byte aligned
        const uint32_t *p = reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(b) & ~(uintptr_t)3);
        sh = ((uint32_t)reinterpret_cast<uintptr_t>(b) & 2u) * 8u;
#pragma unroll
        for (int i = 0; i < 10; i++) w[i] = __ldg(p + i);  // may run a few bytes past the block (buffers are padded)
    }
    __device__ __forceinline__ void decode(float (&v)[32], const uint64_t *) const {
        uint32_t u[9];
#pragma unroll
        for (int i = 0; i < 9; i++) u[i] = __funnelshift_r(w[i], w[i + 1], sh);
        const float d = f16bits(u[0] & 0xFFFF);
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const int at = 2 + j;  // byte index in the block
            const uint32_t word = u[at >> 2] ^ 0x80808080u;  // q + 128 as an unsigned byte
            v[j] = d * (byte_to_f32(word, at & 3) - 128.f);
        }
    }
};
template <> struct ARaw<T_Q2_0> {
    static constexpr int kAhead = 1;
    __device__ static __forceinline__ uint32_t chunk(uint32_t h, uint32_t c4) { return chunk_in_order(h, c4); }
    uint32_t c0, c1, dbits;  // 32 two-bit codes and the block scale
    __device__ __forceinline__ void load(const uint8_t *row, uint32_t kb, uint32_t h) {
        const uint8_t *b = row + (size_t)(kb >> 1) * 34;           // block of 128 weights
        const uint16_t *q = reinterpret_cast<const uint16_t *>(b + 2 + 16 * (kb & 1) + 8 * h);
        dbits = __ldg(reinterpret_cast<const uint16_t *>(b));
        c0 = (uint32_t)__ldg(q) | ((uint32_t)__ldg(q + 1) << 16);
        c1 = (uint32_t)__ldg(q + 2) | ((uint32_t)__ldg(q + 3) << 16);
    }
    __device__ __forceinline__ void decode(float (&v)[32], const uint64_t *) const {
        const float d = f16bits(dbits);
#pragma unroll
        for (int e = 0; e < 16; e++) {
            v[e] = (float)((int)((c0 >> (2 * e)) & 3u) - 1) * d;
            v[16 + e] = (float)((int)((c1 >> (2 * e)) & 3u) - 1) * d;
        }
    }
};

// byte offset of 16-byte chunk j of row r in a 128-byte-swizzled K-major tile
__device__ __forceinline__ uint32_t swz(uint32_t r, uint32_t j) { return r * 128 + ((j ^ (r & 7)) << 4); }

__device__ __forceinline__ void cp_async16_arrive(uint64_t *bar) {
    // the arrival fires when this thread's earlier cp.async copies have landed
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One 2-D tile of the activations, global -> shared, through the tensor map: box =
// 64 k x 256 tokens, written in the 128-byte-swizzled layout the MMA reads; tokens
// past the end of X come back as zeros.  x is the element index along k (a multiple
// of 8, so the copy starts on a 16-byte boundary), y the token.
__device__ __forceinline__ void tma_load_tile(void *dst, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

// Waiting on an mbarrier without taking issue slots from the unpacking warps: try_wait with
// a time hint parks the thread in hardware until the phase completes or the hint runs out,
// so a waiter costs a handful of instructions per microsecond instead of a polling loop.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t *bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// The phase was not over at the first look.  Bounded (about a second): a wait that gives
// up sets the CTA's abort flag and the status word.
__device__ __noinline__ bool mbar_wait_parked(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 16; i++)
            if (mbar_try_wait_hint(bar, parity, 2000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) break;
    }
    *abort_flag = 1;
    if (status) atomicExch(status, kStatusGemmTimeout);
    return false;
}
// One lane waits, the warp follows.
__device__ __forceinline__ bool warp_wait(uint64_t *bar, uint32_t parity, uint32_t lane, volatile int *abort_flag,
                                          int *status) {
    bool ok = true;
    if (lane == 0 && !mbar_try_wait(bar, parity)) ok = mbar_wait_parked(bar, parity, abort_flag, status);
    return __shfl_sync(0xffffffffu, ok, 0);
}
// a single thread (the MMA issuer, the copy engine's clients)
__device__ __forceinline__ bool thread_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status) {
    return mbar_try_wait(bar, parity) || mbar_wait_parked(bar, parity, abort_flag, status);
}

// NACC: token blocks (accumulators) per work item, 1 or 2.
template <int TY, int XDT, typename OT, int NACC>
// (The tensor map comes first so that its 128 bytes start on a 128-byte boundary of the
// parameter block whatever the size of Args: measured 12 % slower when it straddled one.)
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap xmap, Args p, Outs go) {
    constexpr bool F16 = XDT == DT_F16;
    constexpr bool ASYNC_B = XDT != DT_F32;  // 16-bit activations come by TMA, fp32 ones are converted by eight warps
    using R = Rings<TY, NACC>;
    constexpr uint32_t kAStages = R::a_stages, kBStages = R::b_stages, kBStage = R::b_stage;
    constexpr uint32_t kGroups = ASYNC_B ? 2 : 1;  // groups of eight unpacking warps
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *a_ring = smem, *b_ring = smem + R::a_bytes;
    uint64_t *grid = reinterpret_cast<uint64_t *>(smem + R::a_bytes + R::b_bytes);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + R::a_bytes + R::b_bytes + R::grid_bytes);
    uint64_t *full_a = bars, *empty_a = bars + kMaxRing;                    // A producers <-> MMA, one pair per A stage
    uint64_t *full_b = bars + 2 * kMaxRing, *empty_b = bars + 3 * kMaxRing;  // B producer(s) <-> MMA, one pair per B stage
    uint64_t *acc_full = bars + 4 * kMaxRing;  // MMA -> epilogue, one per accumulator
    uint64_t *acc_empty = acc_full + 2;        // epilogue -> MMA
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kAStages; s++) {
            mbar_init(&full_a[s], kAWarps);
            mbar_init(&empty_a[s], 1);
        }
        for (uint32_t s = 0; s < kBStages; s++) {
            mbar_init(&full_b[s], ASYNC_B ? 1 : kBWarps);
            mbar_init(&empty_b[s], 1);
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

    if (warp < kAWarps || (ASYNC_B && warp < kProducerWarps)) {
        // ---------------- A producers: unpack 128 rows x 64 weights into swizzled shared memory.
        // With 16-bit activations there are two groups of eight warps that take the k-blocks
        // in turn: one k-block's latency (load, decode, wait, store, fence) is longer than the
        // MMAs it feeds, two in flight are not.
        const uint32_t grp = warp / kAWarps;
        const uint32_t t = threadIdx.x % (kAWarps * 32);
        const uint32_t arow = t >> 1, ahalf = t & 1;  // thread t unpacks 32 weights of row arow
        uint32_t it0 = 0;  // stage counter at the start of the work item
        Work wk;
        // decoded values -> 16-bit floats -> this thread's four 16-byte chunks of stage s
        auto put = [&](const float (&v)[32], bool live, uint32_t it) -> bool {
            const uint32_t s = it % kAStages, use = it / kAStages;
            uint4 q[4];
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++) {
                q[c4].x = live ? pack16<F16>(v[8 * c4], v[8 * c4 + 1]) : 0u;
                q[c4].y = live ? pack16<F16>(v[8 * c4 + 2], v[8 * c4 + 3]) : 0u;
                q[c4].z = live ? pack16<F16>(v[8 * c4 + 4], v[8 * c4 + 5]) : 0u;
                q[c4].w = live ? pack16<F16>(v[8 * c4 + 6], v[8 * c4 + 7]) : 0u;
            }
            if (use > 0 && !warp_wait(&empty_a[s], (use - 1) & 1, lane, abort_flag, p.status)) return false;
            const uint32_t sa = smem_u32(a_ring) + s * kABytes;
#pragma unroll
            for (int c4 = 0; c4 < 4; c4++)
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sa + swz(arow, ARaw<TY>::chunk(ahalf, c4))), "r"(q[c4].x),
                             "r"(q[c4].y), "r"(q[c4].z), "r"(q[c4].w)
                             : "memory");
            fence_proxy_async();  // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_a[s]);
            return true;
        };
        for (uint32_t j = 0; next_work<NACC>(p, j, wk); j++) {
            const uint32_t m0 = wk.mt * kBM;
            const uint32_t kb0 = wk.kb0, kb1 = wk.kb1;
            const bool arow_live = m0 + arow < p.m;
            const uint32_t wrow = min(m0 + arow, p.m - 1);
            const uint8_t *wp = p.w + (size_t)wrow * p.row_bytes;
            // this group's first k-block: the one whose stage counter has its parity
            const uint32_t first = kb0 + (kGroups == 2 ? ((grp + it0) & 1) : 0);
            // The bytes of the next k-block (Q4_K: of the next two) are fetched while this one is
            // unpacked.  (Tried and slower: refilling a register set only after put(), whose proxy
            // fence waits for the loads in flight; three sets taking turns without moves.)
            if constexpr (ARaw<TY>::kAhead == 2) {
                ARaw<TY> cur, n1, n2;
                if (first < kb1) cur.load(wp, first, ahalf);
                if (first + kGroups < kb1) n1.load(wp, first + kGroups, ahalf);
                for (uint32_t kb = first; kb < kb1; kb += kGroups) {
                    if (kb + 2 * kGroups < kb1) n2.load(wp, kb + 2 * kGroups, ahalf);
                    float v[32];
                    cur.decode(v, grid);
                    if (!put(v, arow_live, it0 + (kb - kb0))) goto done;
                    cur = n1;
                    n1 = n2;
                }
            } else {
                ARaw<TY> cur, nxt;
                if (first < kb1) cur.load(wp, first, ahalf);
                for (uint32_t kb = first; kb < kb1; kb += kGroups) {
                    if (kb + kGroups < kb1) nxt.load(wp, kb + kGroups, ahalf);  // lands while cur is unpacked
                    float v[32];
                    cur.decode(v, grid);
                    if (!put(v, arow_live, it0 + (kb - kb0))) goto done;
                    cur = nxt;
                }
            }
            it0 += kb1 - kb0;
        }
    } else if (warp == kTmaWarp) {
        // ---------------- one thread hands the B tiles to the copy engine
        if (ASYNC_B && lane == 0) {
            // B tiles of 16-bit activations: NACC x 256 tokens x 64 k per stage
            uint32_t it = 0;
            Work wk;
            for (uint32_t j = 0; next_work<NACC>(p, j, wk); j++) {
                const uint32_t nblk = wk.ntok > kBN ? NACC : 1;
                for (uint32_t kb = wk.kb0; kb < wk.kb1; kb++, it++) {
                    const uint32_t s = it % kBStages, use = it / kBStages;
                    if (use > 0 && !thread_wait(&empty_b[s], (use - 1) & 1, abort_flag, p.status)) {
                        // giving up: the copies already handed over land within microseconds;
                        // stay for a while so that they do not write into a CTA that has gone
                        const long long t0 = clock64();
                        while (clock64() - t0 < 100000) {}
                        goto done;
                    }
                    uint8_t *sb = b_ring + (size_t)s * kBStage;
                    mbar_expect_tx(&full_b[s], nblk * kBBytes);
                    for (uint32_t a = 0; a < nblk; a++)
                        tma_load_tile(sb + a * kBBytes, &xmap, kb * kBK, wk.n0 + a * kBN, &full_b[s]);
                }
            }
        }
    } else if (warp < kProducerWarps) {
        // ---------------- B tiles of fp32 activations: eight warps convert them
        if constexpr (!ASYNC_B) {
            const uint32_t t = threadIdx.x - kAWarps * 32;  // 0..255
            constexpr uint32_t kChunks = NACC * kBN * 8 / (kBWarps * 32);  // 16-byte chunks per thread
            uint32_t it = 0;
            Work wk;
            for (uint32_t j = 0; next_work<NACC>(p, j, wk); j++) {
                const uint32_t n0 = wk.n0;
                for (uint32_t kb = wk.kb0; kb < wk.kb1; kb++, it++) {
                    const uint32_t s = it % kBStages, use = it / kBStages;
                    if (use > 0 && !warp_wait(&empty_b[s], (use - 1) & 1, lane, abort_flag, p.status)) goto done;
                    uint8_t *sb = b_ring + (size_t)s * kBStage;
#pragma unroll
                    for (uint32_t i = 0; i < kChunks; i++) {
                        const uint32_t q = t + kBWarps * 32 * i;
                        const uint32_t row = q >> 3, c16 = q & 7;  // row over NACC x 256 tokens; blocks are 32 KB apart
                        const uint32_t tok = n0 + row;
                        uint8_t *dst = sb + (row >> 8) * kBBytes + swz(row & 255, c16);
                        const size_t e = (size_t)min(tok, p.n - 1) * p.k + (size_t)kb * kBK + c16 * 8;
                        uint4 v = make_uint4(0u, 0u, 0u, 0u);
                        if (tok < p.n && row < wk.ntok) {
                            const float4 f0 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + e));
                            const float4 f1 = __ldg(reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.x) + e) + 1);
                            v.x = pack16<false>(f0.x, f0.y); v.y = pack16<false>(f0.z, f0.w);
                            v.z = pack16<false>(f1.x, f1.y); v.w = pack16<false>(f1.z, f1.w);
                        }
                        *reinterpret_cast<uint4 *>(dst) = v;
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&full_b[s]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer: one thread.  Another lane of the warp asks L2 for the CTA's
        // whole slab of W (128 contiguous rows) ahead of the producers, which then read it
        // k-block by k-block, 32 bytes per row at a time.
        if (lane == 1) {
            uint32_t last_mt = 0xFFFFFFFFu;
            Work wk;
            for (uint32_t j = 0; next_work<NACC>(p, j, wk); j++) {
                const uint32_t mt = wk.mt;
                if (mt == last_mt) continue;  // same slab as the previous item
                last_mt = mt;
                const uint32_t m0 = mt * kBM;
                const size_t bytes = (size_t)min(kBM, p.m - m0) * p.row_bytes;
                const uint8_t *base = p.w + (size_t)m0 * p.row_bytes;
                if (((uintptr_t)base & 15) == 0) {
                    for (size_t off = 0; off + 16 <= bytes; off += 32768) {
                        const uint32_t n = (uint32_t)min((size_t)32768, (bytes - off) & ~(size_t)15);
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"(n) : "memory");
                    }
                }
            }
        }
        if (lane == 0) {
            uint32_t it = 0, tile = 0;
            Work wk;
            for (uint32_t j = 0; next_work<NACC>(p, j, wk); j++, tile++) {
                // N of the instruction: the tokens each block of the item really has, in sixteens
                const uint32_t live = min(wk.ntok, p.n - wk.n0);
                uint32_t idesc[NACC];
#pragma unroll
                for (uint32_t a = 0; a < (uint32_t)NACC; a++) {
                    const uint32_t nt = live > a * kBN ? min(live - a * kBN, kBN) : 0u;
                    idesc[a] = instr_desc(F16 ? 0u : 1u, kBM, nt ? (nt + 15u) & ~15u : 16u);
                }
                // accumulators: both for a two-block item, alternating for one-block items
                const uint32_t acc0 = NACC == 2 ? 0 : (tile & 1), acc_use = NACC == 2 ? tile : (tile >> 1);
                bool ok = true;
                for (uint32_t a = 0; a < (uint32_t)NACC && ok; a++)
                    if (acc_use > 0) ok = thread_wait(&acc_empty[acc0 + a], (acc_use - 1) & 1, abort_flag, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t kb0 = wk.kb0, kb1 = wk.kb1;
                for (uint32_t kb = kb0; kb < kb1; kb++, it++) {
                    const uint32_t s_a = it % kAStages, s_b = it % kBStages;
                    if (!thread_wait(&full_a[s_a], (it / kAStages) & 1, abort_flag, p.status) ||
                        !thread_wait(&full_b[s_b], (it / kBStages) & 1, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sb = smem_u32(b_ring + (size_t)s_b * kBStage);
                    const uint64_t da = smem_desc(smem_u32(a_ring + (size_t)s_a * kABytes));
#pragma unroll
                    for (uint32_t a = 0; a < (uint32_t)NACC; a++) {
                        const uint64_t db = smem_desc(sb + a * kBBytes);
                        const uint32_t d_tmem = tmem_base + (acc0 + a) * kBN;
#pragma unroll
                        for (uint32_t k4 = 0; k4 < kBK / 16; k4++) {
                            // 16 k = 32 bytes further along the swizzled 128-byte row
                            umma(d_tmem, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc[a], (kb != kb0 || k4 != 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&empty_a[s_a]);  // both stages are free once these MMAs have read them
                    umma_commit(&empty_b[s_b]);
                }
                if (!ok) break;
                for (uint32_t a = 0; a < (uint32_t)NACC; a++) umma_commit(&acc_full[acc0 + a]);
            }
        }
    } else {
        // ---------------- epilogue: four warps, warp q reads tensor-memory lanes 32q .. 32q + 31
        const uint32_t q = warp & 3;  // a warp may only touch the lane quarter given by warp id % 4
        uint32_t tile = 0;
        Work wk;
        for (uint32_t j = 0; next_work<NACC>(p, j, wk); j++, tile++) {
            const uint32_t mt = wk.mt, n0 = wk.n0;
            const uint32_t n_end = min(p.n, n0 + wk.ntok);
            const uint32_t acc0 = NACC == 2 ? 0 : (tile & 1), acc_use = NACC == 2 ? tile : (tile >> 1);
            const uint32_t row = mt * kBM + q * 32 + lane;
            float *part = p.ksplit > 1 ? p.partial + (size_t)wk.part * p.n * p.m : nullptr;
            for (uint32_t a = 0; a < (uint32_t)NACC; a++) {
                const uint32_t acc = acc0 + a;
                if (!warp_wait(&acc_full[acc], acc_use & 1, lane, abort_flag, p.status)) goto done;
                tc_fence_after();
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < kBN; c0 += 32) {
                    if (n0 + a * kBN + c0 >= n_end) break;  // nothing but padding from here on
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((q * 32) << 16) + acc * kBN + c0, r);
                    tmem_ld_wait();
                    if (row < p.m) {
                        if constexpr (!kIsGather<OT>) {
                            OT *out = reinterpret_cast<OT *>(p.out);
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const uint32_t tok = n0 + a * kBN + c0 + j;
                                if (tok < n_end) {
                                    const float f = __uint_as_float(r[j]);
                                    if (part) part[(size_t)tok * p.m + row] = f;
                                    else if constexpr (sizeof(OT) == 4) out[(size_t)tok * p.m + row] = f;
                                    else out[(size_t)tok * p.m + row] = __float2bfloat16_rn(f);
                                }
                            }
                        } else if (part) {
#pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const uint32_t tok = n0 + a * kBN + c0 + j;
                                if (tok < n_end) part[(size_t)tok * p.m + row] = __uint_as_float(r[j]);
                            }
                        } else {
                            // row shards: a warp stores 32 consecutive rows of one token (128 bytes) into
                            // every rank's buffer, over NVLink for the other ranks'
                            for (uint32_t o = 0; o < go.nout; o++) {
                                float *po = reinterpret_cast<float *>(go.outs[o]) + go.out_row0 + row;
#pragma unroll
                                for (int j = 0; j < 32; j++) {
                                    const uint32_t tok = n0 + a * kBN + c0 + j;
                                    if (tok < n_end) po[(size_t)tok * go.out_ld] = __uint_as_float(r[j]);
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc]);
            }
        }
    }
done:
    if constexpr (kIsGather<OT>)
        if (p.ksplit == 1 && blockIdx.x == 0 && threadIdx.x == 0) go.epoch[0] += go.epoch_inc;
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Sum the k-range partials in a fixed order: out[i] = part[0][i] + part[1][i] + ..., element
// i = token * m + row going to [token * out_ld + out_row0 + row] of every output buffer.
struct ReduceOut {
    uint32_t nout, m, out_ld, out_row0;
    void *outs[8];
    uint32_t *epoch;
    uint32_t epoch_inc;
};
template <typename OT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ part, ReduceOut o, size_t count,
                                                            uint32_t ksplit) {
    const size_t stride = (size_t)gridDim.x * blockDim.x * 4;
    const bool vec = (o.m & 3) == 0 && (o.out_ld & 3) == 0 && (o.out_row0 & 3) == 0;
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < count; i += stride) {
        if (vec) {  // four rows of one token
            float4 s = *reinterpret_cast<const float4 *>(part + i);
            for (uint32_t k = 1; k < ksplit; k++) {
                const float4 v = *reinterpret_cast<const float4 *>(part + k * count + i);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            const size_t at = o.out_ld == o.m ? i : (i / o.m) * o.out_ld + o.out_row0 + i % o.m;
            for (uint32_t b = 0; b < o.nout; b++) {
                if constexpr (sizeof(OT) == 4) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(o.outs[b]) + at) = s;
                else {
                    __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(o.outs[b]) + at;
                    out[0] = __float2bfloat16_rn(s.x); out[1] = __float2bfloat16_rn(s.y);
                    out[2] = __float2bfloat16_rn(s.z); out[3] = __float2bfloat16_rn(s.w);
                }
            }
        } else {
            for (size_t e = i; e < count && e < i + 4; e++) {
                float s = part[e];
                for (uint32_t k = 1; k < ksplit; k++) s += part[k * count + e];
                const size_t at = o.out_ld == o.m ? e : (e / o.m) * o.out_ld + o.out_row0 + e % o.m;
                for (uint32_t b = 0; b < o.nout; b++) {
                    if constexpr (sizeof(OT) == 4) reinterpret_cast<float *>(o.outs[b])[at] = s;
                    else reinterpret_cast<__nv_bfloat16 *>(o.outs[b])[at] = __float2bfloat16_rn(s);
                }
            }
        }
    }
    if (o.epoch && blockIdx.x == 0 && threadIdx.x == 0) o.epoch[0] += o.epoch_inc;
}

// Tensor maps for tma_load_tile.  The driver's encoder is looked up once; nothing is linked
// against libcuda.  2-D, element size 1 or 2 bytes: dims / box in elements, stride in bytes.
static cudaError_t encode_map_2d(CUtensorMap *map, bool bytes, const void *base, uint64_t dim0, uint64_t dim1,
                                 uint64_t stride, uint32_t box0, uint32_t box1, bool swizzle128) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (q != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
        encode = (EncodeFn)fn;
    }
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {stride};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(map, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                              const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}
// the activations X[n][k], 16-bit elements: 64 k x 256 tokens per copy, swizzled as the MMA reads them
static cudaError_t encode_x_map(CUtensorMap *map, const void *x, uint32_t k, uint32_t n) {
    return encode_map_2d(map, false, x, k, n, (uint64_t)k * 2, kBK, kBN, true);
}
template <int TY, int XDT, typename OT, int NACC>
static cudaError_t launch_n(const Args &a, const Outs &go, cudaStream_t s, int sms, int dev) {
    static bool attr_set[64] = {};  // the opt-in is per device
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TY, XDT, OT, NACC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Rings<TY, NACC>::smem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    const uint32_t items = ((a.m + kBM - 1) / kBM) * ((a.n + NACC * kBN - 1) / (NACC * kBN)) * a.ksplit;
    const uint32_t grid = items < (uint32_t)sms ? items : (uint32_t)sms;  // a tail split always has items > sms
    alignas(64) CUtensorMap xmap;
    memset(&xmap, 0, sizeof(xmap));
    if constexpr (XDT != DT_F32) {
        cudaError_t me = encode_x_map(&xmap, a.x, a.k, a.n);
        if (me != cudaSuccess) return me;
    }
    gemm_tc_kernel<TY, XDT, OT, NACC><<<grid, kThreads, Rings<TY, NACC>::smem, s>>>(xmap, a, go);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || a.ksplit == 1) return e;
    const size_t count = (size_t)a.n * a.m;
    ReduceOut ro = {go.nout, a.m, go.out_ld, go.out_row0, {}, go.epoch, go.epoch_inc};
    for (uint32_t o = 0; o < go.nout; o++) ro.outs[o] = go.outs[o];
    using RT = std::conditional_t<kIsGather<OT>, float, OT>;
    splitk_reduce_kernel<RT><<<sms * 4, 256, 0, s>>>(a.partial, ro, count, a.ksplit);
    return cudaGetLastError();
}

template <int TY, int XDT, typename OT>
static cudaError_t launch(const Args &a, const Outs &go, uint32_t nacc, cudaStream_t s, int sms, int dev) {
    if constexpr (XDT != DT_F32) {
        if (nacc == 2) return launch_n<TY, XDT, OT, 2>(a, go, s, sms, dev);
    }
    return launch_n<TY, XDT, OT, 1>(a, go, s, sms, dev);
}

template <int TY, int XDT>
static cudaError_t launch_o(const Args &a, const Outs &go, uint32_t nacc, int odt, cudaStream_t s, int sms, int dev) {
    if (odt == DT_F32 && go.epoch) return launch<TY, XDT, GatherF32>(a, go, nacc, s, sms, dev);
    if (odt == DT_F32) return launch<TY, XDT, float>(a, go, nacc, s, sms, dev);
    if (odt == DT_BF16) return launch<TY, XDT, __nv_bfloat16>(a, go, nacc, s, sms, dev);
    return cudaErrorInvalidValue;
}

template <int TY>
static cudaError_t launch_x(const Args &a, const Outs &go, uint32_t nacc, int xdt, int odt, cudaStream_t s, int sms, int dev) {
    switch (xdt) {
    case DT_F16: return launch_o<TY, DT_F16>(a, go, nacc, odt, s, sms, dev);
    case DT_BF16: return launch_o<TY, DT_BF16>(a, go, nacc, odt, s, sms, dev);
    case DT_F32: return launch_o<TY, DT_F32>(a, go, nacc, odt, s, sms, dev);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace tc

// How to lay a matmul over the SMs.  A work item is a 128-row slab against one
// or two 256-token blocks over all of K or, with a split, over one of ksplit
// k-ranges whose fp32 partial results a second kernel sums (ksplit * n * m floats
// of scratch).  Without a split and with more items than SMs, the items left
// after the full waves can be cut into short runs of tokens, one per CTA,
// instead of costing a whole extra wave.  The plan with the smallest estimated
// time wins.  The estimate: a CTA spends 1.04 us per k-block on an item of two
// token blocks and 0.73 us on one of one block (the unpacking of the slab, not
// the MMAs, sets the pace of a single block), a run of tokens costs no less than
// 0.55 us per k-block, and the partial sums are written and read back at 5 TB/s
// (figures measured on B200 with Q4_K weights).
struct GemmPlan {
    uint32_t nacc, ksplit, tail_items, tail_tok, tail_parts;
};

static GemmPlan gemm_tc_plan(uint32_t k, uint32_t m, uint32_t n, int xdt, int sms, uint32_t force_ksplit) {
    const uint32_t slabs = (m + tc::kBM - 1) / tc::kBM, kblocks = k / tc::kBK;
    GemmPlan best = {1, force_ksplit > 1 ? force_ksplit : 1, 0, 0, 0};
    double best_t = 1e30;
    for (uint32_t nacc = 1; nacc <= 2; nacc++) {
        if (nacc == 2 && (xdt == DT_F32 || n <= tc::kBN)) continue;
        const double t_kb = nacc == 2 ? 1.04e-6 : 0.73e-6;
        const uint32_t base = slabs * ((n + nacc * tc::kBN - 1) / (nacc * tc::kBN));
        for (uint32_t ks = 1; ks <= 8; ks++) {
            if (force_ksplit ? ks != force_ksplit : (ks > 1 && kblocks / ks < 8)) continue;
            if (ks > kblocks) continue;
            const uint32_t items = base * ks, waves = (items + sms - 1) / sms;
            const double per_item = (double)((kblocks + ks - 1) / ks) * t_kb;
            const double t_red = ks > 1 ? (2.0 * ks + 1) * n * (double)m * 4 / 5e12 : 0.0;
            const double t = waves * per_item + t_red;
            if (t < best_t) { best_t = t; best = {nacc, ks, 0, 0, 0}; }
            if (ks == 1 && nacc == 1 && base > (uint32_t)sms && base % sms) {
                const uint32_t full_waves = base / sms, left = base % sms;
                uint32_t tok = 16;
                while (left * (tc::kBN / tok) > (uint32_t)sms) tok *= 2;
                const double run = t_kb * tok / tc::kBN;
                const double t2 = full_waves * per_item + kblocks * (run > 0.55e-6 ? run : 0.55e-6);
                if (t2 < best_t) { best_t = t2; best = {1, 1, left, tok, tc::kBN / tok}; }
            }
        }
    }
    return best;
}

uint32_t gemm_tc_ksplit(uint32_t k, uint32_t m, uint32_t n, int xdt, int sms) {
    return gemm_tc_plan(k, m, n, xdt, sms, 0).ksplit;
}

bool gemm_tc_supported(int ty, uint32_t k, uint32_t m, const void *w, const void *x, int xdt, uint32_t n) {
    if (!has_fast_kernels(ty)) return false;
    if (k % 64 || m == 0 || n == 0) return false;
    if ((uintptr_t)x % 16 || (k * (xdt == DT_F32 ? 4 : 2)) % 16) return false;
    if (ty == T_Q4_K && (uintptr_t)w % 16) return false;
    return true;
}

cudaError_t launch_gemm_tc(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                           uint32_t n, void *out, int odt, int *status, uint32_t ksplit, float *partial,
                           cudaStream_t s, int sms, int dev, const GemvGatherPlan *gather) {
    tc::Args a = {};
    a.w = w; a.x = x; a.out = out; a.status = status; a.k = k; a.m = m; a.n = n;
    tc::Outs go = {};
    if (gather) {
        // row shards: the epilogue (or the reduction) stores into every rank's whole output
        go.nout = gather->nranks;
        go.out_ld = gather->seg[0].m_total;
        go.out_row0 = gather->seg[0].row_first;
        for (uint32_t r = 0; r < gather->nranks; r++) go.outs[r] = gather->seg[0].out[r];
        go.epoch = gather->epoch;
        go.epoch_inc = gather->nranks;
    } else {
        go.nout = 1; go.out_ld = m; go.out_row0 = 0; go.outs[0] = out;
    }
    // the caller decides whether there is a split (it owns the scratch); the rest is planned here
    const GemmPlan plan = gemm_tc_plan(k, m, n, xdt, sms, ksplit > 1 && partial ? ksplit : 1);
    a.ksplit = plan.ksplit;
    a.partial = partial;
    a.tail_items = plan.tail_items; a.tail_tok = plan.tail_tok; a.tail_parts = plan.tail_parts;
    a.row_bytes = (k / block_elems(ty)) * block_bytes(ty);
    switch (ty) {
    case T_Q4_K: return tc::launch_x<T_Q4_K>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_Q8_0: return tc::launch_x<T_Q8_0>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_Q4_0: return tc::launch_x<T_Q4_0>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_Q6_K: return tc::launch_x<T_Q6_K>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_Q5_K: return tc::launch_x<T_Q5_K>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_IQ4_NL: return tc::launch_x<T_IQ4_NL>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_Q2_0: return tc::launch_x<T_Q2_0>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    case T_IQ2_XXS: return tc::launch_x<T_IQ2_XXS>(a, go, plan.nacc, xdt, odt, s, sms, dev);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace okf

// ---- matmul without any allocation ----------------------------------------------------
// okf_gemm_noalloc serves callers that must not allocate device memory while they
// run: code inside a CUDA-graph capture or a real-time decode loop, a process that
// shares the GPU under a fixed memory budget, a plugin host that forbids cudaMalloc
// after start-up.  The split-K matmul normally takes its partial-sum buffer from
// the context, which grows it with cudaMalloc on demand; here the buffer is a
// fixed array that is part of the loaded library image instead.
namespace okf {
constexpr size_t kStaticScratchFloats = (size_t)4 << 20;  // 16 MiB on every GPU that loads the library
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
// In host code the name above is only a stand-in for the symbol; the device address has
// to be asked for, once per device, with that device current.  The cache is not
// synchronised: two threads that meet here for the first time both look the address
// up and both store the same value.
static float *g_static_scratch_addr[64] = {};
}  // namespace okf

extern "C" int okf_gemm_noalloc(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                                const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream) {
    using namespace okf;
    int rc = check_gemm_args(ctx, type, w, woff, k, m, x, xdt, n, out, odt);
    if (rc) return rc;
    const uint8_t *wp = w->dptr + woff;
    if (!gemm_tc_supported(type, k, m, wp, x, xdt, n)) return OKF_E_ALIGN;
    // at least two k-ranges, so the scratch really carries the partial sums
    if (k / tc::kBK < 2) return OKF_E_SHAPE;
    uint32_t ksplit = gemm_tc_ksplit(k, m, n, xdt, ctx->sms);
    if (ksplit < 2) ksplit = 2;
    const size_t per_split = (size_t)n * m;
    if (2 * per_split > kStaticScratchFloats) return OKF_E_LIMIT;  // N * M above 2 Mi outputs
    while (ksplit * per_split > kStaticScratchFloats) ksplit--;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    if (ctx->device < 0 || ctx->device >= 64) return OKF_E_ARG;
    if (!g_static_scratch_addr[ctx->device]) {
        // first call on this device: resolve the array's device address
        float *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&ptr, g_static_scratch);
        if (e != cudaSuccess) return cuda_fail(ctx, e);
        g_static_scratch_addr[ctx->device] = ptr;
    }
    // every (k-range, token, row) slot the reduction reads is written by the main kernel
    // first, so nothing in the array has to be cleared between calls
    cudaError_t e = launch_gemm_tc(type, wp, k, m, x, xdt, n, out, odt, ctx->dev_status, ksplit,
                                   g_static_scratch_addr[ctx->device], (cudaStream_t)stream, ctx->sms, ctx->device, nullptr);
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches += 2;
    return OKF_OK;
}
