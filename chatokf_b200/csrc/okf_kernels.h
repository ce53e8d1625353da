// Launchers of the CUDA kernels, called by the C ABI in okf_api.cu.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace okf {

// Simple kernels: one warp per row (matvec), one fp32 register tile per thread
// (matmul).  They define the numerics the fast kernels are checked against on
// the device and serve shapes the fast kernels do not take.
cudaError_t launch_dequant(int ty, const uint8_t *w, uint64_t count, float *out, cudaStream_t s);
cudaError_t launch_gemv_simple(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x,
                               int xdt, uint32_t n, float *out, cudaStream_t s);
cudaError_t launch_gemm_simple(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x,
                               int xdt, uint32_t n, void *out, int odt, cudaStream_t s);

// Tensor-core matvec for 1..8 activation columns (okf_gemv.cu).  `supported`
// says whether the shape, alignment and element type are ones it takes; the
// caller routes everything else to the simple kernel.
bool gemv_fast_supported(int ty, uint32_t k, uint32_t m, const void *w, const void *x, int xdt, uint32_t n,
                         int sms);
cudaError_t launch_gemv_fast(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                             uint32_t n, float *out, int *status, cudaStream_t s, int sms, int dev,
                             uint64_t *launches);
// The same for up to four matrices of one type and K that multiply the same x:
// one launch (per pass over columns) covers them all.
bool gemv_group_supported(int ty, uint32_t k, uint32_t nseg, const uint32_t *m, const uint8_t *const *w,
                          const void *x, int xdt, uint32_t n, int sms);
// `gather` (may be null): the matrices are row shards of larger ones spread over
// several GPUs; every rank stores its rows into every rank's whole output through
// peer-mapped pointers; the launch neither fences nor waits.  The next gathered launch
// announces this exchange on every rank (one spare warp, after a system-wide fence) and,
// unless it is free-running, waits (bounded; a timeout is reported in the status word)
// for it before it reads x; launch_gather_wait does both as a kernel of its own.
// `out` is unused then.
struct GemvGatherPlan {
    uint32_t nranks, rank;
    uint32_t *arrivals[8];  // rank r's counter, as mapped into this process
    uint32_t *epoch;        // two local device words (see GemvGather)
    const uint32_t *wait_arrivals, *wait_epoch;  // the exchange launched before this one, or null
    bool free_running;      // the caller vouches that x does not depend on an exchange in flight
    uint32_t sig_nranks;    // the exchange launched before this one that is still to be announced (0: none):
    uint32_t *sig_arrivals[8];  // its counters on every rank
    struct {
        uint32_t m_total, row_first;
        float *out[8];      // rank r's [n][m_total] buffer, as mapped into this process
    } seg[4];
};
cudaError_t launch_gemv_group(int ty, uint32_t nseg, const uint8_t *const *w, const uint32_t *m, float *const *out,
                              uint32_t k, const void *x, int xdt, uint32_t n, int *status, cudaStream_t s,
                              int sms, int dev, uint64_t *launches, const GemvGatherPlan *gather);

// One thread that announces the exchange still pending in `plan` (sig_*) and waits (bounded)
// until the local arrival counter has reached the published count (wait_*).
cudaError_t launch_gather_wait(const GemvGatherPlan &plan, int *status, cudaStream_t s);

// Prefill matmul on tcgen05 / tensor memory (okf_gemm_tc.cu), any N.
bool gemm_tc_supported(int ty, uint32_t k, uint32_t m, const void *w, const void *x, int xdt, uint32_t n);
// ksplit > 1 cuts K into ranges whose fp32 partial results go to `partial`
// (ksplit * n * m floats) and are summed by a second kernel; gemm_tc_ksplit
// proposes a split for a shape.
uint32_t gemm_tc_ksplit(uint32_t k, uint32_t m, uint32_t n, int xdt, int sms);
// `gather` (may be null): row shards, as for the matvec; results go to every rank's whole
// output (seg[0]) instead of `out`.
cudaError_t launch_gemm_tc(int ty, const uint8_t *w, uint32_t k, uint32_t m, const void *x, int xdt,
                           uint32_t n, void *out, int odt, int *status, uint32_t ksplit, float *partial,
                           cudaStream_t s, int sms, int dev, const GemvGatherPlan *gather);

}  // namespace okf
