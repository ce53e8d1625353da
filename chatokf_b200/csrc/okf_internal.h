// Internals shared by the translation units that implement the C ABI.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/okf_cuda.h"
#include "okf_blocks.cuh"

struct okf_weights {
    uint8_t *dptr;
    size_t bytes;
    bool owned;
};

#include "okf_kernels.h"

struct okf_ctx {
    int device;
    int sms;
    uint32_t flags;
    int *dev_status;  // device word the kernels' bounded waits report into
    cudaStream_t stream;
    int last_cuda;
    uint64_t launches;
    uint64_t fallbacks;  // calls that took a simple kernel because a fast one declined the shape
    // host-twin staging (device side), grown on demand
    void *stage_x;
    size_t stage_x_bytes;
    void *stage_out;
    size_t stage_out_bytes;
    // scratch for the matmul's k-range partial sums, grown on demand
    void *scratch;
    size_t scratch_bytes;
    // staged faults (host side only)
    double fault_rate;
    uint64_t fault_state;
    // okf_parallel_begin .. okf_parallel_end: narrow matvecs of one x, type and K
    // wait here and leave as one launch
    bool par_open;
    uint32_t par_count;
    int par_type, par_xdt;
    uint32_t par_k, par_n;
    const void *par_x;
    cudaStream_t par_stream;
    const uint8_t *par_w[4];
    uint32_t par_m[4];
    float *par_out[4];
    bool par_gathers;               // the waiting set stores into every rank's output
    okf::GemvGatherPlan par_gather;
    // the exchange launched last (local counter and epoch words), which the next gathered
    // launch or okf_gather_wait waits for; null when there is none
    const uint32_t *last_arrivals, *last_epoch;
    // its counters on every rank while it has not been announced yet (sig_nranks = 0: none pending)
    uint32_t sig_nranks;
    uint32_t *sig_arrivals[8];
};


namespace okf {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) ok = cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

inline int cuda_fail(okf_ctx *ctx, cudaError_t e) {
    if (ctx) ctx->last_cuda = (int)e;
    (void)cudaGetLastError();  // clear the error so later calls start clean
    return OKF_E_CUDA;
}

inline bool type_ok(int ty) { return block_elems(ty) != 0; }
inline bool dtype_ok(int dt) { return dt == DT_F32 || dt == DT_F16 || dt == DT_BF16; }
inline size_t dtype_size(int dt) { return dt == DT_F32 ? 4 : 2; }

// The seeded draw behind okf_fault_inject: a 64-bit LCG, top 53 bits as a
// uniform number in [0, 1).
inline bool fault_fires(okf_ctx *ctx) {
    if (ctx->fault_rate <= 0.0) return false;
    ctx->fault_state = ctx->fault_state * 6364136223846793005ull + 1442695040888963407ull;
    const double u = (double)(ctx->fault_state >> 11) * (1.0 / 9007199254740992.0);
    return u < ctx->fault_rate;
}

inline int check_tensor(const okf_ctx *ctx, int ty, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m) {
    if (!ctx || !w) return OKF_E_ARG;
    if (!type_ok(ty)) return OKF_E_TYPE;
    if (k == 0 || m == 0 || k % (uint32_t)block_elems(ty)) return OKF_E_SHAPE;
    const uint64_t need = (uint64_t)(k / block_elems(ty)) * block_bytes(ty) * m;
    if (woff > w->bytes || need > w->bytes - woff) return OKF_E_RANGE;
    // Q4_K kernels read 32-bit words; the other layouts are 2-byte structured.
    const uint64_t a = ty == T_Q4_K ? 16 : 2;
    if (((uintptr_t)w->dptr + woff) % a) return OKF_E_ALIGN;
    return OKF_OK;
}

// Argument checks common to every matmul entry point.
inline int check_gemm_args(okf_ctx *ctx, int ty, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                           const void *x, int xdt, uint32_t n, const void *out, int odt) {
    int rc = check_tensor(ctx, ty, w, woff, k, m);
    if (rc) return rc;
    if (!x || !out) return OKF_E_ARG;
    if (n == 0) return OKF_E_SHAPE;
    if (!dtype_ok(xdt) || (odt != DT_F32 && odt != DT_BF16)) return OKF_E_TYPE;
    if ((uintptr_t)x % dtype_size(xdt) || (uintptr_t)out % dtype_size(odt)) return OKF_E_ALIGN;
    return OKF_OK;
}

}  // namespace okf
