// C ABI of libokfcuda (include/okf_cuda.h): argument checks, dispatch by type
// and batch width, host staging for the CPU-operator twins.
#include <new>
#include <stdlib.h>
#include <string.h>

#include "okf_internal.h"
#include "okf_kernels.h"

using namespace okf;

namespace {

constexpr size_t kTailPad = 256;  // bytes readable past the last block of an upload

#define OKF_CUDA(ctx, call)                                   \
    do {                                                      \
        cudaError_t e_ = (call);                              \
        if (e_ != cudaSuccess) return cuda_fail((ctx), e_);   \
    } while (0)

int grow(okf_ctx *ctx, void **buf, size_t *have, size_t need) {
    if (*have >= need) return OKF_OK;
    if (*buf) OKF_CUDA(ctx, cudaFree(*buf));
    *buf = nullptr;
    *have = 0;
    cudaError_t e = cudaMalloc(buf, need);
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        return OKF_E_NOMEM;
    }
    OKF_CUDA(ctx, e);
    *have = need;
    return OKF_OK;
}

// A gathered launch waits for the exchange launched before it and becomes the one the
// next launch waits for.
void gather_chain(okf_ctx *ctx, GemvGatherPlan &plan) {
    plan.wait_arrivals = plan.free_running ? nullptr : ctx->last_arrivals;
    plan.wait_epoch = plan.free_running ? nullptr : ctx->last_epoch;
    plan.sig_nranks = ctx->sig_nranks;
    for (uint32_t r = 0; r < ctx->sig_nranks; r++) plan.sig_arrivals[r] = ctx->sig_arrivals[r];
    ctx->last_arrivals = plan.arrivals[plan.rank];
    ctx->last_epoch = plan.epoch;
    ctx->sig_nranks = plan.nranks;
    for (uint32_t r = 0; r < plan.nranks; r++) ctx->sig_arrivals[r] = plan.arrivals[r];
}

// Launch what a parallel region has collected.
int par_flush(okf_ctx *ctx) {
    const uint32_t cnt = ctx->par_count;
    if (cnt == 0) return OKF_OK;
    ctx->par_count = 0;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    cudaError_t e = cudaSuccess;
    if (cnt > 1 && gemv_group_supported(ctx->par_type, ctx->par_k, cnt, ctx->par_m, ctx->par_w, ctx->par_x,
                                        ctx->par_xdt, ctx->par_n, ctx->sms)) {
        if (ctx->par_gathers) gather_chain(ctx, ctx->par_gather);
        e = launch_gemv_group(ctx->par_type, cnt, ctx->par_w, ctx->par_m, ctx->par_out, ctx->par_k, ctx->par_x,
                              ctx->par_xdt, ctx->par_n, ctx->dev_status, ctx->par_stream, ctx->sms, ctx->device,
                              &ctx->launches, ctx->par_gathers ? &ctx->par_gather : nullptr);
    } else {
        // One launch per matrix; with a gather each one is an exchange of its own on the set's
        // counter.  The count an exchange is complete at is a running total that every launch
        // adds its own CTAs to, so exchanges of different grid sizes may share a counter.
        for (uint32_t i = 0; i < cnt && e == cudaSuccess; i++) {
            GemvGatherPlan one = ctx->par_gather;
            one.seg[0] = ctx->par_gather.seg[i];
            if (ctx->par_gathers) gather_chain(ctx, one);
            e = launch_gemv_group(ctx->par_type, 1, &ctx->par_w[i], &ctx->par_m[i], &ctx->par_out[i], ctx->par_k,
                                  ctx->par_x, ctx->par_xdt, ctx->par_n, ctx->dev_status, ctx->par_stream, ctx->sms,
                                  ctx->device, &ctx->launches, ctx->par_gathers ? &one : nullptr);
        }
    }
    return e == cudaSuccess ? OKF_OK : cuda_fail(ctx, e);
}

int gemm_dispatch(okf_ctx *ctx, int ty, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                  const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream,
                  bool force_tile) {
    int rc = check_gemm_args(ctx, ty, w, woff, k, m, x, xdt, n, out, odt);
    if (rc) return rc;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    cudaStream_t s = (cudaStream_t)stream;
    const uint8_t *wp = w->dptr + woff;
    cudaError_t e;
    if (n <= 8 && !force_tile && odt == DT_F32) {
        const bool simple = ctx->flags & OKF_FLAG_SIMPLE_KERNELS;
        if (!simple && gemv_fast_supported(ty, k, m, wp, x, xdt, n, ctx->sms)) {
            if (ctx->par_open) {
                // inside a parallel region: join the waiting matvecs if this one multiplies
                // the same x, else send them off and start a new set
                const bool joins = ctx->par_count > 0 && ctx->par_count < 4 && !ctx->par_gathers && ctx->par_type == ty &&
                                   ctx->par_k == k && ctx->par_x == x && ctx->par_xdt == xdt && ctx->par_n == n &&
                                   ctx->par_stream == s;
                if (!joins && (rc = par_flush(ctx))) return rc;
                const uint32_t i = ctx->par_count++;
                ctx->par_type = ty; ctx->par_k = k; ctx->par_x = x; ctx->par_xdt = xdt; ctx->par_n = n;
                ctx->par_stream = s;
                ctx->par_gathers = false;
                ctx->par_w[i] = wp; ctx->par_m[i] = m; ctx->par_out[i] = (float *)out;
                return OKF_OK;
            }
            e = launch_gemv_fast(ty, wp, k, m, x, xdt, n, (float *)out, ctx->dev_status, s, ctx->sms, ctx->device,
                                 &ctx->launches);
            if (e != cudaSuccess) return cuda_fail(ctx, e);
            return OKF_OK;
        } else {
            if (!simple) ctx->fallbacks++;  // a shape or alignment the tensor-core matvec does not take
            e = launch_gemv_simple(ty, wp, k, m, x, xdt, n, (float *)out, s);
        }
    } else if (!(ctx->flags & OKF_FLAG_SIMPLE_KERNELS) && gemm_tc_supported(ty, k, m, wp, x, xdt, n)) {
        uint32_t ksplit = gemm_tc_ksplit(k, m, n, xdt, ctx->sms);
        if (ksplit > 1) {
            // Growing the scratch allocates, which is not allowed while a stream is being
            // captured into a graph: size it with one call outside the capture first.
            const size_t need = (size_t)ksplit * n * m * sizeof(float);
            if (ctx->scratch_bytes < need) {
                cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
                (void)cudaStreamIsCapturing(s, &cs);
                if (cs != cudaStreamCaptureStatusNone) ksplit = 1;
                else if ((rc = grow(ctx, &ctx->scratch, &ctx->scratch_bytes, need))) return rc;
            }
        }
        e = launch_gemm_tc(ty, wp, k, m, x, xdt, n, out, odt, ctx->dev_status, ksplit, (float *)ctx->scratch, s,
                           ctx->sms, ctx->device, nullptr);
        if (e == cudaSuccess && ksplit > 1) ctx->launches++;
    } else {
        if (!(ctx->flags & OKF_FLAG_SIMPLE_KERNELS)) ctx->fallbacks++;
        e = launch_gemm_simple(ty, wp, k, m, x, xdt, n, out, odt, s);
    }
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

}  // namespace

extern "C" {

const char *okf_strerror(int status) {
    switch (status) {
    case OKF_OK: return "ok";
    case OKF_E_ARG: return "bad argument";
    case OKF_E_TYPE: return "unsupported weight or element type";
    case OKF_E_SHAPE: return "bad shape: K must be a positive multiple of the block size, M and N positive";
    case OKF_E_RANGE: return "tensor runs past the end of the weights buffer";
    case OKF_E_ALIGN: return "pointer or offset not aligned as the kernels need";
    case OKF_E_CUDA: return "CUDA call failed (see okf_last_cuda_error)";
    case OKF_E_NOMEM: return "out of memory";
    case OKF_E_INJECTED: return "staged fault fired (okf_fault_inject)";
    case OKF_E_LIMIT: return "size beyond a fixed maximum";
    case OKF_E_FORMAT: return "not a GGUF file, or a truncated or malformed one";
    case OKF_E_IO: return "file could not be opened or mapped";
    default: return "unknown status";
    }
}

int okf_init(int device, okf_ctx **out) {
    if (!out) return OKF_E_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) {
        (void)cudaGetLastError();
        return OKF_E_CUDA;
    }
    okf_ctx *ctx = new (std::nothrow) okf_ctx();
    if (!ctx) return OKF_E_NOMEM;
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    DeviceGuard g(device);
    cudaError_t e = g.ok ? cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)
                         : cudaErrorInvalidDevice;
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&ctx->sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaMalloc((void **)&ctx->dev_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->dev_status, 0, sizeof(int));
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        delete ctx;
        return OKF_E_CUDA;
    }
    *out = ctx;
    return OKF_OK;
}

void okf_destroy(okf_ctx *ctx) {
    if (!ctx) return;
    DeviceGuard g(ctx->device);
    if (ctx->stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
    }
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->stage_x) cudaFree(ctx->stage_x);
    if (ctx->stage_out) cudaFree(ctx->stage_out);
    (void)cudaGetLastError();
    delete ctx;
}

int okf_last_cuda_error(const okf_ctx *ctx) { return ctx ? ctx->last_cuda : 0; }
okf_stream okf_ctx_stream(const okf_ctx *ctx) { return ctx ? (okf_stream)ctx->stream : nullptr; }
uint64_t okf_launch_count(const okf_ctx *ctx) { return ctx ? ctx->launches : 0; }
uint64_t okf_fallback_count(const okf_ctx *ctx) { return ctx ? ctx->fallbacks : 0; }

int okf_sync(okf_ctx *ctx) {
    if (!ctx) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    // matvecs a parallel region is still holding back are sent off first
    int rc = par_flush(ctx);
    if (rc) return rc;
    OKF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OKF_OK;
}

int okf_weights_upload(okf_ctx *ctx, const void *host, size_t bytes, okf_weights **out) {
    if (!ctx || !out || (!host && bytes)) return OKF_E_ARG;
    *out = nullptr;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    okf_weights *w = new (std::nothrow) okf_weights();
    if (!w) return OKF_E_NOMEM;
    w->bytes = bytes;
    w->owned = true;
    w->dptr = nullptr;
    cudaError_t e = cudaMalloc((void **)&w->dptr, bytes + kTailPad);
    if (e != cudaSuccess) {
        delete w;
        if (e == cudaErrorMemoryAllocation) {
            (void)cudaGetLastError();
            return OKF_E_NOMEM;
        }
        return cuda_fail(ctx, e);
    }
    e = cudaMemsetAsync(w->dptr + bytes, 0, kTailPad, ctx->stream);
    if (e == cudaSuccess && bytes) e = cudaMemcpyAsync(w->dptr, host, bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(w->dptr);
        delete w;
        return cuda_fail(ctx, e);
    }
    *out = w;
    return OKF_OK;
}

int okf_weights_wrap(okf_ctx *ctx, const void *device, size_t bytes, okf_weights **out) {
    if (!ctx || !out || !device) return OKF_E_ARG;
    okf_weights *w = new (std::nothrow) okf_weights();
    if (!w) return OKF_E_NOMEM;
    w->dptr = (uint8_t *)const_cast<void *>(device);
    w->bytes = bytes;
    w->owned = false;
    *out = w;
    return OKF_OK;
}

void okf_weights_free(okf_ctx *ctx, okf_weights *w) {
    if (!w) return;
    if (w->owned && w->dptr) {
        DeviceGuard g(ctx ? ctx->device : 0);
        cudaFree(w->dptr);
        (void)cudaGetLastError();
    }
    delete w;
}

const void *okf_weights_device_ptr(const okf_weights *w) { return w ? w->dptr : nullptr; }
size_t okf_weights_bytes(const okf_weights *w) { return w ? w->bytes : 0; }

size_t okf_row_bytes(int type, size_t k) {
    const int per = block_elems(type);
    return per ? k / (size_t)per * (size_t)block_bytes(type) : 0;
}

int okf_gemv(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
             const void *x, int xdt, float *out, okf_stream stream) {
    return gemm_dispatch(ctx, type, w, woff, k, m, x, xdt, 1, out, DT_F32, stream, false);
}

int okf_gemm(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
             const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream) {
    return gemm_dispatch(ctx, type, w, woff, k, m, x, xdt, n, out, odt, stream, false);
}

int okf_parallel_begin(okf_ctx *ctx) {
    if (!ctx || ctx->par_open) return OKF_E_ARG;
    ctx->par_open = true;
    ctx->par_count = 0;
    return OKF_OK;
}

int okf_parallel_end(okf_ctx *ctx) {
    if (!ctx || !ctx->par_open) return OKF_E_ARG;
    ctx->par_open = false;
    return par_flush(ctx);
}

int okf_shared_alloc(okf_ctx *ctx, size_t bytes, void **device_ptr, okf_ipc_handle *handle) {
    if (!ctx || !device_ptr || !handle || bytes == 0) return OKF_E_ARG;
    static_assert(sizeof(okf_ipc_handle) >= sizeof(cudaIpcMemHandle_t), "handle too small");
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaErrorMemoryAllocation) {
        (void)cudaGetLastError();
        return OKF_E_NOMEM;
    }
    OKF_CUDA(ctx, e);
    e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return cuda_fail(ctx, e);
    }
    memset(handle, 0, sizeof(*handle));
    memcpy(handle->bytes, &h, sizeof(h));
    *device_ptr = p;
    return OKF_OK;
}

int okf_shared_open(okf_ctx *ctx, const okf_ipc_handle *handle, void **device_ptr) {
    if (!ctx || !handle || !device_ptr) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle->bytes, sizeof(h));
    // with this context's device current, the mapping also turns on peer access to the owner
    OKF_CUDA(ctx, cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return OKF_OK;
}

int okf_shared_close(okf_ctx *ctx, void *device_ptr) {
    if (!ctx || !device_ptr) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    OKF_CUDA(ctx, cudaIpcCloseMemHandle(device_ptr));
    return OKF_OK;
}

int okf_shared_free(okf_ctx *ctx, void *device_ptr) {
    if (!ctx || !device_ptr) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    OKF_CUDA(ctx, cudaFree(device_ptr));
    return OKF_OK;
}

int okf_copy_to_host(okf_ctx *ctx, const void *device_ptr, void *host, size_t bytes) {
    if (!ctx || !device_ptr || !host) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    OKF_CUDA(ctx, cudaMemcpy(host, device_ptr, bytes, cudaMemcpyDeviceToHost));
    return OKF_OK;
}

int okf_gemm_gather(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                    const void *x, int xdt, uint32_t n, const okf_gather *gt, okf_stream stream) {
    if (!gt || gt->nranks < 2 || gt->nranks > 8 || gt->rank >= gt->nranks || !gt->epoch) return OKF_E_ARG;
    if ((uint64_t)gt->row_first + m > gt->m_total) return OKF_E_SHAPE;
    for (uint32_t r = 0; r < gt->nranks; r++)
        if (!gt->out[r] || !gt->arrivals[r] || (uintptr_t)gt->out[r] % 16) return OKF_E_ARG;
    int rc = check_gemm_args(ctx, type, w, woff, k, m, x, xdt, n, gt->out[gt->rank], DT_F32);
    if (rc) return rc;
    const uint8_t *wp = w->dptr + woff;
    if (n > 8) {
        // More than eight tokens: the tensor-core matmul, whose epilogue (or k-range reduction)
        // stores the tile rows into every rank's output while the other tiles are still in
        // the tensor cores.  The exchange before it is announced, and unless the call is
        // free-running waited for, by a one-thread kernel ahead of the matmul.
        if (!gemm_tc_supported(type, k, m, wp, x, xdt, n)) return OKF_E_ALIGN;
        if (fault_fires(ctx)) return OKF_E_INJECTED;
        if ((rc = par_flush(ctx))) return rc;
        DeviceGuard g(ctx->device);
        if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
        cudaStream_t s = (cudaStream_t)stream;
        GemvGatherPlan plan = {};
        plan.nranks = gt->nranks;
        plan.rank = gt->rank;
        plan.epoch = gt->epoch;
        plan.free_running = (gt->flags & OKF_GATHER_FREE) != 0;
        for (uint32_t r = 0; r < gt->nranks; r++) {
            plan.arrivals[r] = gt->arrivals[r];
            plan.seg[0].out[r] = gt->out[r];
        }
        plan.seg[0].m_total = gt->m_total;
        plan.seg[0].row_first = gt->row_first;
        gather_chain(ctx, plan);
        if (plan.sig_nranks || plan.wait_arrivals) {
            cudaError_t e = launch_gather_wait(plan, ctx->dev_status, s);
            if (e != cudaSuccess) return cuda_fail(ctx, e);
            ctx->launches++;
        }
        uint32_t ksplit = gemm_tc_ksplit(k, m, n, xdt, ctx->sms);
        if (ksplit > 1) {
            const size_t need = (size_t)ksplit * n * m * sizeof(float);
            if (ctx->scratch_bytes < need) {
                cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
                (void)cudaStreamIsCapturing(s, &cs);
                if (cs != cudaStreamCaptureStatusNone) ksplit = 1;
                else if ((rc = grow(ctx, &ctx->scratch, &ctx->scratch_bytes, need))) return rc;
            }
        }
        cudaError_t e = launch_gemm_tc(type, wp, k, m, x, xdt, n, nullptr, DT_F32, ctx->dev_status, ksplit,
                                       (float *)ctx->scratch, s, ctx->sms, ctx->device, &plan);
        if (e != cudaSuccess) return cuda_fail(ctx, e);
        ctx->launches += ksplit > 1 ? 2 : 1;
        return OKF_OK;
    }
    if (!gemv_fast_supported(type, k, m, wp, x, xdt, n, ctx->sms)) return OKF_E_ALIGN;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    cudaStream_t s = (cudaStream_t)stream;
    // a set that is waiting takes this matrix in if it gathers the same way
    const bool joins = ctx->par_open && ctx->par_count > 0 && ctx->par_count < 4 && ctx->par_gathers &&
                       ctx->par_type == type && ctx->par_k == k && ctx->par_x == x && ctx->par_xdt == xdt &&
                       ctx->par_n == n && ctx->par_stream == s && ctx->par_gather.nranks == gt->nranks;
    if (ctx->par_open && !joins && (rc = par_flush(ctx))) return rc;
    const uint32_t i = ctx->par_open ? ctx->par_count : 0;
    GemvGatherPlan fresh = {};
    GemvGatherPlan &plan = ctx->par_open ? ctx->par_gather : fresh;
    if (i == 0) {  // the exchange counts on the first matrix's counter
        plan = GemvGatherPlan{};
        plan.nranks = gt->nranks;
        plan.rank = gt->rank;
        plan.epoch = gt->epoch;
        plan.free_running = (gt->flags & OKF_GATHER_FREE) != 0;
        for (uint32_t r = 0; r < gt->nranks; r++) plan.arrivals[r] = gt->arrivals[r];
    }
    plan.seg[i].m_total = gt->m_total;
    plan.seg[i].row_first = gt->row_first;
    for (uint32_t r = 0; r < gt->nranks; r++) plan.seg[i].out[r] = gt->out[r];
    if (ctx->par_open) {
        ctx->par_count = i + 1;
        ctx->par_type = type; ctx->par_k = k; ctx->par_x = x; ctx->par_xdt = xdt; ctx->par_n = n;
        ctx->par_stream = s;
        ctx->par_gathers = true;
        ctx->par_w[i] = wp; ctx->par_m[i] = m; ctx->par_out[i] = nullptr;
        return OKF_OK;
    }
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    float *none = nullptr;
    gather_chain(ctx, plan);
    cudaError_t e = launch_gemv_group(type, 1, &wp, &m, &none, k, x, xdt, n, ctx->dev_status, s, ctx->sms,
                                      ctx->device, &ctx->launches, &plan);
    return e == cudaSuccess ? OKF_OK : cuda_fail(ctx, e);
}

int okf_gather_wait(okf_ctx *ctx, okf_stream stream) {
    if (!ctx) return OKF_E_ARG;
    int rc = par_flush(ctx);
    if (rc) return rc;
    if (!ctx->last_arrivals && !ctx->sig_nranks) return OKF_OK;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    GemvGatherPlan plan = {};
    plan.wait_arrivals = ctx->last_arrivals;
    plan.wait_epoch = ctx->last_epoch;
    plan.sig_nranks = ctx->sig_nranks;
    for (uint32_t r = 0; r < ctx->sig_nranks; r++) plan.sig_arrivals[r] = ctx->sig_arrivals[r];
    cudaError_t e = launch_gather_wait(plan, ctx->dev_status, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->last_arrivals = ctx->last_epoch = nullptr;
    ctx->sig_nranks = 0;
    ctx->launches++;
    return OKF_OK;
}

int okf_gemm_tile(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                  const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream) {
    return gemm_dispatch(ctx, type, w, woff, k, m, x, xdt, n, out, odt, stream, true);
}

int okf_dequant(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint64_t count,
                float *out, okf_stream stream) {
    if (!ctx || !w || !out) return OKF_E_ARG;
    if (!type_ok(type)) return OKF_E_TYPE;
    const uint64_t per = (uint64_t)block_elems(type);
    if (count % per) return OKF_E_SHAPE;
    const uint64_t need = count / per * (uint64_t)block_bytes(type);
    if (woff > w->bytes || need > w->bytes - woff) return OKF_E_RANGE;
    const uint64_t a = type == T_Q4_K ? 16 : 2;
    if (((uintptr_t)w->dptr + woff) % a || (uintptr_t)out % 16) return OKF_E_ALIGN;
    if (count == 0) return OKF_OK;
    if (fault_fires(ctx)) return OKF_E_INJECTED;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t e = launch_dequant(type, w->dptr + woff, count, out, s);
    if (e != cudaSuccess) return cuda_fail(ctx, e);
    ctx->launches++;
    return OKF_OK;
}

int okf_matmul_host(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k,
                    uint32_t m, const float *x, uint32_t n, float *out) {
    int rc = check_tensor(ctx, type, w, woff, k, m);
    if (rc) return rc;
    if (!x || !out) return OKF_E_ARG;
    if (n == 0) return OKF_E_SHAPE;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    const size_t xb = (size_t)n * k * sizeof(float), ob = (size_t)n * m * sizeof(float);
    if ((rc = grow(ctx, &ctx->stage_x, &ctx->stage_x_bytes, xb))) return rc;
    // Page-locked host memory is addressable from the device: the kernel then stores the
    // result straight into the caller's buffer and the copy back falls away.  (x is read
    // by every CTA, so it still goes to the device first.)
    void *dev_out = nullptr;
    cudaPointerAttributes pa;
    if (cudaPointerGetAttributes(&pa, out) == cudaSuccess && pa.type == cudaMemoryTypeHost && pa.devicePointer &&
        (uintptr_t)pa.devicePointer % 16 == 0)
        dev_out = pa.devicePointer;
    else
        (void)cudaGetLastError();
    if (!dev_out && (rc = grow(ctx, &ctx->stage_out, &ctx->stage_out_bytes, ob))) return rc;
    OKF_CUDA(ctx, cudaMemcpyAsync(ctx->stage_x, x, xb, cudaMemcpyHostToDevice, ctx->stream));
    rc = gemm_dispatch(ctx, type, w, woff, k, m, ctx->stage_x, DT_F32, n, dev_out ? dev_out : ctx->stage_out, DT_F32,
                       (okf_stream)ctx->stream, false);
    if (rc) return rc;
    // inside a parallel region the matvec was only queued: the host twin returns a finished
    // result, so the waiting set leaves now
    if (ctx->par_open && (rc = par_flush(ctx))) return rc;
    if (!dev_out) OKF_CUDA(ctx, cudaMemcpyAsync(out, ctx->stage_out, ob, cudaMemcpyDeviceToHost, ctx->stream));
    OKF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OKF_OK;
}

int okf_matvec_host(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k,
                    uint32_t m, const float *x, float *out) {
    return okf_matmul_host(ctx, type, w, woff, k, m, x, 1, out);
}

int okf_dequant_host(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint64_t count,
                     float *out) {
    if (!ctx || !out) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    int rc = grow(ctx, &ctx->stage_out, &ctx->stage_out_bytes, (size_t)count * sizeof(float) + 16);
    if (rc) return rc;
    rc = okf_dequant(ctx, type, w, woff, count, (float *)ctx->stage_out, (okf_stream)ctx->stream);
    if (rc || count == 0) return rc;
    OKF_CUDA(ctx, cudaMemcpyAsync(out, ctx->stage_out, (size_t)count * sizeof(float),
                                  cudaMemcpyDeviceToHost, ctx->stream));
    OKF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return OKF_OK;
}

int okf_device_status(okf_ctx *ctx, int *out) {
    if (!ctx || !out) return OKF_E_ARG;
    DeviceGuard g(ctx->device);
    if (!g.ok) return cuda_fail(ctx, cudaErrorInvalidDevice);
    OKF_CUDA(ctx, cudaMemcpy(out, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    return OKF_OK;
}

int okf_set_flags(okf_ctx *ctx, uint32_t flags) {
    if (!ctx) return OKF_E_ARG;
    ctx->flags = flags;
    return OKF_OK;
}

int okf_fault_inject(okf_ctx *ctx, double rate, uint64_t seed) {
    if (!ctx || !(rate >= 0.0) || rate > 1.0) return OKF_E_ARG;
    ctx->fault_rate = rate;
    ctx->fault_state = seed + 0x9E3779B97F4A7C15ull;
    return OKF_OK;
}

}  // extern "C"
