/*
 * okf_cuda.h -- C ABI of libokfcuda: ChatOKF's block-quantized matvec / matmul
 * operator on NVIDIA B200 (sm_100a).
 *
 * This is the boundary a Swift module map binds (module.modulemap in this
 * directory).  Plain pointers and sizes only.  Every entry point returns OKF_OK
 * (0) or a negative okf_status; nothing aborts or throws.  Device work is
 * asynchronous on the stream the caller passes unless stated otherwise.
 *
 * Data conventions are the reference's (LLM/metal/Kernels.metal:22-24, :112;
 * LLM/Base/GGUF.swift:49-57, :160-188):
 *   - weights are native GGUF block bytes, M rows of K/qk blocks, rows
 *     contiguous, addressed as (weights buffer + woff) with a 64-bit woff;
 *   - x is [K] (or X is [N][K]), out is [M] (or out[n*M + m]);
 *   - K must be a multiple of the type's block size; M is arbitrary.
 *
 * A context serves one engine thread at a time (like one Metal command
 * encoder); different contexts may be used from different threads.
 */
#ifndef OKF_CUDA_H
#define OKF_CUDA_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define OKF_API __attribute__((visibility("default")))
#else
#define OKF_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ggml tensor type ids: GGUFType, LLM/Base/GGUF.swift:3-14 */
typedef enum okf_type {
    OKF_Q8_0 = 8,     /* 34 B / 32 weights   */
    OKF_Q4_K = 12,    /* 144 B / 256 weights */
    OKF_IQ2_XXS = 16, /* 66 B / 256 weights  */
    OKF_Q2_0 = 42,    /* 34 B / 128 weights, ternary */
    OKF_Q4_0 = 2,     /* 18 B / 32 weights (gemma trunks; Gemma/Gemma4Quant.swift:30-49) */
    /* The rest of the decoder table the trunks' files mix in (Blocks.decoder,
     * Quantize/Blocks.swift:10-29; Gemma/Gemma4Quant.swift:5-49): the same entry
     * points take them, bit-exact decode included, on the same kernels. */
    OKF_Q5_K = 13,    /* 176 B / 256 weights */
    OKF_Q6_K = 14,    /* 210 B / 256 weights */
    OKF_IQ4_NL = 20   /* 18 B / 32 weights, codebook of 16 values */
} okf_type;

/* element type of activations / outputs */
typedef enum okf_dtype { OKF_F32 = 0, OKF_F16 = 1, OKF_BF16 = 2 } okf_dtype;

typedef enum okf_status {
    OKF_OK = 0,
    OKF_E_ARG = -1,      /* null pointer or otherwise malformed argument      */
    OKF_E_TYPE = -2,     /* weight or element type not supported (the
                            reference's fatalError in MetalEnc.swift:108-110,
                            :144-146 becomes this code)                       */
    OKF_E_SHAPE = -3,    /* K not a multiple of the block size, N or M zero,
                            (precondition in LLM/Base/Quant.swift:31)         */
    OKF_E_RANGE = -4,    /* woff + tensor bytes runs past the weights buffer  */
    OKF_E_ALIGN = -5,    /* pointer alignment a kernel needs is not met       */
    OKF_E_CUDA = -6,     /* a CUDA call failed; see okf_last_cuda_error       */
    OKF_E_NOMEM = -7,    /* host or device allocation failed                  */
    OKF_E_INJECTED = -8, /* a staged fault from okf_fault_inject fired        */
    OKF_E_LIMIT = -9,    /* a size exceeds a documented fixed maximum         */
    OKF_E_FORMAT = -10,  /* not a GGUF file, or a truncated / malformed one   */
    OKF_E_IO = -11       /* the file could not be opened or mapped            */
} okf_status;

typedef struct okf_ctx okf_ctx;         /* replaces MetalContext (Base/MetalContext.swift:58-80) */
typedef struct okf_weights okf_weights; /* replaces WeightRef windows (Base/MetalContext.swift:4-11, :114-185) */
typedef struct CUstream_st *okf_stream; /* a cudaStream_t; NULL = CUDA's default stream */

OKF_API const char *okf_strerror(int status);

/* Create a context on `device`: its own stream, host staging, codebook tables
 * in device memory.  Replaces MetalContext.init (Base/MetalContext.swift:58-80). */
OKF_API int okf_init(int device, okf_ctx **out);
OKF_API void okf_destroy(okf_ctx *ctx);
/* cudaError_t value of the last failed CUDA call on this context (0 if none). */
OKF_API int okf_last_cuda_error(const okf_ctx *ctx);
/* The context's stream, for callers that want to order their own work on it. */
OKF_API okf_stream okf_ctx_stream(const okf_ctx *ctx);
OKF_API int okf_sync(okf_ctx *ctx);

/* Copy `bytes` of GGUF tensor data (the whole data region, one tensor, or one
 * row shard) into one device allocation.  Synchronous.  Replaces the zero-copy
 * buffer windows of MetalContext.cuts/mapped/window (Base/MetalContext.swift:114-185);
 * woff in the calls below is a byte offset into this buffer, as WeightRef.local is. */
OKF_API int okf_weights_upload(okf_ctx *ctx, const void *host, size_t bytes, okf_weights **out);
/* Adopt device memory the caller already owns (no copy, not freed by the
 * library).  The memory must stay valid while the handle is in use and should
 * be readable for 256 bytes past `bytes` (kernels may fetch whole 16-byte
 * words at the tail). */
OKF_API int okf_weights_wrap(okf_ctx *ctx, const void *device, size_t bytes, okf_weights **out);
OKF_API void okf_weights_free(okf_ctx *ctx, okf_weights *w);
OKF_API const void *okf_weights_device_ptr(const okf_weights *w);
OKF_API size_t okf_weights_bytes(const okf_weights *w);

/* Bytes of one row of K weights: GGUF.rowByteCount (Base/GGUF.swift:160-188).
 * Returns 0 for an unsupported type. */
OKF_API size_t okf_row_bytes(int type, size_t k);

/* out[m] = sum_k W[m][k] * x[k].  Replaces MetalEnc.gemv (Base/MetalEnc.swift:84-93)
 * and its kernels q2_0_gemv / q8_0_gemv / q4_k_gemv / iq2_xxs_gemv
 * (metal/Kernels.metal:26-109, :1572-1655).  x and out are device pointers;
 * x holds K elements of xdt, out holds M floats. */
OKF_API int okf_gemv(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
             const void *x, int xdt, float *out, okf_stream stream);

/* out[n*M + m] = sum_k X[n*K + k] * W[m][k].  Replaces MetalEnc.gemm
 * (Base/MetalEnc.swift:241-289): N == 1 runs the matvec kernel, 2 <= N <= 8
 * the narrow (speculative-verify) kernel (gemmNarrowIQ, MetalEnc.swift:222-239),
 * larger N the tensor-core tile (gemmTiled, MetalEnc.swift:377-400).  X holds
 * N*K elements of xdt; out holds N*M elements of odt (OKF_F32 or OKF_BF16).
 * For deep, short matrices the tile cuts K into ranges whose partial sums live
 * in ONE scratch buffer of the context: calls of one context that may take that
 * route must be ordered on the GPU (same stream, or events between streams).
 * Numerics: for N <= 8 (fp32 out) every 256-wide run of an activation column is
 * reduced to 16-bit integers with one fp32 scale and the sums are exact integers
 * (results within 1e-4 of max|y| of an fp32 evaluation on the test shapes, the
 * same for a column at every N); the tile rounds weights and activations to
 * 16-bit floats and accumulates in fp32 (within 1e-2). */
OKF_API int okf_gemm(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
             const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream);

/* Calls between begin and end have no order among themselves: the reference's
 * MetalEnc.parallel { ... } (Base/MetalEnc.swift:42-47), which the engines wrap
 * around gate || up and q || k || v (Qwen/QwenMetalEngine.swift:464-469, :691-696).
 * Inside a region, okf_gemv / okf_gemm calls with N <= 8 that multiply the same
 * x by matrices of one type and K (up to four) are held back and leave as ONE
 * kernel launch (one per four columns of N), at okf_parallel_end or as soon as
 * a call does not fit the set;
 * every other call runs at once, as outside a region.  A launch error of a
 * held-back call is returned by the call that sends the set off.  Regions do
 * not nest.  Outputs of the region must not alias its inputs. */
OKF_API int okf_parallel_begin(okf_ctx *ctx);
OKF_API int okf_parallel_end(okf_ctx *ctx);

/* ---- row shards on several GPUs -------------------------------------------------
 * The reference runs on one GPU and has no counterpart for this block.  A matrix
 * is cut by output rows, rank r holding rows [row_first, row_first + M) of
 * m_total; every rank computes its rows and the whole output is needed on every
 * rank.  okf_gemm_gather does both in one kernel: each rank stores its rows
 * straight into every rank's copy of the output (pointers mapped from the other
 * processes, plain 16-byte stores over NVLink).  The launch neither fences nor
 * waits.  The exchange is announced (a system-wide fence, then one count on every
 * rank's arrival counter) by a spare warp of the context's next gathered launch
 * or by okf_gather_wait, once the storing kernel is complete, and whoever reads
 * the gathered output waits for the counts:
 *   - the next okf_gemm_gather call of the context waits, inside its kernel and
 *     before it reads x, until the exchange launched before it is complete on
 *     this GPU (its own weights are already streaming in meanwhile);
 *   - okf_gather_wait enqueues that wait as a kernel of its own, for any other
 *     reader (another library's kernel, a copy to the host).
 * So a chain of gathered matvecs needs one okf_gather_wait at its end.  Every
 * wait is bounded (about a second): if a rank never arrives, the waiting kernel
 * carries on and okf_device_status reports 4.  The calls of one context must be
 * issued in the order they run on the GPU (one stream, or streams ordered by
 * events), since the context remembers which exchange came last.
 *   An exchange costs a few NVLink crossings (the stores, their acknowledgement,
 * the count), several microseconds that a chain of dependent matvecs pays once per
 * launch.  A caller whose next x does not depend on rows still in flight (another
 * sequence of a batch, a projection of the same activations) sets
 * OKF_GATHER_FREE: that launch does not wait, and the exchange overlaps the
 * launches that follow.  A wait covers every exchange launched so far on the
 * counter it waits on, so matrices that share one arrival counter and epoch (as
 * tp.PeerOutputs sets them up) are all complete after one okf_gather_wait.
 *
 * Buffers other ranks write into come from okf_shared_alloc (zero-filled), whose
 * handle another process on the same machine turns into a pointer with
 * okf_shared_open.  All ranks must issue the same sequence of calls with the same
 * shapes.  fp32 outputs only.  N <= 8 runs the matvec kernels; more tokens run the
 * tensor-core matmul, whose epilogue stores each finished tile into every rank's
 * output while the other tiles are still being multiplied, so the transfer
 * overlaps the arithmetic (K a multiple of 64 and x 16-byte aligned, else
 * OKF_E_ALIGN).  A buffer must not be written by the next exchange while a rank
 * may still read the previous one: alternate two buffers or order the work. */
typedef struct okf_ipc_handle { unsigned char bytes[64]; } okf_ipc_handle;
typedef struct okf_gather {
    uint32_t nranks;         /* 2..8 */
    uint32_t rank;           /* this process */
    uint32_t m_total;        /* rows of the whole matrix */
    uint32_t row_first;      /* first of this rank's rows */
    float *out[8];           /* rank r's [N][m_total] output, as mapped into this process */
    uint32_t *arrivals[8];   /* rank r's arrival counter (4 bytes, shared; one count per rank and exchange), as mapped here */
    uint32_t *epoch;         /* 8 bytes of this rank's own device memory per counter, zero at start, used by the library */
    uint32_t flags;          /* 0 or OKF_GATHER_FREE */
} okf_gather;
#define OKF_GATHER_FREE 1u   /* x does not depend on an exchange in flight: do not wait for the one before */
OKF_API int okf_shared_alloc(okf_ctx *ctx, size_t bytes, void **device_ptr, okf_ipc_handle *handle);
OKF_API int okf_shared_open(okf_ctx *ctx, const okf_ipc_handle *handle, void **device_ptr);
OKF_API int okf_shared_close(okf_ctx *ctx, void *device_ptr);
OKF_API int okf_shared_free(okf_ctx *ctx, void *device_ptr);
/* Synchronous device -> host copy of `bytes` (for reading shared buffers back). */
OKF_API int okf_copy_to_host(okf_ctx *ctx, const void *device_ptr, void *host, size_t bytes);
OKF_API int okf_gemm_gather(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                            const void *x, int xdt, uint32_t n, const okf_gather *g, okf_stream stream);
/* Enqueue a wait for the exchange this context launched last (nothing if there is
 * none): work that follows on `stream` sees the whole gathered output. */
OKF_API int okf_gather_wait(okf_ctx *ctx, okf_stream stream);

/* Same contract as okf_gemm but always the tensor-core tile, whatever N is.
 * Replaces MetalEnc.gemmTile (Base/MetalEnc.swift:326-352), which the
 * reference's kernel bench uses to time the tile at small N. */
OKF_API int okf_gemm_tile(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                  const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream);

/* The matmul of okf_gemm on the tensor-core tile at every N (the same result as
 * okf_gemm for N >= 9; for N <= 8 okf_gemm runs the narrow integer kernel, which
 * is closer to fp32 than the tile's 16-bit operands), for callers that cannot allocate device memory
 * while they run (inside a stream capture, in a latency-bound decode loop, under
 * a host that forbids cudaMalloc after start-up).  It has no counterpart in the
 * reference.  okf_gemm's tensor-core path keeps the partial sums of its k-ranges
 * in a buffer the context grows with cudaMalloc when a larger shape arrives; this
 * entry point uses a fixed 16 MiB array inside the library image instead (every
 * GPU that loads the library holds it until the process exits) and calls no
 * allocator of any kind.
 *   - N * M must not exceed 2 Mi outputs (2 097 152): larger shapes return
 *     OKF_E_LIMIT.  K must span at least two 64-wide k-blocks, and the pointers
 *     must meet the tensor-core path's alignment (x 16-byte aligned, K a multiple
 *     of 64), else OKF_E_SHAPE / OKF_E_ALIGN.
 *   - The first call on a device looks up the array's device address; make that
 *     call before any stream capture begins.
 *   - All calls on a GPU share the one array, whatever context or stream they come
 *     from: two calls whose kernels overlap on the GPU race on it.  Keep them on
 *     one stream, or otherwise ordered.  Nothing needs clearing between calls. */
OKF_API int okf_gemm_noalloc(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                             const void *x, int xdt, uint32_t n, void *out, int odt, okf_stream stream);

/* Unpack `count` weights starting at a block boundary (woff) to fp32, bit for
 * bit what the reference's block decoders produce.  Replaces
 * MetalEnc.dequantRow (Base/MetalEnc.swift:402-459) and GQ.gather / QB.dequant
 * (Gemma/Gemma4Quant.swift:320-364, Base/Quant.swift:73-76). */
OKF_API int okf_dequant(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint64_t count,
                float *out, okf_stream stream);

/* ---- GGUF files ---------------------------------------------------------------------
 * Replaces GGUF.init (Base/GGUF.swift:92-158): the file is mapped read-only and parsed
 * once; tensors keep the file's order.  dims[0] is the fastest axis (K of a weight
 * matrix), dims[1] its rows (M).  `offset` counts from the start of the data region,
 * which okf_gguf_upload copies to the GPU in one piece (the zero-copy windows of
 * Base/MetalContext.swift:114-185 become one device allocation), so a tensor's offset
 * is the woff of okf_gemv / okf_gemm / okf_dequant / okf_embed_batch.  An id the
 * reference's GGUFType does not know is OKF_E_TYPE, as it is a parse error there. */
typedef struct okf_gguf okf_gguf;
typedef struct okf_gguf_tensor {
    const char *name;   /* owned by the okf_gguf */
    uint32_t n_dims;
    uint64_t dims[4];   /* unused axes are 1 */
    int32_t type;       /* ggml type id */
    uint64_t offset;    /* bytes from the start of the data region */
    uint64_t bytes;     /* GGUF.rowByteCount(type, element count) */
    const void *host;   /* the tensor's bytes in the mapping */
} okf_gguf_tensor;
OKF_API int okf_gguf_open(const char *path, okf_gguf **out);
OKF_API void okf_gguf_close(okf_gguf *g);
OKF_API uint32_t okf_gguf_version(const okf_gguf *g);
OKF_API uint64_t okf_gguf_tensor_count(const okf_gguf *g);
OKF_API int okf_gguf_tensor_at(const okf_gguf *g, uint64_t index, okf_gguf_tensor *out);
OKF_API int okf_gguf_find(const okf_gguf *g, const char *name, okf_gguf_tensor *out); /* OKF_E_RANGE: no such tensor */
OKF_API uint64_t okf_gguf_data_offset(const okf_gguf *g); /* where the data region starts in the file */
OKF_API uint64_t okf_gguf_data_bytes(const okf_gguf *g);
/* Metadata (GGUFValue, Base/GGUF.swift:15-23).  kind: 0 absent, 1 integer, 2 floating
 * point, 3 string, 4 bool, 5 integer array, 6 floating-point array, 7 string table.
 * Strings point into the mapping and are NOT terminated: use the length.  A missing key is
 * OKF_E_RANGE, a key of another kind OKF_E_TYPE (integers read as doubles too). */
OKF_API uint64_t okf_gguf_meta_count(const okf_gguf *g);
OKF_API const char *okf_gguf_meta_key(const okf_gguf *g, uint64_t index);
OKF_API int okf_gguf_meta_kind(const okf_gguf *g, const char *key);
OKF_API int okf_gguf_meta_int(const okf_gguf *g, const char *key, int64_t *out);
OKF_API int okf_gguf_meta_double(const okf_gguf *g, const char *key, double *out);
OKF_API int okf_gguf_meta_string(const okf_gguf *g, const char *key, const char **out, uint64_t *len);
OKF_API int okf_gguf_meta_array(const okf_gguf *g, const char *key, uint64_t *count, const int64_t **ints,
                                const double **doubles);
OKF_API int okf_gguf_meta_string_at(const okf_gguf *g, const char *key, uint64_t index, const char **out,
                                    uint64_t *len);
/* The whole data region into one device allocation (okf_weights_upload of it). */
OKF_API int okf_gguf_upload(okf_ctx *ctx, const okf_gguf *g, okf_weights **out);

/* ---- the linears' neighbours in the engines' command streams ---------------------
 * Small memory-bound operators that read or write the same activations as the
 * quantized linears; all asynchronous on `stream`, device pointers throughout. */

/* out[n][K] = row ids[n] of the embedding matrix (rows x K, any supported type),
 * unpacked bit for bit as okf_dequant does.  Replaces MetalEnc.embedBatch
 * (Base/MetalEnc.swift:1096-1147) and QwenEngine.embed (Qwen/QwenEngine.swift:68-76).
 * An id outside [0, rows) yields a row of zeros and okf_device_status 8. */
OKF_API int okf_embed_batch(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t rows,
                            const int32_t *ids, uint32_t n, float *out, okf_stream stream);

/* out[r] = index of the largest of x[r][0..n); ties go to the lower index, NaNs never
 * win.  Replaces MetalEnc.argmaxRows / argmax_rows (Base/MetalEnc.swift:496-503,
 * metal/Kernels.metal:2756-2794): a verify step keeps its logits on the device. */
OKF_API int okf_argmax_rows(okf_ctx *ctx, const float *x, uint32_t n, uint32_t rows, int32_t *out, okf_stream stream);

/* x[row] += r[row] (r may be NULL: plain RMS norm), then y[row] = x[row] * scale * weight
 * with scale = 1 / sqrt(mean(x[row]^2) + eps); rows are x_stride / y_stride floats apart.
 * Replaces add_rmsnorm_batch / rmsnorm_batch (metal/Kernels.metal:2811-2864) and
 * Kernels.rmsnorm (Base/Kernels.swift:12-20).  `weight` is n floats in device memory. */
OKF_API int okf_add_rmsnorm(okf_ctx *ctx, float *x, const float *r, const float *weight, float *y, uint32_t n,
                            uint32_t rows, float eps, uint32_t x_stride, uint32_t y_stride, okf_stream stream);

/* a[i] = silu(a[i]) * b[i], silu(v) = v / (1 + exp(-v)): the FFN's gate * up.  Replaces
 * silu_mul (metal/Kernels.metal:3280-3285; Qwen/QwenEngine.swift:83). */
OKF_API int okf_silu_mul(okf_ctx *ctx, float *a, const float *b, size_t n, okf_stream stream);

/* One side of gemma's clamp around a linear (SRQ.Side, Gemma/Gemma4Quant.swift:367-377):
 * scale != 0 -> clamp(round_half_even(x / scale), -128, 127) * scale; else lo < hi -> clamp
 * to [lo, hi] without rounding; else inactive. */
typedef struct okf_srq_side { float scale, lo, hi; } okf_srq_side;
/* dst[i] = bound(src[i]); dst may be src.  Replaces srq_to / srq_inplace
 * (metal/Kernels.metal:4743-4767), bit for bit SRQ.apply (Gemma4Quant.swift:413-427). */
OKF_API int okf_srq(okf_ctx *ctx, const float *src, float *dst, size_t n, const okf_srq_side *side, okf_stream stream);
/* clamp the input into `scratch` (n * K floats; only needed when `in` is active), okf_gemm,
 * clamp the output in place: MetalEnc.linear (Base/MetalEnc.swift:762-794).  fp32 x and
 * out.  Three dependent launches: not allowed inside a parallel region (OKF_E_ARG). */
OKF_API int okf_linear(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k, uint32_t m,
                       const float *x, uint32_t n, float *out, const okf_srq_side *in, const okf_srq_side *out_side,
                       float *scratch, okf_stream stream);

/* Host-buffer twins of the CPU operator: QB.matvec (Base/Quant.swift:68-71),
 * GQ.matmul (Gemma/Gemma4Quant.swift:150-170), QB.dequant (Base/Quant.swift:73-76).
 * x / out are HOST pointers to fp32; each call copies x to the device, runs the
 * kernel on the context's stream, copies the result back and waits for it.
 * Pinned host memory makes the copies asynchronous; pageable memory works. */
OKF_API int okf_matvec_host(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k,
                    uint32_t m, const float *x, float *out);
OKF_API int okf_matmul_host(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint32_t k,
                    uint32_t m, const float *x, uint32_t n, float *out);
OKF_API int okf_dequant_host(okf_ctx *ctx, int type, const okf_weights *w, uint64_t woff, uint64_t count,
                     float *out);

/* Stage seeded, host-side faults: afterwards each compute call fails with
 * OKF_E_INJECTED with probability `rate` before anything is launched, so an
 * engine's retry path can be exercised without disturbing the GPU.  rate 0
 * switches it off.  Mirrors GPUGate.simulate(thermal:faultRate:seed:)
 * (Base/MetalGates.swift:101-108). */
OKF_API int okf_fault_inject(okf_ctx *ctx, double rate, uint64_t seed);

/* Waits inside the kernels (on copies landing in shared memory, on other warps)
 * are bounded; one that gives up writes a non-zero code here and the kernel
 * returns early with its outputs incomplete.  Synchronous; call it after the
 * streams that carried the work have been synchronised.  0 = no wait gave up
 * (1, 2, 3: a copy never landed; 4: a rank never arrived; 8: okf_embed_batch met
 * an id outside the matrix).
 * The role of the reference's command-buffer error check in GPUGate.verdict
 * (Base/MetalGates.swift:144-165). */
OKF_API int okf_device_status(okf_ctx *ctx, int *out);

/* Behaviour switches for testing.  OKF_FLAG_SIMPLE_KERNELS routes every call to
 * the plain warp-per-row / fp32-tile kernels, which the fast kernels are
 * checked against on the device.  No counterpart in the reference. */
#define OKF_FLAG_SIMPLE_KERNELS 1u
OKF_API int okf_set_flags(okf_ctx *ctx, uint32_t flags);

/* Number of kernels this context has launched since it was created. */
OKF_API uint64_t okf_launch_count(const okf_ctx *ctx);
/* Number of calls that ran on the plain warp-per-row / fp32-tile kernels because
 * the tensor-core kernels do not take the shape or alignment (K not a multiple
 * of 256 for the matvec or of 64 for the tile, x not 16-byte aligned): correct
 * but many times slower.  A caller that cares about speed checks that this
 * stays 0.  Calls made under OKF_FLAG_SIMPLE_KERNELS are not counted.  No
 * counterpart in the reference. */
OKF_API uint64_t okf_fallback_count(const okf_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* OKF_CUDA_H */
