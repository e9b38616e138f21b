/* dlr_b200 - C ABI of the B200 (sm_100a) DLR-Net forward library.
 *
 * The library computes, for every token row independently and for layers
 * i = 0..L-1 (per-layer math of the reference module, dlr_lock/model.py:93-101):
 *
 *     rstd = rsqrt(mean(h^2) + eps)
 *     z    = (h . V'_i^T) * rstd          V'_i = V_i * rms_w_i     (r x d)
 *     h    = h + silu(z) . U'_i^T         U'_i = alpha_i * U_i     (d x r)
 *
 * on "folded" bf16 weights (gain folded into V, ReZero scalar into U, once,
 * as kernels/reference.py:68-91 does).  All pointers are plain device (or,
 * where stated, host) addresses; there are no framework types in this
 * interface.  Every buffer is owned by the caller, nothing is allocated or
 * kept by the library between calls, and every call is asynchronous on the
 * given CUDA stream unless stated otherwise.
 *
 * What each entry point stands in for in the reference:
 *   dlrb200_forward        - the pybind entry points of the fused kernels,
 *                            e.g. dlrnet_cooperative(x, Vs, Us)
 *                            (kernels/kernels/cuda/cooperative.cu:601-641) and
 *                            its six siblings, and below them the eager loop
 *                            DLRNet._forward_impl (dlr_lock/model.py:93-101).
 *   dlrb200_workspace_bytes- the per-call torch allocations of those entry
 *                            points (cooperative.cu:608-614), hoisted to the
 *                            caller.
 *   dlrb200_query          - the per-batch tile tables of the Python wrappers
 *                            (kernels/kernels/cooperative.py:24-38) and
 *                            kernels/registry.py:130-135.
 *   dlrb200_fold_weights   - pack_dlrnet_weights (kernels/reference.py:68-91).
 *   dlrb200_forward_host   - the same forward for callers whose activations
 *                            live in host memory (no counterpart: the
 *                            reference only takes device tensors).
 */
#ifndef DLR_B200_H
#define DLR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported symbols; everything else in the library has hidden visibility. */
#if defined(__GNUC__)
#define DLRB200_API __attribute__((visibility("default")))
#else
#define DLRB200_API
#endif

/* Return codes.  7 and 8 are also the low byte of the device status word. */
#define DLRB200_OK 0
#define DLRB200_ERR_INVALID_ARG 1
#define DLRB200_ERR_UNSUPPORTED_SHAPE 2
#define DLRB200_ERR_ALIGNMENT 3
#define DLRB200_ERR_WORKSPACE 4
#define DLRB200_ERR_OCCUPANCY 5
#define DLRB200_ERR_CUDA 6
#define DLRB200_ERR_TIMEOUT_BARRIER 7
#define DLRB200_ERR_TIMEOUT_COPY 8
#define DLRB200_ERR_STATIC_LIMIT 9 /* only from dlrb200_forward_static: request larger than its built-in scratch */

/* Execution paths reported by dlrb200_query. */
#define DLRB200_PATH_STRIPED 1 /* small batch: width-striped CTAs, weight streaming, mma.sync */
#define DLRB200_PATH_CLUSTER 2 /* large batch: row tiles on CTA clusters, tcgen05 + tensor memory */
#define DLRB200_PATH_CLUSTER_SMALL 3 /* small batch: one cluster per 2 rows, exchange in distributed shared memory */
#define DLRB200_PATH_STREAMED 4 /* large batch: one CTA per 128-row tile, activations streamed through shared memory */
#define DLRB200_PATH_STRIPED_CLUSTERS 6 /* small batch: width-striped CTAs in clusters of 8, exchange first inside the cluster, then through L2 */
#define DLRB200_PATH_STREAMED_PAIRS 5 /* large batch: one CTA pair per 256-row tile (tcgen05 cta_group::2), activations streamed */

typedef struct dlrb200_plan {
    int path;           /* DLRB200_PATH_* */
    int grid;           /* CTAs per launch */
    int cluster;        /* CTAs per cluster (1 = none) */
    int stripe_cols;    /* columns of the model width owned by one CTA */
    int rows_per_pass;  /* token rows handled by one launch (striped) or one cluster tile */
    int passes;         /* striped path: launches per forward; cluster and streamed paths: waves of row tiles in the one launch */
    int stages;         /* depth of the weight ring, in layers (striped) or tiles (cluster) */
    size_t smem_bytes;  /* dynamic shared memory per CTA */
    size_t workspace_bytes;
} dlrb200_plan;

/* Library version: major*10000 + minor*100 + patch. */
DLRB200_API int dlrb200_version(void);

/* Static, human-readable text for a return code or the low byte of a status word. */
DLRB200_API const char* dlrb200_strerror(int code);

/* The last CUDA runtime/driver error code seen by this thread inside the
 * library (0 if none); for diagnostics after DLRB200_ERR_CUDA. */
DLRB200_API int dlrb200_last_cuda_error(void);

/* Bytes of scratch device memory a forward of this shape needs.  The caller
 * allocates it once (256-byte aligned) and may reuse it for any later call
 * with a shape whose requirement is not larger; calls that share a workspace
 * must not overlap on the GPU.  Returns 0 for an unsupported shape. */
DLRB200_API size_t dlrb200_workspace_bytes(int M, int d, int r, int L);

/* How a forward of this shape would run on the current device.  Launches
 * nothing.  Returns DLRB200_ERR_UNSUPPORTED_SHAPE / _OCCUPANCY when it cannot. */
DLRB200_API int dlrb200_query(int M, int d, int r, int L, dlrb200_plan* plan);

/* y = DLRNet(x).
 *   x, y        (M, d) bf16 row-major device buffers, 16-byte aligned; may not alias.
 *   Vp          (L, r, d) bf16 folded V', 16-byte aligned.
 *   Up          (L, d, r) bf16 folded U', 16-byte aligned.
 *   eps         RMS-norm epsilon (the reference uses 1e-6).
 *   workspace   >= dlrb200_workspace_bytes(M, d, r, L) bytes, 256-byte aligned.
 *   status_dev  one int in device memory, zero before the first call.  It is
 *               written only if a bounded device-side wait gives up:
 *               (layer << 8) | DLRB200_ERR_TIMEOUT_*; the output is then
 *               undefined.  The caller reads it after synchronising (or
 *               mirrors it to host memory with dlrb200_status_to_host).
 *               A non-zero word is also an abort signal: every kernel of the
 *               library that is given this word, on any stream and through
 *               any entry point, makes its waits give up while it is set, so
 *               later calls return undefined output too.  After reading a
 *               non-zero value the caller must set the word back to 0.
 *   stream      a cudaStream_t (NULL = legacy default stream).
 * Supported: d a multiple of 16, r in {16, 32, 64, 128, 256}, M >= 1, L >= 1
 * (M = 0 returns DLRB200_OK and does nothing). */
DLRB200_API int dlrb200_forward(const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L,
                    float eps, void* workspace, size_t workspace_bytes, int* status_dev, void* stream);

/* The same forward for activations in HOST memory: copies x_host (pinned or
 * pageable, M*d bf16) into the caller's device staging buffer x_dev, runs the
 * forward into y_dev, copies the result to y_host, all on `stream`.  The copy
 * back has completed only after the caller synchronises the stream. */
DLRB200_API int dlrb200_forward_host(const void* x_host, void* y_host, void* x_dev, void* y_dev, const void* Vp,
                         const void* Up, int M, int d, int r, int L, float eps, void* workspace,
                         size_t workspace_bytes, int* status_dev, void* stream);

/* Queue a 4-byte copy of the device status word to `status_host` (pinned host
 * memory) on `stream`, behind the forwards already queued there.  A serving
 * loop can then notice a device-side timeout by reading host memory at its next
 * call, without synchronising the stream.  Stands in for the TORCH_CHECK errors
 * of the reference's entry points (kernels/kernels/cuda/cooperative.cu:602-607),
 * which have no device-side failure mode to report because their waits are
 * unbounded. */
DLRB200_API int dlrb200_status_to_host(const int* status_dev, int* status_host, void* stream);

/* Fold the per-layer gain into V and the ReZero scalar into U and stack the
 * result in the layouts dlrb200_forward takes.
 *   V (L, r, d), U (L, d, r), gain (L, d): bf16 device buffers; alpha (L) fp32.
 *   Vp (L, r, d), Up (L, d, r): bf16 outputs.
 * Products are formed in fp32 and rounded once to bf16. */
DLRB200_API int dlrb200_fold_weights(const void* V, const void* U, const void* gain, const float* alpha, void* Vp,
                         void* Up, int d, int r, int L, void* stream);

/* Transpose a stack of L bf16 matrices (rows, cols) -> (cols, rows) on the
 * device; used to accept the reference CUDA convention Us (L, r, d). */
DLRB200_API int dlrb200_transpose_stack(const void* src, void* dst, int L, int rows, int cols, void* stream);

/* Small-batch forward for hosts that must not allocate device memory while
 * serving (no counterpart in the reference, whose entry points allocate their
 * scratch with torch on every call).  Think of a decode server whose memory
 * budget is fixed at start-up, or a bare C caller that has no allocator of its
 * own: a cudaMalloc on the request path would also synchronise the device.
 * This entry point takes no workspace: the exchange scratch of the small-batch
 * kernel lives in a fixed array inside the library's device image
 * (DLRB200_STATIC_SCRATCH_BYTES, held by every GPU that loads the library until
 * the process exits).  It calls no allocating routine.
 *
 *   Arguments as dlrb200_forward, minus workspace / workspace_bytes.
 *   Limits: M <= DLRB200_STATIC_MAX_ROWS rows per call (r up to 256); anything
 *   larger returns DLRB200_ERR_STATIC_LIMIT and launches nothing.  Always runs
 *   the small-batch (striped) path.
 *   First call on a device: looks up the device address of the array (once per
 *   device, with that device current); make that first call before any stream
 *   capture begins.
 *   All calls on a device share the one array: the part a call needs is cleared
 *   on the stream at the start of the call, and two calls that overlap on the
 *   GPU (different streams, no dependency) race - serialise them. */
#define DLRB200_STATIC_MAX_ROWS 64
#define DLRB200_STATIC_SCRATCH_BYTES 221184
DLRB200_API int dlrb200_forward_static(const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                                       int L, float eps, int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DLR_B200_H */
