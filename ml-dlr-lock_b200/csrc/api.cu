// C-ABI layer: argument checks, path selection, tensor-map encoding, launches.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "cluster.h"
#include "decode.h"
#include "decode_cluster.h"
#include "decode_tl.h"
#include "stream.h"
#include "stream_pair.h"

namespace {

thread_local int g_last_cuda_error = 0;

inline bool cuda_ok(cudaError_t e) {
    if (e != cudaSuccess) {
        g_last_cuda_error = int(e);
        (void)cudaGetLastError();
        return false;
    }
    return true;
}

struct DevInfo {
    int num_sms = 0;
    int smem_optin = 0;
    int cc_major = 0;
    int l2_bytes = 0;
    bool ok = false;
};

DevInfo g_dev[64];
std::mutex g_dev_mutex;

// Device facts are cached per device index; the only process-wide state.
int device_info(DevInfo* out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return DLRB200_ERR_CUDA;
    if (dev < 0 || dev >= 64) return DLRB200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DevInfo& d = g_dev[dev];
    if (!d.ok) {
        if (!cuda_ok(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev)) ||
            !cuda_ok(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) ||
            !cuda_ok(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev)) ||
            !cuda_ok(cudaDeviceGetAttribute(&d.l2_bytes, cudaDevAttrL2CacheSize, dev)))
            return DLRB200_ERR_CUDA;
        d.ok = true;
    }
    *out = d;
    return DLRB200_OK;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static std::atomic<EncodeTiledFn> cached{nullptr};
    EncodeTiledFn f = cached.load(std::memory_order_acquire);
    if (f) return f;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (!cuda_ok(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q)) ||
        q != cudaDriverEntryPointSuccess || !p)
        return nullptr;
    f = reinterpret_cast<EncodeTiledFn>(p);
    cached.store(f, std::memory_order_release);
    return f;
}

int env_int(const char* name, int dflt) {
    const char* v = std::getenv(name);
    return (v && *v) ? std::atoi(v) : dflt;
}

bool supported_rank(int r) { return r == 16 || r == 32 || r == 64 || r == 128 || r == 256; }

// Stripe width of the small-batch path.  Every CTA adds its partial z into the same accumulator words, so
// the exchange costs L2 atomics in proportion to the number of stripes: wide stripes win as long as a CTA
// can still pull its share of the weights in time.  Measured at M = 1 / 8 (us): d = 4096: 310 / 432 with 64
// columns against 418 / 664 with 32; d = 2048: 277 / 325 against 269 / 361; d = 1024: 271 / 302 (64), 263 / 296
// (32), 258 / 320 (16).  All CTAs must be co-resident (one per SM).
int pick_stripe_cols(int d, int num_sms) {
    const int forced = env_int("DLRB200_STRIPE_COLS", 0);
    // a forced width obeys the same limit: one CTA per SM, and the per-CTA words of the workspace are sized for
    // at most 160 CTAs
    if (forced == 16 || forced == 32 || forced == 64)
        return (d % forced == 0 && d / forced <= num_sms && d / forced <= 160) ? forced : 0;
    const int want = d >= 2048 ? 64 : 32;
    for (int dc : {64, 32, 16})
        if (dc <= want && d % dc == 0 && d / dc <= num_sms && d / dc <= 160) return dc;
    return 0;
}

constexpr size_t kCtrlBytes = 256;

size_t striped_workspace_bytes(int r) { return kCtrlBytes + dlr::decode_zacc_floats(r) * sizeof(float); }

unsigned int spin_limit() { return unsigned(env_int("DLRB200_SPIN_LIMIT", 1 << 21)); }

int striped_forward(const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L,
                    float eps, void* workspace, int* status_dev, cudaStream_t stream, const DevInfo& di) {
    const int dc = pick_stripe_cols(d, di.num_sms);
    if (dc == 0) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return DLRB200_ERR_CUDA;

    dlr::DecodeLaunch a;
    std::memset(&a, 0, sizeof(a));
    int vbc, vbr, ubc, ubr, vsw, usw;
    if (!dlr::decode_box_dims(r, dc, &vbc, &vbr, &ubc, &ubr, &vsw, &usw)) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    if (!dlr::encode_2d_bf16(reinterpret_cast<void*>(enc), &a.tmV, Vp, uint64_t(d), uint64_t(L) * r, vbc, vbr, vsw) ||
        !dlr::encode_2d_bf16(reinterpret_cast<void*>(enc), &a.tmU, Up, uint64_t(r), uint64_t(L) * d, ubc, ubr, usw)) {
        g_last_cuda_error = -1;
        return DLRB200_ERR_CUDA;
    }
    a.d = d; a.r = r; a.L = L; a.dc = dc;
    a.num_sms = di.num_sms;
    a.smem_optin = di.smem_optin;
    a.max_stages = env_int("DLRB200_MAX_STAGES", 0);
    a.stream = stream;

    uint8_t* ws = static_cast<uint8_t*>(workspace);
    a.p.d = d; a.p.L = L; a.p.eps = eps; a.p.inv_d = 1.0f / float(d);
    a.p.counter = reinterpret_cast<unsigned int*>(ws);
    a.p.zacc = reinterpret_cast<float*>(ws + kCtrlBytes);
    a.p.status = status_dev;
    a.p.spin_limit = spin_limit();

    const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* yb = static_cast<__nv_bfloat16*>(y);
    for (int row0 = 0; row0 < M; row0 += 64) {
        const int rows = (M - row0 < 64) ? (M - row0) : 64;
        const int mp = rows <= 8 ? 8 : (rows <= 16 ? 16 : (rows <= 32 ? 32 : 64));
        // up to 16 rows the accumulator words are 64-bit (counted exchange), otherwise fp32
        const size_t clear = kCtrlBytes + size_t(3) * mp * (r + 4) * (mp <= 16 ? sizeof(unsigned long long) : sizeof(float));
        if (!cuda_ok(cudaMemsetAsync(ws, 0, clear, stream))) return DLRB200_ERR_CUDA;
        a.p.x = xb + size_t(row0) * d;
        a.p.y = yb + size_t(row0) * d;
        a.p.M = rows;
        const int rc = dlr::decode_launch(a);
        if (rc != DLRB200_OK) {
            if (rc == DLRB200_ERR_CUDA) g_last_cuda_error = int(cudaGetLastError());
            return rc;
        }
    }
    return DLRB200_OK;
}

// The striped kernel with the two-level exchange (clusters of 8 first reduce among themselves): what small
// batches beyond a few rows run on.  Measured at d = 4096, r = 128, L = 143 (us): see use_striped_clusters.
int striped_tl_launch(const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L, float eps,
                      void* workspace, int* status_dev, cudaStream_t stream, const DevInfo& di, dlrb200_plan* plan_only) {
    const int dc = pick_stripe_cols(d, di.num_sms);
    if (dc == 0 || !dlr::decode_tl_supported(d, r, dc)) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    dlr::DecodeTLLaunch a;
    std::memset(&a, 0, sizeof(a));
    a.d = d; a.r = r; a.L = L; a.dc = dc;
    a.num_sms = di.num_sms;
    a.smem_optin = di.smem_optin;
    a.stream = stream;
    a.p.M = M; a.p.d = d; a.p.L = L; a.p.eps = eps; a.p.inv_d = 1.0f / float(d);
    a.p.status = status_dev;
    a.p.spin_limit = spin_limit();
    if (plan_only) return dlr::decode_tl_launch(a, plan_only);
    EncodeTiledFn enc = encode_fn();
    if (!enc) return DLRB200_ERR_CUDA;
    int vbc, vbr, ubc, ubr, vsw, usw;
    if (!dlr::decode_box_dims(r, dc, &vbc, &vbr, &ubc, &ubr, &vsw, &usw)) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    if (!dlr::encode_2d_bf16(reinterpret_cast<void*>(enc), &a.tmV, Vp, uint64_t(d), uint64_t(L) * r, vbc, vbr, vsw) ||
        !dlr::encode_2d_bf16(reinterpret_cast<void*>(enc), &a.tmU, Up, uint64_t(r), uint64_t(L) * d, ubc, ubr, usw)) {
        g_last_cuda_error = -1;
        return DLRB200_ERR_CUDA;
    }
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const size_t clear = dlr::decode_tl_clear_bytes(M, r, L);
    if (!cuda_ok(cudaMemsetAsync(ws, 0, clear, stream))) return DLRB200_ERR_CUDA;
    a.p.x = static_cast<const __nv_bfloat16*>(x);
    a.p.y = static_cast<__nv_bfloat16*>(y);
    a.p.counter = reinterpret_cast<unsigned int*>(ws);
    a.p.words = reinterpret_cast<unsigned long long*>(ws + 256);
    a.p.pre = reinterpret_cast<float*>(ws + clear);
    const int rc = dlr::decode_tl_launch(a, nullptr);
    if (rc == DLRB200_ERR_CUDA) g_last_cuda_error = int(cudaGetLastError());
    return rc;
}

__global__ void fold_v_kernel(const __nv_bfloat16* __restrict__ V, const __nv_bfloat16* __restrict__ gain,
                              __nv_bfloat16* __restrict__ Vp, int d, int r, size_t total) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t layer = i / (size_t(r) * d);
    const int col = int(i % d);
    Vp[i] = __float2bfloat16_rn(__bfloat162float(V[i]) * __bfloat162float(gain[layer * d + col]));
}

__global__ void fold_u_kernel(const __nv_bfloat16* __restrict__ U, const float* __restrict__ alpha,
                              __nv_bfloat16* __restrict__ Up, int d, int r, size_t total) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t layer = i / (size_t(r) * d);
    Up[i] = __float2bfloat16_rn(__bfloat162float(U[i]) * alpha[layer]);
}

__global__ void transpose_stack_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                       int rows, int cols) {
    __shared__ __nv_bfloat16 tile[32][33];
    const size_t base = size_t(blockIdx.z) * rows * cols;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int rr = r0 + j, cc = c0 + threadIdx.x;
        if (rr < rows && cc < cols) tile[j][threadIdx.x] = src[base + size_t(rr) * cols + cc];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int cc = c0 + j, rr = r0 + threadIdx.x;
        if (rr < rows && cc < cols) dst[base + size_t(cc) * rows + rr] = tile[threadIdx.x][j];
    }
}

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int check_shape(int M, int d, int r, int L) {
    if (M < 0 || d <= 0 || r <= 0 || L <= 0) return DLRB200_ERR_INVALID_ARG;
    if (d % 16 != 0 || !supported_rank(r)) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    return DLRB200_OK;
}

// Which path serves a large batch (M > 64).  Three kernels apply to most shapes:
//   cluster kernel   activations resident in tensor memory, the width split over a cluster of d/512 CTAs,
//                    one exchange per layer; holds one 128-row tile per cluster, so 8192 rows at d = 4096 are
//                    five waves on 15 clusters
//   streamed kernel  whole rows per cluster of 1, 2 or 4 CTAs, activations streamed through L2
//   pair kernel      the streamed data flow on CTA pairs (256-row tiles, tcgen05 cta_group::2), two pairs per
//                    cluster when that still fits the GPU
// All were timed on a B200 over widths 512..8192, ranks 64 and 128 and 512..32768 rows; the choice is a cost
// model fitted to those times (microseconds):
//   cluster   waves * L * t_layer, t_layer = 8.2 (r = 128) or 6.4 (r = 64) whatever the width
//   streamed  waves * (L + 1) * (chunks per CTA * t_chunk + t_pass), t_chunk = 1.26 (r = 128) or 1.15 (r = 64),
//             t_pass = 2.5 / 5.5 / 6.8 for a split of 1 / 2 / 4 (normalise + SiLU, and the exchange); 30 % more
//             when over 100 unsplit CTAs stream weights that do not fit in L2
//   pairs     waves * (L + 1) * (chunks per pair * t_chunk + t_pass), t_chunk = 1.09 (r = 128) or 0.80 (r = 64),
//             t_pass = 4.4 with two pairs per cluster (exchange in distributed shared memory), 2.5 with one.
//             One pair per cluster at rank 128 means at least 9000 rows, where the activations no longer fit in
//             L2 and the unsplit streamed kernel is as fast or faster: not taken there.
// At d = 4096, r = 128, L = 143 (ms, cluster / streamed / pairs): 2048 rows 2.34 / 2.47 / 3.09, 4096 rows
// 3.55 / 2.49 / 3.08, 6144 rows 4.72 / 3.66 / 3.10, 8192 rows 6.37 / 3.86 / 3.14, 16384 rows 12.1 / 7.97 / 8.71.
// At d = 2048, r = 64, L = 142: 8192 rows 1.82 / 1.98 / 1.51, 16384 rows 3.66 / 2.97 / 2.70.
// Shapes the cluster kernel does not cover (d > 4096, d not a multiple of 512, r > d / 32) stream.
struct RouteEntry {
    int tiles, d, r, L, sms, path;         // the plans depend on M only through the number of 128-row tiles
};
constexpr int kRouteSlots = 32;
RouteEntry g_route[kRouteSlots];
int g_route_n = 0;          // entries in use
int g_route_next = 0;       // slot the next new shape goes to (oldest first once the table is full)
std::mutex g_route_mutex;

// DLRB200_PATH_* of the kernel that serves M > 64 rows, or 0 when none of the large-batch kernels applies
// (then the striped kernel runs in 64-row launches).
int large_batch_path(int M, int d, int r, int L, const DevInfo& di) {
    const int forced = env_int("DLRB200_FORCE_PATH", 0);
    if (M <= 64) return 0;
    const bool can_stream = dlr::stream_supported(d, r);
    const bool can_pair = dlr::stream_pair_supported(d, r);
    const bool can_cluster = dlr::cluster_supported(d, r, L);
    if (forced == DLRB200_PATH_STREAMED) return can_stream ? forced : 0;
    if (forced == DLRB200_PATH_STREAMED_PAIRS) return can_pair ? forced : 0;
    if (forced == DLRB200_PATH_CLUSTER) return can_cluster ? forced : 0;
    if (forced != 0) return 0;
    if (!can_stream && !can_pair) return can_cluster ? DLRB200_PATH_CLUSTER : 0;
    const int tiles = (M + 127) / 128;
    {   // the plans below ask the driver for occupancy: remember the answer per shape
        std::lock_guard<std::mutex> lock(g_route_mutex);
        for (int i = 0; i < g_route_n; ++i) {
            const RouteEntry& e = g_route[i];
            if (e.tiles == tiles && e.d == d && e.r == r && e.L == L && e.sms == di.num_sms) return e.path;
        }
    }
    double best = 1e30;
    int path = 0;
    dlrb200_plan pl;
    if (can_cluster) {
        std::memset(&pl, 0, sizeof(pl));
        if (dlr::cluster_plan(M, d, r, L, di.num_sms, di.smem_optin, &pl) == DLRB200_OK) {
            best = 0.97 * double(pl.passes) * L * (r >= 128 ? 8.2 : 6.4);     // ties go to the cluster kernel
            path = DLRB200_PATH_CLUSTER;
        }
    }
    if (can_stream) {
        std::memset(&pl, 0, sizeof(pl));
        if (dlr::stream_plan(M, d, r, L, di.num_sms, di.smem_optin, &pl) == DLRB200_OK) {
            const double t_pass = pl.cluster >= 4 ? 6.8 : (pl.cluster == 2 ? 5.5 : 2.5);
            double t = double(pl.passes) * (L + 1) * (double(d / 128 / pl.cluster) * (r >= 128 ? 1.26 : 1.15) + t_pass);
            if (pl.cluster == 1 && pl.grid > 100 && 4.0 * L * d * r > 100e6) t *= 1.3;
            // every layer rewrites the rows in flight in place: once they outgrow L2 (beside the weight stream)
            // each layer's traffic goes to DRAM (measured at d = 4096: 12288 / 16384 / 18944 rows in flight
            // cost 1.11 / 1.24 / 1.41 times the estimate)
            if (di.l2_bytes > 0) {
                const double ratio = double(pl.grid / pl.cluster) * 128.0 * d * 2.0 / double(di.l2_bytes);
                if (ratio > 0.62) t *= 1.0 + 0.65 * (ratio - 0.62);
            }
            if (t < best) { best = t; path = DLRB200_PATH_STREAMED; }
        }
    }
    if (can_pair) {
        std::memset(&pl, 0, sizeof(pl));
        if (dlr::stream_pair_plan(M, d, r, L, di.num_sms, di.smem_optin, &pl) == DLRB200_OK) {
            const int pp = pl.cluster / 2;
            // (measured only where the pairs cover most of the GPU: not taken for smaller grids)
            if (pp == 4 || ((pp == 2 || r == 64) && pl.grid >= 96)) {
                const double pause = (r >= 128 ? 3.4 : 2.0) + (pp == 4 ? 2.8 : (pp == 2 ? 1.0 : 0.0));
                const double t = double(pl.passes) * (L + 1) * (double(d / 128 / pp) * (r >= 128 ? 1.09 : 0.80) + pause);
                if (t < best) { best = t; path = DLRB200_PATH_STREAMED_PAIRS; }
            }
        }
    }
    std::lock_guard<std::mutex> lock(g_route_mutex);
    g_route[g_route_next] = RouteEntry{tiles, d, r, L, di.num_sms, path};
    g_route_next = (g_route_next + 1) % kRouteSlots;
    if (g_route_n < kRouteSlots) ++g_route_n;
    return path;
}

bool use_stream_path(int M, int d, int r, int L, const DevInfo& di) {
    return large_batch_path(M, d, r, L, di) == DLRB200_PATH_STREAMED;
}

bool use_pair_path(int M, int d, int r, int L, const DevInfo& di) {
    return large_batch_path(M, d, r, L, di) == DLRB200_PATH_STREAMED_PAIRS;
}

bool use_cluster_path(int M, int d, int r, int L) {
    const int forced = env_int("DLRB200_FORCE_PATH", 0);
    if (forced == DLRB200_PATH_STRIPED || forced == DLRB200_PATH_STREAMED || forced == DLRB200_PATH_CLUSTER_SMALL ||
        forced == DLRB200_PATH_STREAMED_PAIRS)
        return false;
    if (!dlr::cluster_supported(d, r, L)) return false;
    if (forced == DLRB200_PATH_CLUSTER) return true;
    // One 128-row tile on one cluster costs the same for any M <= 128 (1.16 ms at d = 4096, r = 128, L = 143),
    // while the striped kernel grows with M (about 0.35 + 0.0153 M ms there): from about 52 rows on, the padded
    // tile is the faster way.  At d = 2048 the striped kernel stays ahead up to 64 rows (0.76 against 0.89 ms).
    if (M > 64) return true;
    return M >= 52 && d >= 4096;
}

// Small batches: the cluster kernel (one cluster per pair of rows, exchange in
// distributed shared memory) or the striped kernel (all SMs on every row,
// exchange through global memory).  Measured on B200, L about 142 (us): d = 1024:
// cluster kernel 291 for every M <= 64 against 263 (M = 1), 297 (M = 2..8), 349
// (M = 16), 490 (M = 64) striped; d = 2048: 386 for M <= 32 against 277 (M = 1),
// 325 (M = 8), 344 (M = 16) and about 530 (M = 32) striped; d = 4096: 625 against
// 310 (a cluster of 16 SMs cannot pull 2 MB of weights per layer fast enough).
// All its clusters must be resident at once to share the weight stream through
// L2, hence the cap on the grid.  DLRB200_FORCE_PATH=1 or 3 overrides the choice.
bool use_cluster_small(int M, int d, int r) {
    const int forced = env_int("DLRB200_FORCE_PATH", 0);
    if (forced == DLRB200_PATH_STRIPED || forced == DLRB200_PATH_CLUSTER) return false;
    if (M > 64 || !dlr::decode_cluster_supported(d, r)) return false;
    if (forced == DLRB200_PATH_CLUSTER_SMALL) return true;
    const int grid = ((M + 1) / 2) * (d / 256);
    if (grid > 128) return false;
    return (d <= 1024 && M >= 2) || (d <= 2048 && M > 16);
}

// Small batches on the striped kernel with the two-level exchange (decode_tl.cu).  Measured on a B200, L about
// 143, against the best of the other small-batch kernels (us): d = 4096, r = 128: 665 against 719 at 17 rows,
// 754 / 853 at 32, 1012 / 1177 at 48, 1109 / 1184 at 64 (there the other is one padded 128-row tile on one
// cluster), but 452 / 349 at one row and 598 / 554 at 16: its two hops through distributed shared memory cost
// more than they save while the counted exchange of decode.cu applies.  d = 5120, r = 256: 785 / 933 at 16 rows,
// 1117 / 1390 at 32 (more rows do not fit its shared memory).  d = 2048, r = 64: 585 / 794 at 32 rows, 735 / 759
// at 48, 787 / 832 at 64, but 561 / 422 at 17 (cluster-small kernel).  d = 1024: never.
// DLRB200_FORCE_PATH=6 forces it wherever it applies.
bool use_striped_clusters(int M, int d, int r, int L, const DevInfo& di) {
    const int forced = env_int("DLRB200_FORCE_PATH", 0);
    if (M > 64) return false;
    if (forced != 0 && forced != DLRB200_PATH_STRIPED_CLUSTERS) return false;
    if (forced == 0) {
        const int from = d >= 4096 ? (r >= 256 ? 16 : 17) : (d >= 2048 ? 29 : 65);
        if (M < from) return false;
    }
    dlrb200_plan pl;
    std::memset(&pl, 0, sizeof(pl));
    return striped_tl_launch(nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, nullptr, di, &pl) == DLRB200_OK;
}

}  // namespace

namespace dlr {

bool encode_2d_bf16(void* encode_fn_ptr, CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer,
                    int box_inner, int box_outer, int swizzle_bytes) {
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(encode_fn_ptr);
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {cuuint32_t(box_inner), cuuint32_t(box_outer)};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
    if (swizzle_bytes == 32) sw = CU_TENSOR_MAP_SWIZZLE_32B;
    else if (swizzle_bytes == 64) sw = CU_TENSOR_MAP_SWIZZLE_64B;
    else if (swizzle_bytes == 128) sw = CU_TENSOR_MAP_SWIZZLE_128B;
    else return false;
    const CUresult rc = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

}  // namespace dlr

extern "C" {

int dlrb200_version(void) { return 100; }

const char* dlrb200_strerror(int code) {
    switch (code & 0xff) {
        case DLRB200_OK: return "ok";
        case DLRB200_ERR_INVALID_ARG: return "invalid argument (null pointer or non-positive size)";
        case DLRB200_ERR_UNSUPPORTED_SHAPE: return "unsupported shape (d must be a multiple of 16, r one of 16/32/64/128/256, and the stripes must fit the device)";
        case DLRB200_ERR_ALIGNMENT: return "misaligned buffer (activations and weights need 16-byte, the workspace 256-byte alignment)";
        case DLRB200_ERR_WORKSPACE: return "workspace too small";
        case DLRB200_ERR_OCCUPANCY: return "the grid cannot be made co-resident on this device";
        case DLRB200_ERR_CUDA: return "CUDA runtime or driver error (see dlrb200_last_cuda_error)";
        case DLRB200_ERR_TIMEOUT_BARRIER: return "device-side wait on the per-layer exchange gave up";
        case DLRB200_ERR_TIMEOUT_COPY: return "device-side wait on a weight copy gave up";
        case DLRB200_ERR_STATIC_LIMIT: return "request exceeds the built-in scratch of dlrb200_forward_static (at most 64 rows per call)";
    }
    return "unknown error";
}

int dlrb200_last_cuda_error(void) { return g_last_cuda_error; }

size_t dlrb200_workspace_bytes(int M, int d, int r, int L) {
    if (check_shape(M, d, r, L) != DLRB200_OK) return 0;
    size_t need = striped_workspace_bytes(r);
    const size_t tl = dlr::decode_tl_workspace_bytes(M, r, L);
    if (tl > need) need = tl;
    const size_t c = dlr::cluster_workspace_bytes(M, d, r, L);
    if (c > need) need = c;
    const size_t st = dlr::stream_workspace_bytes(M, d, r);
    if (st > need) need = st;
    return (need + 255) & ~size_t(255);
}

int dlrb200_query(int M, int d, int r, int L, dlrb200_plan* plan) {
    if (!plan) return DLRB200_ERR_INVALID_ARG;
    int rc = check_shape(M, d, r, L);
    if (rc != DLRB200_OK) return rc;
    DevInfo di;
    rc = device_info(&di);
    if (rc != DLRB200_OK) return rc;
    std::memset(plan, 0, sizeof(*plan));
    plan->workspace_bytes = dlrb200_workspace_bytes(M, d, r, L);
    if (use_pair_path(M, d, r, L, di)) return dlr::stream_pair_plan(M, d, r, L, di.num_sms, di.smem_optin, plan);
    if (use_stream_path(M, d, r, L, di)) return dlr::stream_plan(M, d, r, L, di.num_sms, di.smem_optin, plan);
    if (use_striped_clusters(M, d, r, L, di)) {
        const size_t ws = plan->workspace_bytes;
        rc = striped_tl_launch(nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, nullptr, di, plan);
        plan->workspace_bytes = ws;
        return rc;
    }
    if (use_cluster_path(M, d, r, L)) return dlr::cluster_plan(M, d, r, L, di.num_sms, di.smem_optin, plan);
    if (use_cluster_small(M, d, r)) return dlr::decode_cluster_plan(M, d, r, L, di.smem_optin, plan);
    const int dc = pick_stripe_cols(d, di.num_sms);
    if (dc == 0) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    plan->path = DLRB200_PATH_STRIPED;
    plan->grid = d / dc;
    plan->cluster = 1;
    plan->stripe_cols = dc;
    plan->rows_per_pass = M < 64 ? M : 64;
    plan->passes = (M + 63) / 64;
    return DLRB200_OK;
}

int dlrb200_forward(const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L,
                    float eps, void* workspace, size_t workspace_bytes, int* status_dev, void* stream) {
    int rc = check_shape(M, d, r, L);
    if (rc != DLRB200_OK) return rc;
    if (M == 0) return DLRB200_OK;
    if (!x || !y || !Vp || !Up || !workspace || !status_dev || x == y) return DLRB200_ERR_INVALID_ARG;
    if (!aligned(x, 16) || !aligned(y, 16) || !aligned(Vp, 16) || !aligned(Up, 16) || !aligned(workspace, 256) ||
        !aligned(status_dev, 4))
        return DLRB200_ERR_ALIGNMENT;
    if (workspace_bytes < dlrb200_workspace_bytes(M, d, r, L)) return DLRB200_ERR_WORKSPACE;
    DevInfo di;
    rc = device_info(&di);
    if (rc != DLRB200_OK) return rc;
    if (di.cc_major != 10) return DLRB200_ERR_CUDA;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (use_pair_path(M, d, r, L, di) && dlr::stream_aligned(x, y)) {
        EncodeTiledFn enc = encode_fn();
        if (!enc) return DLRB200_ERR_CUDA;
        rc = dlr::stream_pair_forward(reinterpret_cast<void*>(enc), x, y, Vp, Up, M, d, r, L, eps, status_dev, st, di.num_sms,
                                      di.smem_optin, spin_limit(),
                                      env_int("DLRB200_PROFILE", 0) ? reinterpret_cast<unsigned long long*>(
                                                                          static_cast<uint8_t*>(workspace) + 256)
                                                                    : nullptr);
        if (rc == DLRB200_ERR_CUDA) g_last_cuda_error = int(cudaGetLastError());
        return rc;
    }
    if (use_stream_path(M, d, r, L, di) && dlr::stream_aligned(x, y)) {
        EncodeTiledFn enc = encode_fn();
        if (!enc) return DLRB200_ERR_CUDA;
        rc = dlr::stream_forward(reinterpret_cast<void*>(enc), x, y, Vp, Up, M, d, r, L, eps, workspace, status_dev, st, di.num_sms,
                                 di.smem_optin, spin_limit(),
                                 env_int("DLRB200_PROFILE", 0) ? reinterpret_cast<unsigned long long*>(
                                                                     static_cast<uint8_t*>(workspace) + 256)
                                                               : nullptr);
        if (rc == DLRB200_ERR_CUDA) g_last_cuda_error = int(cudaGetLastError());
        return rc;
    }
    if (use_striped_clusters(M, d, r, L, di))
        return striped_tl_launch(x, y, Vp, Up, M, d, r, L, eps, workspace, status_dev, st, di, nullptr);
    if (use_cluster_path(M, d, r, L)) {
        EncodeTiledFn enc = encode_fn();
        if (!enc) return DLRB200_ERR_CUDA;
        rc = dlr::cluster_forward(reinterpret_cast<void*>(enc), x, y, Vp, Up, M, d, r, L, eps, workspace, status_dev,
                                  st, di.num_sms, di.smem_optin, spin_limit());
        if (rc == DLRB200_ERR_CUDA) g_last_cuda_error = int(cudaGetLastError());
        return rc;
    }
    if (use_cluster_small(M, d, r)) {
        EncodeTiledFn enc = encode_fn();
        if (!enc) return DLRB200_ERR_CUDA;
        rc = dlr::decode_cluster_forward(reinterpret_cast<void*>(enc), x, y, Vp, Up, M, d, r, L, eps, status_dev, st,
                                         di.smem_optin, spin_limit(),
                                         env_int("DLRB200_PROFILE", 0) ? reinterpret_cast<unsigned long long*>(
                                                                             static_cast<uint8_t*>(workspace) + 256)
                                                                       : nullptr);
        if (rc == DLRB200_ERR_CUDA) g_last_cuda_error = int(cudaGetLastError());
        return rc;
    }
    return striped_forward(x, y, Vp, Up, M, d, r, L, eps, workspace, status_dev, st, di);
}

int dlrb200_forward_host(const void* x_host, void* y_host, void* x_dev, void* y_dev, const void* Vp,
                         const void* Up, int M, int d, int r, int L, float eps, void* workspace,
                         size_t workspace_bytes, int* status_dev, void* stream) {
    if (!x_host || !y_host) return DLRB200_ERR_INVALID_ARG;
    if (M <= 0 || d <= 0) return M == 0 ? DLRB200_OK : DLRB200_ERR_INVALID_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t bytes = size_t(M) * d * 2;
    if (!x_dev || !y_dev) return DLRB200_ERR_INVALID_ARG;
    if (!cuda_ok(cudaMemcpyAsync(x_dev, x_host, bytes, cudaMemcpyHostToDevice, st))) return DLRB200_ERR_CUDA;
    const int rc = dlrb200_forward(x_dev, y_dev, Vp, Up, M, d, r, L, eps, workspace, workspace_bytes, status_dev,
                                   stream);
    if (rc != DLRB200_OK) return rc;
    if (!cuda_ok(cudaMemcpyAsync(y_host, y_dev, bytes, cudaMemcpyDeviceToHost, st))) return DLRB200_ERR_CUDA;
    return DLRB200_OK;
}

int dlrb200_status_to_host(const int* status_dev, int* status_host, void* stream) {
    if (!status_dev || !status_host) return DLRB200_ERR_INVALID_ARG;
    return cuda_ok(cudaMemcpyAsync(status_host, status_dev, sizeof(int), cudaMemcpyDeviceToHost,
                                   static_cast<cudaStream_t>(stream)))
               ? DLRB200_OK
               : DLRB200_ERR_CUDA;
}

int dlrb200_fold_weights(const void* V, const void* U, const void* gain, const float* alpha, void* Vp,
                         void* Up, int d, int r, int L, void* stream) {
    if (!V || !U || !gain || !alpha || !Vp || !Up || d <= 0 || r <= 0 || L <= 0) return DLRB200_ERR_INVALID_ARG;
    const size_t total = size_t(L) * r * d;
    const int threads = 256;
    const unsigned blocks = unsigned((total + threads - 1) / threads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    fold_v_kernel<<<blocks, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(V),
                                              static_cast<const __nv_bfloat16*>(gain),
                                              static_cast<__nv_bfloat16*>(Vp), d, r, total);
    fold_u_kernel<<<blocks, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(U), alpha,
                                              static_cast<__nv_bfloat16*>(Up), d, r, total);
    return cuda_ok(cudaGetLastError()) ? DLRB200_OK : DLRB200_ERR_CUDA;
}

int dlrb200_transpose_stack(const void* src, void* dst, int L, int rows, int cols, void* stream) {
    if (!src || !dst || L <= 0 || rows <= 0 || cols <= 0 || src == dst) return DLRB200_ERR_INVALID_ARG;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, L), block(32, 8);
    transpose_stack_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), rows, cols);
    return cuda_ok(cudaGetLastError()) ? DLRB200_OK : DLRB200_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Forward without any caller- or library-side allocation.
//
// The exchange scratch of the small-batch kernel (arrival counter + three
// accumulator slots of 64 rows x (256+4) floats) sits in this fixed array in the
// library's device image.  Host code may not hand `g_static_scratch` to a
// kernel: on the host that name is only a handle for the symbol, not a device
// address.  The address is fetched with cudaGetSymbolAddress, once per device
// and with that device current, and cached below.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[DLRB200_STATIC_SCRATCH_BYTES];

namespace {
void* g_static_ptr[64] = {};
std::mutex g_static_mutex;

// Device address of the scratch array on the current device (set-up on first use).
int static_scratch_ptr(void** out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return DLRB200_ERR_CUDA;
    if (dev < 0 || dev >= 64) return DLRB200_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&p, g_static_scratch)) || !p) return DLRB200_ERR_CUDA;
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return DLRB200_OK;
}
}  // namespace

int dlrb200_forward_static(const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L,
                           float eps, int* status_dev, void* stream) {
    int rc = check_shape(M, d, r, L);
    if (rc != DLRB200_OK) return rc;
    if (M == 0) return DLRB200_OK;
    if (M > DLRB200_STATIC_MAX_ROWS || striped_workspace_bytes(r) > size_t(DLRB200_STATIC_SCRATCH_BYTES))
        return DLRB200_ERR_STATIC_LIMIT;
    if (!x || !y || !Vp || !Up || !status_dev || x == y) return DLRB200_ERR_INVALID_ARG;
    if (!aligned(x, 16) || !aligned(y, 16) || !aligned(Vp, 16) || !aligned(Up, 16) || !aligned(status_dev, 4))
        return DLRB200_ERR_ALIGNMENT;
    DevInfo di;
    rc = device_info(&di);
    if (rc != DLRB200_OK) return rc;
    if (di.cc_major != 10) return DLRB200_ERR_CUDA;
    void* scratch = nullptr;
    rc = static_scratch_ptr(&scratch);
    if (rc != DLRB200_OK) return rc;
    // the striped launcher clears the counter and the accumulator slots it uses on the
    // stream before the kernel, so whatever the previous call left behind does not matter
    return striped_forward(x, y, Vp, Up, M, d, r, L, eps, scratch, status_dev, static_cast<cudaStream_t>(stream), di);
}

}  // extern "C"
