// Large-batch ("prefill") DLR-Net forward on thread-block clusters with tcgen05
// tensor cores and tensor memory.
//
// Work split.  A cluster of CS = d/256 CTAs (4, 8 or 16) walks all L layers for
// a PAIR of 128-row tiles; CTA `rank` owns columns [256*rank, 256*rank+256) of
// the model width for BOTH contractions of a layer (K-stripe of the V
// contraction, N-stripe of the U contraction - the reference's cooperative
// scheme, kernels/kernels/cuda/cooperative.cu:10-16, moved from global memory
// to distributed shared memory).  Per layer and tile (dlr_lock/model.py:96-100
// on folded weights, kernels/README.md:5-7):
//
//   V:  z_part[128 x r]  = h[128 x 256] . V'[:, stripe]^T     tcgen05.mma, A from TMEM
//   X:  z = sum over the cluster of z_part, sumsq likewise    DSMEM reduce-scatter by rows
//       s = silu(z * rsqrt(sumsq/d + eps)) as bf16            DSMEM all-gather
//   U:  dh[128 x 256]    = s[128 x r] . U'[stripe, :]^T       tcgen05.mma, A and B from smem
//       h += dh ; sumsq_part = sum h^2                        fused epilogue out of TMEM
//
// Two tiles per CTA.  The exchange X is a latency chain during which a tile
// has no tensor work, so every CTA runs TWO independent pipelines, one per row
// tile, each with its own weight ring, TMA warp, MMA warp and four epilogue
// warps; whenever one tile waits on its exchange or epilogue the other tile's
// contractions use the tensor core.  Two issuing warps are also what it takes
// to keep the tensor core busy here: one thread issues a 128x128x16
// tcgen05.mma only every ~130 cycles (measured), half of what the pipe can
// execute.
//
// On-chip residency.  Per tile, 128 tensor-memory columns hold the activation
// stripe as packed bf16 (the A operand of the V contraction, straight from
// TMEM) and 128 columns hold one fp32 accumulator (z, then the two dh chunks).
// The activation is re-rounded to bf16 once per layer, like every fused kernel
// of the reference (fp32 accumulation inside a layer).  Partial z travels
// between CTAs as bf16 (summed in fp32): it is rounded once more to bf16 right
// after the sum anyway, and the end-to-end error is unchanged by it.
//
// Exchange mechanics.  Every remote write is an asynchronous store
// (st.async ... shared::cluster) whose bytes are counted on the RECEIVER's
// mbarrier, so no fences or remote arrivals are needed: a row's partial z
// (bf16) and its partial sum of squares go straight from the accumulator to
// the row's owner; the owner's s rows go to every CTA of the cluster, written
// directly in the core-matrix layout the MMA reads (8 rows x 16 bytes
// contiguous, no swizzle), which also makes each warp's stores contiguous.
//
// Roles.  Per tile: one warp streams 8 KB weight tiles (32 K-columns, 64-byte
// swizzle) with TMA into that tile's ring, one lane of another warp issues the
// tile's MMAs, four warps (one thread per row) run exchange and epilogue.
// Warps 0/1 = TMA/MMA of tile A, 2/3 = TMA/MMA of tile B, 4-7 and 8-11 the two
// epilogue groups.  All waits are bounded mbarrier waits; a wait that gives up
// records a status word and every role drains to a common exit.
#include <cstdlib>
#include <cstring>

#include "cluster.h"
#include "ptx.cuh"

namespace dlr {

namespace {

constexpr int kRows = 128;
constexpr int kStripe = 256;         // columns of the model width per CTA
constexpr int kWK = 32;              // K columns per weight tile (one 64-byte swizzle span)
constexpr int kVT = kStripe / kWK;   // V tiles per layer
constexpr int kNCH = kStripe / 128;  // 128-column output chunks per stripe
constexpr int kStageBytes = 8192;
constexpr int kMaxStages = 8;        // per tile
constexpr int kThreads = 384;
constexpr uint32_t kTileCols = 256;  // tensor-memory columns per tile
constexpr uint32_t kHOff = 0;        // packed bf16 activation: 128 columns
constexpr uint32_t kAccOff = 128;    // fp32 accumulator: 128 columns

struct ClusterParams {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int M, d, L;
    float eps, inv_d;
    int* status;
    unsigned int spin_limit;
    int stages;
    int num_pairs;
    int cs;
    unsigned long long* prof;   // optional per-CTA phase cycle counters (debug), or null
};

template <int R>
struct CCfg {
    static constexpr int S_BYTES = kRows * R * 2;  // s tile (A operand of the U contraction)
    static constexpr int NCK = R / 8;              // 16-byte K chunks per row
    static constexpr int S_GROUP_BYTES = NCK * 128;          // one 8-row group of the s tile
    static constexpr int R_GROUP_BYTES = (NCK + 1) * 128;    // same plus one chunk for the sums of squares
    static constexpr int RECV_BYTES = (kRows / 8) * R_GROUP_BYTES;
    static constexpr int V_TILE_BYTES = R * kWK * 2;         // R rows x 32 K-columns
    static constexpr int U_TILE_BYTES = 128 * kWK * 2;       // 128 rows x 32 K-columns
    static constexpr int UT = R / kWK;                       // U tiles per 128-column chunk
    static constexpr uint32_t W_LAYOUT = 4u;                 // descriptor layout type: 64-byte swizzle
    static constexpr uint32_t W_SBO = 8 * kWK * 2;           // bytes between 8-row groups of a weight tile
};

// per-tile shared-memory bytes besides the ring: the s tile and the receive buffer
__host__ __device__ constexpr int tile_bytes(int R) {
    return kRows * R * 2 + (kRows / 8) * (R / 8 + 1) * 128;
}

// K-major shared-memory operand descriptor: 8-row groups `sbo` bytes apart,
// swizzle span 128 B (layout 2) or 64 B (layout 4); version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t layout, uint32_t sbo) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3ffffu) >> 4);
    d |= uint64_t(1) << 16;
    d |= uint64_t(sbo >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(layout) << 61;
    return d;
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]),
                 "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Asynchronous 16-byte store into a peer's (or this CTA's own) shared memory;
// the 16 bytes are counted on the RECEIVER's mbarrier.  Both addresses are
// shared::cluster addresses from mapa().
__device__ __forceinline__ void st_async_v4(uint32_t dst_cluster, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                            uint32_t bar_cluster) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1,%2,%3,%4}, [%5];" ::"r"(
                     dst_cluster),
                 "r"(a), "r"(b), "r"(c), "r"(d), "r"(bar_cluster)
                 : "memory");
}

// Shared-memory operand descriptor for the un-swizzled K-major layout: core
// matrices of 8 rows x 16 bytes, `lbo` bytes apart along K, `sbo` bytes apart
// along the rows.
__device__ __forceinline__ uint64_t umma_desc_nosw(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3ffffu) >> 4);
    d |= uint64_t(lbo >> 4) << 16;
    d |= uint64_t(sbo >> 4) << 32;
    d |= uint64_t(1) << 46;
    return d;
}

__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1) : "memory");
}

#define DLR_CLK() (p.prof ? clock64() : 0ll)

struct Waiter {
    volatile int* abort_flag;
    uint32_t limit;
    __device__ __forceinline__ bool cta(uint32_t bar, uint32_t parity) const {
        for (uint32_t i = 0; i < limit; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            if ((i & 63u) == 63u && *abort_flag) return false;
        }
        return false;
    }
    __device__ __forceinline__ bool cluster(uint32_t bar, uint32_t parity) const {
        for (uint32_t i = 0; i < limit; ++i) {
            if (mbar_try_wait_cluster(bar, parity)) return true;
            if ((i & 63u) == 63u && *abort_flag) return false;
        }
        return false;
    }
};

// Per-tile mbarriers.
struct TileBars {
    uint64_t z_full;       // MMA -> epilogue: partial z is in the accumulator
    uint64_t recv_full;    // peers -> owner: all partials and sums of squares landed (byte count)
    uint64_t s_full;       // peers -> MMA: the whole s tile landed (byte count)
    uint64_t dh_full;      // MMA -> epilogue: a dh chunk is in the accumulator
    uint64_t acc_empty;    // epilogue -> MMA: accumulator drained
    uint64_t h_ready;      // epilogue -> MMA: activation stripe updated in tensor memory
};

template <int R, int CS>
__global__ void __launch_bounds__(kThreads, 1)
dlr_cluster_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU,
                   ClusterParams p) {
    using C = CCfg<R>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int S = p.stages;                       // ring stages per tile
    constexpr int rows_own = kRows / CS;
    uint8_t* ring = smem;                         // [2][S][kStageBytes]
    uint8_t* tile_mem = ring + size_t(2 * S) * kStageBytes;
    // per tile: [s tile : S_BYTES][recv : RECV_BYTES]
    constexpr int tile_stride = tile_bytes(R);
    uint64_t* bars = reinterpret_cast<uint64_t*>(tile_mem + 2 * size_t(tile_stride));
    uint64_t* ring_full = bars;                   // [2][kMaxStages]
    uint64_t* ring_empty = bars + 2 * kMaxStages; // [2][kMaxStages]
    TileBars* tb = reinterpret_cast<TileBars*>(bars + 4 * kMaxStages);   // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tb + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x / CS;
    const int num_clusters = gridDim.x / CS;
    const int stripe0 = int(rank) * kStripe;
    const Waiter w{abort_flag, p.spin_limit >> 2};

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2 * kMaxStages; ++s) {
            mbar_init(smem_u32(&ring_full[s]), 1);
            mbar_init(smem_u32(&ring_empty[s]), 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(smem_u32(&tb[t].z_full), 1);
            mbar_init(smem_u32(&tb[t].recv_full), 1);   // the local arrive that arms the byte count
            mbar_init(smem_u32(&tb[t].s_full), 1);
            mbar_init(smem_u32(&tb[t].dh_full), 1);
            mbar_init(smem_u32(&tb[t].acc_empty), 128);
            mbar_init(smem_u32(&tb[t].h_ready), 128);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmU);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive_release();
    cluster_wait_acquire();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tile_s = smem_u32(tile_mem);

    int err = 0;
    int err_layer = 0;

    if (warp < 4) {
        const int t = warp >> 1;                  // tile served by this warp
        const uint32_t ring_s = smem_u32(ring) + uint32_t(t * S) * kStageBytes;
        uint64_t* rfull = ring_full + t * kMaxStages;
        uint64_t* rempty = ring_empty + t * kMaxStages;
        if ((warp & 1) == 0) {
            // =============================== TMA producer of tile t =====================
            if (lane == 0) {
                uint32_t n = 0;
                long long pw = 0;
                for (int pair = cluster_id; pair < p.num_pairs && !err; pair += num_clusters) {
                    for (int l = 0; l < p.L && !err; ++l) {
                        for (int i = 0; i < kVT + kNCH * C::UT; ++i, ++n) {
                            const uint32_t st = n % uint32_t(S);
                            const uint32_t ph = (n / uint32_t(S)) & 1u;
                            const long long t0 = DLR_CLK();
                            if (!w.cta(smem_u32(&rempty[st]), ph ^ 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; err_layer = l; break; }
                            pw += DLR_CLK() - t0;
                            const uint32_t bar = smem_u32(&rfull[st]);
                            const uint32_t dst = ring_s + st * kStageBytes;
                            if (i < kVT) {
                                mbar_arrive_expect_tx(bar, C::V_TILE_BYTES);
                                tma_load_2d(dst, &tmV, stripe0 + kWK * i, l * R, bar);
                                // pull the same tile of the NEXT layer into L2 (tile A's producer only:
                                // both tiles read the same weights)
                                if (t == 0 && l + 1 < p.L) tma_prefetch_2d(&tmV, stripe0 + kWK * i, (l + 1) * R);
                            } else {
                                const int j = i - kVT;
                                const int nc = j / C::UT, kq = j % C::UT;
                                mbar_arrive_expect_tx(bar, C::U_TILE_BYTES);
                                tma_load_2d(dst, &tmU, kq * kWK, l * p.d + stripe0 + 128 * nc, bar);
                                if (t == 0 && l + 1 < p.L) tma_prefetch_2d(&tmU, kq * kWK, (l + 1) * p.d + stripe0 + 128 * nc);
                            }
                        }
                    }
                }
                if (p.prof) p.prof[(blockIdx.x * 6 + t) * 16 + 0] = (unsigned long long)pw;
                if (err) {
                    // copies issued before giving up still land in this CTA's ring:
                    // wait (bounded) for them before leaving.
                    for (uint32_t back = 1; back <= uint32_t(S) && back <= n; ++back) {
                        const uint32_t m = n - back;
                        mbar_wait(smem_u32(&rfull[m % uint32_t(S)]), (m / uint32_t(S)) & 1u, p.spin_limit >> 6);
                    }
                }
            }
        } else {
            // =============================== MMA issuer of tile t =======================
            if (lane == 0) {
                const uint32_t idesc_v = umma_idesc_bf16(128, R);
                const uint32_t idesc_u = umma_idesc_bf16(128, 128);
                const uint32_t tcol = tmem_base + uint32_t(t) * kTileCols;
                const uint32_t sb = tile_s + uint32_t(t) * uint32_t(tile_stride);
                uint32_t n = 0;                      // ring position of the next weight tile
                uint32_t c_h = 0, c_s = 0, c_e = 0;
                long long m[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                const long long mstart = DLR_CLK();
                for (int pair = cluster_id; pair < p.num_pairs && !err; pair += num_clusters) {
                    for (int l = 0; l < p.L && !err; ++l) {
                        err_layer = l;
                        // ---- V contraction: accumulator = h . V'^T over the 8 K tiles of the stripe
                        long long t0 = DLR_CLK();
                        if (!w.cta(smem_u32(&tb[t].h_ready), c_h & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        ++c_h;
                        tc_fence_after();
                        long long t1 = DLR_CLK();
                        m[0] += t1 - t0;
                        for (int kt = 0; kt < kVT && !err; ++kt, ++n) {
                            const uint32_t st = n % uint32_t(S);
                            const long long r0 = DLR_CLK();
                            if (!w.cta(smem_u32(&rfull[st]), (n / uint32_t(S)) & 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                            m[4] += DLR_CLK() - r0;
                            tc_fence_after();
                            const uint64_t bdesc = umma_desc(ring_s + st * kStageBytes, C::W_LAYOUT, C::W_SBO);
#pragma unroll
                            for (int k = 0; k < kWK / 16; ++k)
                                umma_ts(tcol + kAccOff, tcol + kHOff + uint32_t(kt * (kWK / 2) + k * 8), bdesc + uint64_t(2 * k),
                                        idesc_v, (kt | k) ? 1u : 0u);
                            umma_commit(smem_u32(&rempty[st]));
                        }
                        if (err) break;
                        umma_commit(smem_u32(&tb[t].z_full));
                        t0 = DLR_CLK();
                        m[1] += t0 - t1;
                        // ---- U contraction: two 128-column chunks through the one accumulator
                        if (!w.cluster(smem_u32(&tb[t].s_full), c_s & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        ++c_s;
                        tc_fence_after();
                        t1 = DLR_CLK();
                        m[2] += t1 - t0;
                        for (int nc = 0; nc < kNCH && !err; ++nc) {
                            const long long a0 = DLR_CLK();
                            if (!w.cta(smem_u32(&tb[t].acc_empty), c_e & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                            ++c_e;
                            tc_fence_after();
                            m[6] += DLR_CLK() - a0;
                            for (int kq = 0; kq < C::UT && !err; ++kq, ++n) {
                                const uint32_t st = n % uint32_t(S);
                                const long long r0 = DLR_CLK();
                                if (!w.cta(smem_u32(&rfull[st]), (n / uint32_t(S)) & 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                                m[5] += DLR_CLK() - r0;
                                tc_fence_after();
                                const uint64_t bdesc = umma_desc(ring_s + st * kStageBytes, C::W_LAYOUT, C::W_SBO);
#pragma unroll
                                for (int k = 0; k < kWK / 16; ++k) {
                                    // K step ks of the s tile: two 16-byte chunks, 128 bytes apart
                                    const int ks = kq * (kWK / 16) + k;
                                    const uint64_t adesc = umma_desc_nosw(sb + uint32_t(ks) * 256u, 128u, C::S_GROUP_BYTES);
                                    umma_ss(tcol + kAccOff, adesc, bdesc + uint64_t(2 * k), idesc_u, (kq | k) ? 1u : 0u);
                                }
                                umma_commit(smem_u32(&rempty[st]));
                            }
                            if (err) break;
                            umma_commit(smem_u32(&tb[t].dh_full));
                        }
                        m[3] += DLR_CLK() - t1;
                    }
                }
                if (p.prof) {
                    m[7] = DLR_CLK() - mstart;
                    for (int k = 0; k < 8; ++k) p.prof[(blockIdx.x * 6 + 2 + t) * 16 + k] = (unsigned long long)m[k];
                }
            }
        }
    } else {
        // =============================== epilogue warps =============================
        const int t = (warp - 4) >> 2;               // tile served by this warp group
        const int gw = (warp - 4) & 3;               // warp inside the group
        const int gt = gw * 32 + lane;               // thread inside the group, 0..127
        const int q = warp & 3;                      // tensor-memory lane quadrant of this warp
        const int er = 32 * q + lane;                // row of the tile this thread owns
        const uint32_t tl = tmem_base + uint32_t(t) * kTileCols + (uint32_t(32 * q) << 16);
        const uint32_t sbuf_s = tile_s + uint32_t(t) * uint32_t(tile_stride);
        const uint32_t recv_s = sbuf_s + C::S_BYTES;
        const uint8_t* recv_g = tile_mem + size_t(t) * tile_stride + C::S_BYTES;
        TileBars& B = tb[t];
        const int owner = er / rows_own;
        const int lr = er % rows_own;
        constexpr int groups_own = rows_own / 8;         // 8-row groups per owner
        constexpr uint32_t src_bytes = uint32_t(groups_own) * C::R_GROUP_BYTES;   // one source's block in recv
        constexpr int items = rows_own * C::NCK / 128;   // 16-byte chunks of s per thread in the reduce
        uint32_t c_z = 0, c_recv = 0, c_dh = 0;
        long long e[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long estart = DLR_CLK();

        for (int pair = cluster_id; pair < p.num_pairs && !err; pair += num_clusters) {
            const int grow = (2 * pair + t) * kRows + er;
            const bool valid = grow < p.M;
            const long long x0 = DLR_CLK();
            const __nv_bfloat16* xrow = p.x + size_t(valid ? grow : 0) * p.d + stripe0;
            float ssq = 0.f;
            // ---- input stripe -> tensor memory (packed bf16), partial sum of squares
#pragma unroll 4
            for (int c = 0; c < kStripe / 16; ++c) {
                uint32_t v[8];
                if (valid) {
                    const uint4 a = __ldg(reinterpret_cast<const uint4*>(xrow + 16 * c));
                    const uint4 b = __ldg(reinterpret_cast<const uint4*>(xrow + 16 * c + 8));
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
                } else {
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float lo = bf16lo_to_f(v[j]), hi = bf16hi_to_f(v[j]);
                    ssq += lo * lo + hi * hi;
                }
                tmem_st8(tl + kHOff + uint32_t(8 * c), v);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&B.h_ready));
            e[6] += DLR_CLK() - x0;

            for (int l = 0; l < p.L && !err; ++l) {
                err_layer = l;
                long long t0 = DLR_CLK();
                // ---- partial z of this row: accumulator -> bf16 -> the row's owner
                if (!__all_sync(0xffffffffu, w.cta(smem_u32(&B.z_full), c_z & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                ++c_z;
                tc_fence_after();
                long long t1 = DLR_CLK();
                e[0] += t1 - t0;
                if (gt == 0) mbar_arrive_expect_tx(smem_u32(&B.recv_full), C::RECV_BYTES);   // arm this layer's receive
                {
                    // this row's slot in its owner's receive buffer: [source][8-row group][chunk][row in group]
                    const uint32_t dst = mapa(recv_s + uint32_t(rank) * src_bytes + uint32_t(lr >> 3) * C::R_GROUP_BYTES +
                                                  uint32_t(lr & 7) * 16u, uint32_t(owner));
                    const uint32_t rbar = mapa(smem_u32(&B.recv_full), uint32_t(owner));
#pragma unroll
                    for (int c = 0; c < R / 32; ++c) {
                        uint32_t v[32];
                        tmem_ld32(tl + kAccOff + uint32_t(32 * c), v);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            st_async_v4(dst + uint32_t(4 * c + j) * 128u,
                                        pack_bf16x2(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1])),
                                        pack_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                                        pack_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                                        pack_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])), rbar);
                    }
                    st_async_v4(dst + uint32_t(C::NCK) * 128u, __float_as_uint(ssq), 0u, 0u, 0u, rbar);
                }
                tc_fence_before();
                mbar_arrive(smem_u32(&B.acc_empty));     // z has left the accumulator
                t0 = DLR_CLK();
                e[1] += t0 - t1;

                // ---- owner: sum the CS partials of its rows, normalise, SiLU, all-gather
                if (!__all_sync(0xffffffffu, w.cluster(smem_u32(&B.recv_full), c_recv & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                ++c_recv;
                t1 = DLR_CLK();
                e[2] += t1 - t0;
                if (gt == 0) mbar_arrive_expect_tx(smem_u32(&B.s_full), C::S_BYTES);      // arm this layer's s tile
#pragma unroll
                for (int it = 0; it < items; ++it) {
                    const int i = gt + 128 * it;
                    const int r8 = i & 7;
                    const int c = (i >> 3) % C::NCK;
                    const int gl = i / R;                 // 8-row group inside this owner's rows
                    const uint8_t* base = recv_g + size_t(gl) * C::R_GROUP_BYTES + r8 * 16;
                    float tot = 0.f;
                    float a[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
                    for (int src = 0; src < CS; ++src) {
                        const uint8_t* bp = base + size_t(src) * src_bytes;
                        const uint4 u = *reinterpret_cast<const uint4*>(bp + c * 128);
                        tot += *reinterpret_cast<const float*>(bp + C::NCK * 128);
                        a[0] += bf16lo_to_f(u.x); a[1] += bf16hi_to_f(u.x);
                        a[2] += bf16lo_to_f(u.y); a[3] += bf16hi_to_f(u.y);
                        a[4] += bf16lo_to_f(u.z); a[5] += bf16hi_to_f(u.z);
                        a[6] += bf16lo_to_f(u.w); a[7] += bf16hi_to_f(u.w);
                    }
                    const float rstd = rsqrtf(tot * p.inv_d + p.eps);
                    const uint32_t p0 = pack_bf16x2(silu_f(a[0] * rstd), silu_f(a[1] * rstd));
                    const uint32_t p1 = pack_bf16x2(silu_f(a[2] * rstd), silu_f(a[3] * rstd));
                    const uint32_t p2 = pack_bf16x2(silu_f(a[4] * rstd), silu_f(a[5] * rstd));
                    const uint32_t p3 = pack_bf16x2(silu_f(a[6] * rstd), silu_f(a[7] * rstd));
                    // row (rank*rows_own + 8*gl + r8) of the s tile, chunk c, in every CTA of the cluster
                    const uint32_t soff = uint32_t(int(rank) * groups_own + gl) * C::S_GROUP_BYTES + uint32_t(c) * 128u +
                                          uint32_t(r8) * 16u;
#pragma unroll
                    for (int dc = 0; dc < CS; ++dc)
                        st_async_v4(mapa(sbuf_s + soff, uint32_t(dc)), p0, p1, p2, p3,
                                    mapa(smem_u32(&B.s_full), uint32_t(dc)));
                }
                t0 = DLR_CLK();
                e[3] += t0 - t1;

                // ---- fused epilogue of the U contraction: h += dh, new sum of squares
                float ssq_new = 0.f;
                for (int nc = 0; nc < kNCH && !err; ++nc) {
                    const long long d0 = DLR_CLK();
                    if (!__all_sync(0xffffffffu, w.cta(smem_u32(&B.dh_full), c_dh & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_dh;
                    tc_fence_after();
                    e[4] += DLR_CLK() - d0;
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t dh[32], hp[16];
                        tmem_ld32(tl + kAccOff + uint32_t(32 * c), dh);
                        tmem_ld16(tl + kHOff + uint32_t(64 * nc + 16 * c), hp);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float lo = bf16lo_to_f(hp[j]) + __uint_as_float(dh[2 * j]);
                            const float hi = bf16hi_to_f(hp[j]) + __uint_as_float(dh[2 * j + 1]);
                            ssq_new += lo * lo + hi * hi;
                            hp[j] = pack_bf16x2(lo, hi);
                        }
                        tmem_st16(tl + kHOff + uint32_t(64 * nc + 16 * c), hp);
                    }
                    if (nc + 1 < kNCH) {
                        tc_fence_before();
                        mbar_arrive(smem_u32(&B.acc_empty));
                    }
                }
                if (err) break;
                ssq = ssq_new;
                tmem_wait_st();
                if (l + 1 < p.L) {
                    tc_fence_before();
                    mbar_arrive(smem_u32(&B.h_ready));
                }
                e[5] += DLR_CLK() - t0;
            }
            if (err) break;
            // ---- final activation stripe -> global
            __nv_bfloat16* yrow = p.y + size_t(valid ? grow : 0) * p.d + stripe0;
#pragma unroll 4
            for (int c = 0; c < kStripe / 16; ++c) {
                uint32_t v[8];
                tmem_ld8(tl + kHOff + uint32_t(8 * c), v);
                tmem_wait_ld();
                if (valid) {
                    *reinterpret_cast<uint4*>(yrow + 16 * c) = make_uint4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<uint4*>(yrow + 16 * c + 8) = make_uint4(v[4], v[5], v[6], v[7]);
                }
            }
        }
        if (p.prof && gt == 0) {
            e[7] = DLR_CLK() - estart;
            for (int k = 0; k < 8; ++k) p.prof[(blockIdx.x * 6 + 4 + t) * 16 + k] = (unsigned long long)e[k];
        }
    }

    if (err) {
        *abort_flag = 1;
        atomicCAS(p.status, 0, err | (err_layer << 8));
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    // no CTA may leave while a peer can still write into its shared memory
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int R, int CS>
int launch_cluster(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int L, float eps,
                   int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
                   dlrb200_plan* plan_only, unsigned long long* prof) {
    using C = CCfg<R>;
    auto kern = dlr_cluster_kernel<R, CS>;
    const int cs = CS;
    if (d != CS * kStripe) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    const int fixed = 2 * tile_bytes(R) + 1024 /*barriers*/ + 1024 /*alignment*/;
    int stages = (smem_optin - fixed) / (2 * kStageBytes);      // per tile
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 3) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    const int smem = 2 * stages * kStageBytes + fixed;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return DLRB200_ERR_CUDA;
    if (cs > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return DLRB200_ERR_CUDA;

    const int num_tiles = (M + kRows - 1) / kRows;
    const int num_pairs = (num_tiles + 1) / 2;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(cs * (num_sms / cs));
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) return DLRB200_ERR_CUDA;
    if (max_clusters < 1) return DLRB200_ERR_OCCUPANCY;
    const int clusters = num_pairs < max_clusters ? num_pairs : max_clusters;
    cfg.gridDim = dim3(cs * clusters);
    if (plan_only) {
        plan_only->path = DLRB200_PATH_CLUSTER;
        plan_only->grid = cs * clusters;
        plan_only->cluster = cs;
        plan_only->stripe_cols = kStripe;
        plan_only->rows_per_pass = 2 * kRows;
        plan_only->passes = 1;
        plan_only->stages = stages;
        plan_only->smem_bytes = size_t(smem);
        return DLRB200_OK;
    }

    ClusterParams p;
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.y = static_cast<__nv_bfloat16*>(y);
    p.M = M; p.d = d; p.L = L; p.eps = eps; p.inv_d = 1.0f / float(d);
    p.status = status_dev;
    p.spin_limit = spin_limit;
    p.stages = stages;
    p.num_pairs = num_pairs;
    p.cs = cs;
    p.prof = prof;
    CUtensorMap tmV, tmU;
    if (!encode_2d_bf16(enc, &tmV, Vp, uint64_t(d), uint64_t(L) * R, kWK, R, kWK * 2) ||
        !encode_2d_bf16(enc, &tmU, Up, uint64_t(R), uint64_t(L) * d, kWK, 128, kWK * 2))
        return DLRB200_ERR_CUDA;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, tmV, tmU, p);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

int dispatch(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L, float eps,
             int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
             dlrb200_plan* plan_only, unsigned long long* prof) {
#define DLR_CASE(RR, CC)                                                                                          \
    if (r == RR && d == CC * kStripe)                                                                             \
        return launch_cluster<RR, CC>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin,   \
                                      spin_limit, plan_only, prof);
    DLR_CASE(32, 4)
    DLR_CASE(64, 4)
    DLR_CASE(64, 8)
    DLR_CASE(128, 4)
    DLR_CASE(128, 8)
    DLR_CASE(128, 16)
#undef DLR_CASE
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

// Debug aid: with DLRB200_PROFILE=1 in the environment every CTA writes cycle
// counts of its phases (6 roles x 16 counters) at offset 256 of the workspace.
constexpr size_t kProfBytes = 256 + size_t(256) * 6 * 16 * 8;

bool profiling() {
    const char* v = std::getenv("DLRB200_PROFILE");
    return v && *v && *v != '0';
}

}  // namespace

bool cluster_supported(int d, int r, int L) {
    (void)L;
    if (d % kStripe != 0) return false;
    const int cs = d / kStripe;
    if (!(cs == 4 || cs == 8 || cs == 16)) return false;
    if (!(r == 32 || r == 64 || r == 128)) return false;
    return r / cs >= 8;
}

size_t cluster_workspace_bytes(int, int, int, int) { return profiling() ? kProfBytes : 0; }

int cluster_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan) {
    const size_t ws = plan->workspace_bytes;
    const int rc = dispatch(nullptr, nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, num_sms,
                            smem_optin, 0, plan, nullptr);
    plan->workspace_bytes = ws;
    return rc;
}

int cluster_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                    int L, float eps, void* workspace, int* status_dev, cudaStream_t stream, int num_sms,
                    int smem_optin, unsigned int spin_limit) {
    unsigned long long* prof = nullptr;
    if (profiling() && workspace) {
        if (cudaMemsetAsync(workspace, 0, kProfBytes, stream) != cudaSuccess) return DLRB200_ERR_CUDA;
        prof = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(workspace) + 256);
    }
    return dispatch(encode_fn_ptr, x, y, Vp, Up, M, d, r, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit,
                    nullptr, prof);
}

}  // namespace dlr
