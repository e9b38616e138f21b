// Large-batch ("prefill") DLR-Net forward on thread-block clusters with tcgen05
// tensor cores and tensor memory.
//
// Work split.  A cluster of CS = d/512 CTAs (1, 2, 4 or 8) walks all L layers
// for one tile of 128 token rows; CTA `rank` owns columns [512*rank,
// 512*rank+512) of the model width for BOTH contractions of a layer (K-stripe
// of the V contraction, N-stripe of the U contraction - the reference's
// cooperative scheme, kernels/kernels/cuda/cooperative.cu:10-16, moved from
// global memory to distributed shared memory).  Per layer
// (dlr_lock/model.py:96-100 on folded weights, kernels/README.md:5-7):
//
//   V:  z_part[128 x r]  = h[128 x 512] . V'[:, stripe]^T     tcgen05.mma, A from TMEM
//   X:  z = sum over the cluster of z_part, sumsq likewise    DSMEM reduce-scatter by rows
//       s = silu(z * rsqrt(sumsq/d + eps)) as bf16            DSMEM all-gather
//   U:  dh[128 x 512]    = s[128 x r] . U'[stripe, :]^T       tcgen05.mma, A and B from smem
//       h += dh ; sumsq_part = sum h^2                        fused epilogue out of TMEM
//
// On-chip residency.  256 tensor-memory columns hold the activation stripe
// (128 x 512) as packed bf16 for the whole stack - it is the A operand of the V
// contraction straight from TMEM - and the other 256 columns are two fp32
// accumulators of 128 columns.  The activation is re-rounded to bf16 once per
// layer, like every fused kernel of the reference (fp32 accumulation inside a
// layer).  Partial z travels between CTAs as bf16 (summed in fp32): it is
// rounded to bf16 right after the sum anyway, and the end-to-end error is
// unchanged by it.
//
// Two MMA warps.  One thread can issue a 128xNx16 tcgen05.mma only about every
// 125 cycles for any N <= 128 (measured), half of what the tensor pipe executes
// at N = 128, while two issuing warps run side by side at full rate.  So the V
// contraction is split along K over two warps into the two accumulators (the
// halves are added when z is read out), and the four 128-column chunks of the
// U contraction alternate between the two warps and accumulators.
//
// Exchange mechanics.  Every remote write is an asynchronous store
// (st.async ... shared::cluster) whose bytes are counted on the RECEIVER's
// mbarrier, so no fences or remote arrivals are needed: a row's partial z
// (bf16) and its partial sum of squares go straight from the accumulators to
// the row's owner; the owner's s rows go to every CTA of the cluster, written
// directly in the core-matrix layout the MMA reads (8 rows x 16 bytes
// contiguous, no swizzle), which also makes each warp's stores contiguous.
//
// Roles.  Warp 0 streams 16 KB weight tiles with TMA into a deep ring and
// never waits for activations; warps 1 and 2 issue MMAs; warps 4-11 (two
// threads per row, each taking half of the columns) run exchange and epilogue.
// All waits are bounded mbarrier waits; a wait that gives up records a status
// word and every role drains to a common exit.
#include <cstdlib>
#include <cstring>

#include "cluster.h"
#include "ptx.cuh"

namespace dlr {

namespace {

constexpr int kRows = 128;
constexpr int kKT = 8;               // 64-column K tiles per stripe
constexpr int kStripe = 64 * kKT;    // 512 columns per CTA
constexpr int kNCH = kStripe / 128;  // 128-column output chunks per stripe
constexpr int kStageBytes = 16384;
constexpr int kMaxStages = 12;
constexpr int kThreads = 384;
constexpr int kEpi = 256;            // epilogue threads
constexpr uint32_t kHOff = 0;        // packed bf16 activation: 256 columns
constexpr uint32_t kAcc0 = 256;      // fp32 accumulator 0 (accumulator 1 follows at +128)

struct ClusterParams {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int M, d, L;
    float eps, inv_d;
    int* status;
    unsigned int spin_limit;
    int stages;
    int num_tiles;
    unsigned long long* prof;   // optional per-CTA phase cycle counters (debug), or null
};

template <int R>
struct CCfg {
    static constexpr int KW = R < 64 ? R : 64;     // K columns per U weight tile
    static constexpr int UK = R / KW;              // U weight tiles per 128-column chunk
    static constexpr int S_BYTES = kRows * R * 2;  // s tile (A operand of the U contraction)
    static constexpr int NCK = R / 8;              // 16-byte K chunks per row
    static constexpr int S_GROUP_BYTES = NCK * 128;          // one 8-row group of the s tile
    static constexpr int R_GROUP_BYTES = (NCK + 2) * 128;    // same plus two chunks for the sums of squares
    static constexpr int RECV_BYTES = (kRows / 8) * R_GROUP_BYTES;
    static constexpr int V_TILE_BYTES = R * 128;             // R rows x 64 K-columns, 128-byte swizzle
    static constexpr int U_TILE_BYTES = 128 * KW * 2;        // 128 rows x KW K-columns
    static constexpr uint32_t U_LAYOUT = KW == 64 ? 2u : 4u; // descriptor layout type (128- / 64-byte swizzle)
    static constexpr uint32_t U_SBO = 8 * KW * 2;            // bytes between 8-row groups of a U tile
    static constexpr int LOADS_PER_LAYER = kKT + kNCH * UK;
    static constexpr int FIXED_BYTES = S_BYTES + RECV_BYTES + 1024 /*barriers*/ + 1024 /*alignment*/;
};

#define DLR_CLK() (p.prof ? clock64() : 0ll)

struct Bars {
    uint64_t ring_full[kMaxStages];
    uint64_t ring_empty[kMaxStages];
    uint64_t z_full[2];      // MMA warp b -> epilogue: its half of the partial z is in accumulator b
    uint64_t recv_full;      // peers -> owner: all partials and sums of squares landed (byte count)
    uint64_t s_full;         // peers -> MMA warps: the whole s tile landed (byte count)
    uint64_t dh_full[2];     // MMA warp b -> epilogue: a dh chunk is in accumulator b
    uint64_t acc_empty[2];   // epilogue -> MMA warp b: accumulator b drained
    uint64_t h_ready;        // epilogue -> MMA warps: activation stripe updated in tensor memory
};

template <int R, int CS>
__global__ void __launch_bounds__(kThreads, 1)
dlr_cluster_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU,
                   ClusterParams p) {
    using C = CCfg<R>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int S = p.stages;
    constexpr int rows_own = kRows / CS;
    uint8_t* ring = smem;
    uint8_t* sbuf = ring + size_t(S) * kStageBytes;   // s tile, core-matrix layout
    uint8_t* recv = sbuf + C::S_BYTES;                // [source][8-row group][chunk][row in group] x 16 B
    Bars* bars = reinterpret_cast<Bars*>(recv + C::RECV_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x / CS;
    const int num_clusters = gridDim.x / CS;
    const int stripe0 = int(rank) * kStripe;
    const Waiter w{abort_flag, p.spin_limit >> 2};

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(smem_u32(&bars->ring_full[s]), 1);
            mbar_init(smem_u32(&bars->ring_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->z_full[b]), 1);
            mbar_init(smem_u32(&bars->dh_full[b]), 1);
            mbar_init(smem_u32(&bars->acc_empty[b]), kEpi);
        }
        mbar_init(smem_u32(&bars->recv_full), 1);   // the local arrive that arms the byte count
        mbar_init(smem_u32(&bars->s_full), 1);
        mbar_init(smem_u32(&bars->h_ready), kEpi);
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
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t sbuf_s = smem_u32(sbuf);
    const uint32_t recv_s = smem_u32(recv);

    int err = 0;
    int err_layer = 0;

    if (warp == 0) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            uint32_t n = 0;
            RingPos rp;
            long long pw = 0;
            for (int tile = cluster_id; tile < p.num_tiles && !err; tile += num_clusters) {
                for (int l = 0; l < p.L && !err; ++l) {
                    for (int i = 0; i < C::LOADS_PER_LAYER; ++i, ++n, rp.step(uint32_t(S))) {
                        const uint32_t st = rp.st;
                        const uint32_t ph = rp.ph;
                        const long long t0 = DLR_CLK();
                        if (!w.cta(smem_u32(&bars->ring_empty[st]), ph ^ 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; err_layer = l; break; }
                        pw += DLR_CLK() - t0;
                        const uint32_t bar = smem_u32(&bars->ring_full[st]);
                        const uint32_t dst = ring_s + st * kStageBytes;
                        if (i < kKT) {
                            mbar_arrive_expect_tx(bar, C::V_TILE_BYTES);
                            tma_load_2d(dst, &tmV, stripe0 + 64 * i, l * R, bar);
                        } else {
                            const int j = i - kKT;
                            const int nc = j / C::UK, kh = j % C::UK;
                            mbar_arrive_expect_tx(bar, C::U_TILE_BYTES);
                            tma_load_2d(dst, &tmU, kh * C::KW, l * p.d + stripe0 + 128 * nc, bar);
                        }
                    }
                }
            }
            if (p.prof) p.prof[(blockIdx.x * 4 + 0) * 16 + 0] = (unsigned long long)pw;
            if (err) {
                // copies issued before giving up still land in this CTA's ring:
                // wait (bounded) for them before leaving.
                for (uint32_t back = 1; back <= uint32_t(S) && back <= n; ++back) {
                    const uint32_t m = n - back;
                    mbar_wait(smem_u32(&bars->ring_full[m % uint32_t(S)]), (m / uint32_t(S)) & 1u, kDrainPolls);
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // =============================== MMA issuer b ===============================
        // b = 0: K tiles 0-3 of the V contraction, U chunks 0 and 2, accumulator 0
        // b = 1: K tiles 4-7,                       U chunks 1 and 3, accumulator 1
        if (lane == 0) {
            const int b = warp - 1;
            const uint32_t acc = tmem_base + kAcc0 + uint32_t(b) * 128u;
            const uint32_t idesc_v = umma_idesc_bf16(128, R);
            const uint32_t idesc_u = umma_idesc_bf16(128, 128);
            RingPos rb;                          // ring position of this layer's first weight tile
            uint32_t c_h = 0, c_s = 0, c_e = 0;
            long long m[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            const long long mstart = DLR_CLK();
            for (int tile = cluster_id; tile < p.num_tiles && !err; tile += num_clusters) {
                for (int l = 0; l < p.L && !err; ++l, rb.advance(uint32_t(C::LOADS_PER_LAYER), uint32_t(S))) {
                    err_layer = l;
                    long long t0 = DLR_CLK();
                    if (!w.cta(smem_u32(&bars->h_ready), c_h & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_h;
                    tc_fence_after();
                    long long t1 = DLR_CLK();
                    m[0] += t1 - t0;
                    // ---- this warp's half of the V contraction
                    for (int kk = 0; kk < kKT / 2 && !err; ++kk) {
                        const int kt = b * (kKT / 2) + kk;
                        const RingPos rq = rb.at(uint32_t(kt), uint32_t(S));
                        const uint32_t st = rq.st;
                        const long long r0 = DLR_CLK();
                        if (!w.cta(smem_u32(&bars->ring_full[st]), rq.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                        m[4] += DLR_CLK() - r0;
                        tc_fence_after();
                        const uint64_t bdesc = umma_desc(ring_s + st * kStageBytes, 2u, 1024u);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_ts(acc, tmem_base + kHOff + uint32_t(kt * 32 + k * 8), bdesc + uint64_t(2 * k), idesc_v,
                                    (kk | k) ? 1u : 0u);
                        umma_commit(smem_u32(&bars->ring_empty[st]));
                    }
                    if (err) break;
                    umma_commit(smem_u32(&bars->z_full[b]));
                    t0 = DLR_CLK();
                    m[1] += t0 - t1;
                    // ---- this warp's two chunks of the U contraction
                    if (!w.cluster(smem_u32(&bars->s_full), c_s & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_s;
                    tc_fence_after();
                    t1 = DLR_CLK();
                    m[2] += t1 - t0;
                    for (int j = 0; j < kNCH / 2 && !err; ++j) {
                        const int nc = b + 2 * j;
                        const long long a0 = DLR_CLK();
                        if (!w.cta(smem_u32(&bars->acc_empty[b]), c_e & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        ++c_e;
                        tc_fence_after();
                        m[6] += DLR_CLK() - a0;
                        for (int kh = 0; kh < C::UK && !err; ++kh) {
                            const RingPos rq = rb.at(uint32_t(kKT + nc * C::UK + kh), uint32_t(S));
                            const uint32_t st = rq.st;
                            const long long r0 = DLR_CLK();
                            if (!w.cta(smem_u32(&bars->ring_full[st]), rq.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                            m[5] += DLR_CLK() - r0;
                            tc_fence_after();
                            const uint64_t bdesc = umma_desc(ring_s + st * kStageBytes, C::U_LAYOUT, C::U_SBO);
#pragma unroll
                            for (int k = 0; k < C::KW / 16; ++k) {
                                // K step ks of the s tile: two 16-byte chunks, 128 bytes apart
                                const int ks = kh * (C::KW / 16) + k;
                                const uint64_t adesc = umma_desc_nosw(sbuf_s + uint32_t(ks) * 256u, 128u, C::S_GROUP_BYTES);
                                umma_ss(acc, adesc, bdesc + uint64_t(2 * k), idesc_u, (kh | k) ? 1u : 0u);
                            }
                            umma_commit(smem_u32(&bars->ring_empty[st]));
                        }
                        if (err) break;
                        umma_commit(smem_u32(&bars->dh_full[b]));
                    }
                    m[3] += DLR_CLK() - t1;
                }
            }
            if (p.prof) {
                m[7] = DLR_CLK() - mstart;
                for (int k = 0; k < 8; ++k) p.prof[(blockIdx.x * 4 + 1 + b) * 16 + k] = (unsigned long long)m[k];
            }
        }
    } else if (warp >= 4) {
        // =============================== epilogue warps =============================
        // Two threads per row: thread (row er, half hh) owns the columns of half hh of
        // z, of every dh chunk and of the activation stripe.
        const int et = threadIdx.x - 128;            // 0..255
        const int hh = (warp - 4) >> 2;              // column half
        const int q = warp & 3;                      // tensor-memory lane quadrant of this warp
        const int er = 32 * q + lane;                // row of the tile
        const uint32_t tl = tmem_base + (uint32_t(32 * q) << 16);
        const int owner = er / rows_own;
        const int lr = er % rows_own;
        constexpr int groups_own = rows_own / 8;     // 8-row groups per owner
        constexpr uint32_t src_bytes = uint32_t(groups_own) * C::R_GROUP_BYTES;   // one source's block in recv
        constexpr int items = rows_own * C::NCK / kEpi;   // 16-byte chunks of s per thread in the reduce
        constexpr int NZ = R / 2;                    // columns of z per thread
        uint32_t c_z = 0, c_recv = 0, c_dh[2] = {0, 0};
        long long e[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const long long estart = DLR_CLK();

        for (int tile = cluster_id; tile < p.num_tiles && !err; tile += num_clusters) {
            const int grow = tile * kRows + er;
            const bool valid = grow < p.M;
            const long long x0 = DLR_CLK();
            const __nv_bfloat16* xrow = p.x + size_t(valid ? grow : 0) * p.d + stripe0 + 256 * hh;
            float ssq = 0.f;
            // ---- input half-stripe -> tensor memory (packed bf16), partial sum of squares
#pragma unroll 4
            for (int c = 0; c < 16; ++c) {
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
                tmem_st8(tl + kHOff + uint32_t(128 * hh + 8 * c), v);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(&bars->h_ready));
            e[6] += DLR_CLK() - x0;

            for (int l = 0; l < p.L && !err; ++l) {
                err_layer = l;
                long long t0 = DLR_CLK();
                // ---- partial z of this row (both K halves added) -> bf16 -> the row's owner
                bool ok = w.cta(smem_u32(&bars->z_full[0]), c_z & 1u);
                ok = ok && w.cta(smem_u32(&bars->z_full[1]), c_z & 1u);
                if (!__all_sync(0xffffffffu, ok)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                ++c_z;
                tc_fence_after();
                long long t1 = DLR_CLK();
                e[0] += t1 - t0;
                if (et == 0) mbar_arrive_expect_tx(smem_u32(&bars->recv_full), C::RECV_BYTES);   // arm this layer's receive
                {
                    // this row's slot in its owner's receive buffer
                    const uint32_t dst = mapa(recv_s + uint32_t(rank) * src_bytes + uint32_t(lr >> 3) * C::R_GROUP_BYTES +
                                                  uint32_t(lr & 7) * 16u, uint32_t(owner));
                    const uint32_t rbar = mapa(smem_u32(&bars->recv_full), uint32_t(owner));
#pragma unroll
                    for (int c = 0; c < NZ / 16; ++c) {
                        uint32_t v0[16], v1[16];
                        tmem_ld16(tl + kAcc0 + uint32_t(NZ * hh + 16 * c), v0);
                        tmem_ld16(tl + kAcc0 + 128u + uint32_t(NZ * hh + 16 * c), v1);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            uint32_t pk[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                pk[i] = pack_bf16x2(__uint_as_float(v0[8 * j + 2 * i]) + __uint_as_float(v1[8 * j + 2 * i]),
                                                    __uint_as_float(v0[8 * j + 2 * i + 1]) + __uint_as_float(v1[8 * j + 2 * i + 1]));
                            const int chunk = (NZ * hh + 16 * c + 8 * j) / 8;
                            st_async_v4(dst + uint32_t(chunk) * 128u, pk[0], pk[1], pk[2], pk[3], rbar);
                        }
                    }
                    st_async_v4(dst + uint32_t(C::NCK + hh) * 128u, __float_as_uint(ssq), 0u, 0u, 0u, rbar);
                }
                tc_fence_before();
                mbar_arrive(smem_u32(&bars->acc_empty[0]));   // z has left both accumulators
                mbar_arrive(smem_u32(&bars->acc_empty[1]));
                t0 = DLR_CLK();
                e[1] += t0 - t1;

                // ---- owner: sum the CS partials of its rows, normalise, SiLU, all-gather
                if (!__all_sync(0xffffffffu, w.cluster(smem_u32(&bars->recv_full), c_recv & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                ++c_recv;
                t1 = DLR_CLK();
                e[2] += t1 - t0;
                if (et == 0) mbar_arrive_expect_tx(smem_u32(&bars->s_full), C::S_BYTES);      // arm this layer's s tile
#pragma unroll
                for (int it = 0; it < items; ++it) {
                    const int i = et + kEpi * it;
                    const int r8 = i & 7;
                    const int c = (i >> 3) % C::NCK;
                    const int gl = i / R;                 // 8-row group inside this owner's rows
                    const uint8_t* base = recv + size_t(gl) * C::R_GROUP_BYTES + r8 * 16;
                    float tot = 0.f;
                    float a[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) a[j] = 0.f;
#pragma unroll
                    for (int src = 0; src < CS; ++src) {
                        const uint8_t* bp = base + size_t(src) * src_bytes;
                        const uint4 u = *reinterpret_cast<const uint4*>(bp + c * 128);
                        tot += *reinterpret_cast<const float*>(bp + C::NCK * 128) +
                               *reinterpret_cast<const float*>(bp + (C::NCK + 1) * 128);
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
                                    mapa(smem_u32(&bars->s_full), uint32_t(dc)));
                }
                t0 = DLR_CLK();
                e[3] += t0 - t1;

                // ---- fused epilogue of the U contraction: h += dh, new sum of squares
                float ssq_new = 0.f;
                for (int nc = 0; nc < kNCH && !err; ++nc) {
                    const int b = nc & 1;
                    const long long d0 = DLR_CLK();
                    if (!__all_sync(0xffffffffu, w.cta(smem_u32(&bars->dh_full[b]), c_dh[b] & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_dh[b];
                    tc_fence_after();
                    e[4] += DLR_CLK() - d0;
                    const uint32_t acc = tl + kAcc0 + uint32_t(b) * 128u + uint32_t(64 * hh);
                    const uint32_t hcol = tl + kHOff + uint32_t(64 * nc + 32 * hh);
                    {
                        // both 32-column halves are fetched before either is processed: one
                        // tensor-memory round trip per chunk instead of two
                        uint32_t dh0[32], dh1[32], hp0[16], hp1[16];
                        tmem_ld32(acc, dh0);
                        tmem_ld16(hcol, hp0);
                        tmem_ld32(acc + 32u, dh1);
                        tmem_ld16(hcol + 16u, hp1);
                        tmem_wait_ld();
                        if (nc + 2 < kNCH) {
                            // the dh values are in registers: the accumulator can take the next chunk
                            tc_fence_before();
                            mbar_arrive(smem_u32(&bars->acc_empty[b]));
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float lo = bf16lo_to_f(hp0[j]) + __uint_as_float(dh0[2 * j]);
                            const float hi = bf16hi_to_f(hp0[j]) + __uint_as_float(dh0[2 * j + 1]);
                            ssq_new += lo * lo + hi * hi;
                            hp0[j] = pack_bf16x2(lo, hi);
                        }
                        tmem_st16(hcol, hp0);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float lo = bf16lo_to_f(hp1[j]) + __uint_as_float(dh1[2 * j]);
                            const float hi = bf16hi_to_f(hp1[j]) + __uint_as_float(dh1[2 * j + 1]);
                            ssq_new += lo * lo + hi * hi;
                            hp1[j] = pack_bf16x2(lo, hi);
                        }
                        tmem_st16(hcol + 16u, hp1);
                    }
                }
                if (err) break;
                ssq = ssq_new;
                tmem_wait_st();
                if (l + 1 < p.L) {
                    tc_fence_before();
                    mbar_arrive(smem_u32(&bars->h_ready));
                }
                e[5] += DLR_CLK() - t0;
            }
            if (err) break;
            // ---- final activation half-stripe -> global
            __nv_bfloat16* yrow = p.y + size_t(valid ? grow : 0) * p.d + stripe0 + 256 * hh;
#pragma unroll 4
            for (int c = 0; c < 16; ++c) {
                uint32_t v[8];
                tmem_ld8(tl + kHOff + uint32_t(128 * hh + 8 * c), v);
                tmem_wait_ld();
                if (valid) {
                    *reinterpret_cast<uint4*>(yrow + 16 * c) = make_uint4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<uint4*>(yrow + 16 * c + 8) = make_uint4(v[4], v[5], v[6], v[7]);
                }
            }
        }
        if (p.prof && et == 0) {
            e[7] = DLR_CLK() - estart;
            for (int k = 0; k < 8; ++k) p.prof[(blockIdx.x * 4 + 3) * 16 + k] = (unsigned long long)e[k];
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
    if (d != CS * kStripe) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    int stages = (smem_optin - C::FIXED_BYTES) / kStageBytes;
    if (stages > kMaxStages) stages = kMaxStages;
    // the two MMA warps read the two halves of a layer's V tiles at the same time
    if (stages < kKT + 1) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    const int smem = stages * kStageBytes + C::FIXED_BYTES;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return DLRB200_ERR_CUDA;

    const int num_tiles = (M + kRows - 1) / kRows;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(CS * (num_sms / CS));
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) return DLRB200_ERR_CUDA;
    if (max_clusters < 1) return DLRB200_ERR_OCCUPANCY;
    const int clusters = num_tiles < max_clusters ? num_tiles : max_clusters;
    cfg.gridDim = dim3(CS * clusters);
    if (plan_only) {
        plan_only->path = DLRB200_PATH_CLUSTER;
        plan_only->grid = CS * clusters;
        plan_only->cluster = CS;
        plan_only->stripe_cols = kStripe;
        plan_only->rows_per_pass = kRows;
        plan_only->passes = (num_tiles + clusters - 1) / clusters;   // waves of row tiles
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
    p.num_tiles = num_tiles;
    p.prof = prof;
    CUtensorMap tmV, tmU;
    memset(&tmV, 0, sizeof(tmV));
    memset(&tmU, 0, sizeof(tmU));
    if ((!encode_2d_bf16(enc, &tmV, Vp, uint64_t(d), uint64_t(L) * R, 64, R, 128) ||
        !encode_2d_bf16(enc, &tmU, Up, uint64_t(R), uint64_t(L) * d, C::KW, 128, C::KW * 2)))
        return DLRB200_ERR_CUDA;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, tmV, tmU, p);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

// (r, cluster size) pairs that are built; the reduce needs r >= 16 * CS so that
// every epilogue thread owns at least one 16-byte chunk of s.
bool combo_ok(int r, int cs) {
    if (!(cs == 1 || cs == 2 || cs == 4 || cs == 8)) return false;
    if (!(r == 32 || r == 64 || r == 128)) return false;
    return r >= 16 * cs;
}

int dispatch(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L, float eps,
             int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
             dlrb200_plan* plan_only, unsigned long long* prof) {
#define DLR_CASE(RR, CC)                                                                                          \
    if (r == RR && d == CC * kStripe)                                                                             \
        return launch_cluster<RR, CC>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin,   \
                                      spin_limit, plan_only, prof);
    DLR_CASE(32, 1)
    DLR_CASE(32, 2)
    DLR_CASE(64, 1)
    DLR_CASE(64, 2)
    DLR_CASE(64, 4)
    DLR_CASE(128, 1)
    DLR_CASE(128, 2)
    DLR_CASE(128, 4)
    DLR_CASE(128, 8)
#undef DLR_CASE
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

// Debug aid: with DLRB200_PROFILE=1 in the environment every CTA writes cycle
// counts of its phases (4 roles x 16 counters) at offset 256 of the workspace.
constexpr size_t kProfBytes = 256 + size_t(256) * 4 * 16 * 8;

bool profiling() {
    const char* v = std::getenv("DLRB200_PROFILE");
    return v && *v && *v != '0';
}

}  // namespace

bool cluster_supported(int d, int r, int L) {
    (void)L;
    if (d % kStripe != 0) return false;
    return combo_ok(r, d / kStripe);
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
