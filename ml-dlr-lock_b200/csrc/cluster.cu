// Large-batch ("prefill") DLR-Net forward on thread-block clusters with tcgen05
// tensor cores and tensor memory.
//
// Work split.  A cluster of CS = d/512 CTAs owns one tile of 128 token rows for
// all L layers; CTA `rank` owns columns [512*rank, 512*rank+512) of the model
// width for BOTH contractions of a layer (K-stripe of the V contraction,
// N-stripe of the U contraction - the reference's cooperative scheme,
// kernels/kernels/cuda/cooperative.cu:10-16, moved from global memory to
// distributed shared memory).  Per layer (dlr_lock/model.py:96-100 on folded
// weights, kernels/README.md:5-7):
//
//   V:  z_part[128 x r]  = h[128 x 512] . V'[:, stripe]^T     tcgen05.mma, A from TMEM
//   X:  z = sum over the cluster of z_part, sumsq likewise    DSMEM reduce-scatter by rows
//       s = silu(z * rsqrt(sumsq/d + eps)) as bf16            DSMEM all-gather
//   U:  dh[128 x 512]    = s[128 x r] . U'[stripe, :]^T       tcgen05.mma, A and B from smem
//       h += dh ; sumsq_part = sum h^2                        fused epilogue out of TMEM
//
// On-chip residency.  The activation stripe (128 x 512) lives in tensor memory
// for the whole stack as packed bf16 (256 of the 512 columns) and is the A
// operand of the V contraction directly; the other 256 columns hold two fp32
// accumulators of 128 columns (z, then the dh chunks, double-buffered).  The
// activation is therefore re-rounded to bf16 once per layer, like every fused
// kernel of the reference (fp32 accumulation inside a layer).
//
// Roles.  Warp 0 streams weight tiles with TMA into a ring of 16 KB stages
// (it never waits for the activations, so it runs ahead across layers and
// tiles); one lane of warp 1 issues all MMAs; warps 2-5 (one thread per row)
// move accumulators, run the exchange and the epilogue.  All waits are bounded
// mbarrier waits; a wait that gives up records a status word and every role
// drains to a common exit.
#include <cstring>

#include "cluster.h"
#include "ptx.cuh"

namespace dlr {

namespace {

constexpr int kRows = 128;
constexpr int kKT = 8;               // 64-column K tiles per stripe
constexpr int kStripe = 64 * kKT;    // 512 columns per CTA
constexpr int kNCH = kKT / 2;        // 128-column output chunks per stripe
constexpr int kStageBytes = 16384;
constexpr int kMaxStages = 8;
constexpr int kThreads = 192;
constexpr uint32_t kH0 = 0;          // packed bf16 activation: 256 columns
constexpr uint32_t kAcc0 = 256;      // fp32 accumulator 0 (z, even dh chunks)
constexpr uint32_t kAcc1 = 384;      // fp32 accumulator 1 (odd dh chunks)

struct ClusterParams {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int M, d, L;
    float eps, inv_d;
    int* status;
    unsigned int spin_limit;
    int stages;
    int num_tiles;
    int cs;
};

template <int R>
struct CCfg {
    static constexpr int KW = R < 64 ? R : 64;     // K columns per s / U tile
    static constexpr int UK = R / KW;              // K tiles of the U contraction
    static constexpr int S_TILE_BYTES = kRows * KW * 2;
    static constexpr int S_BYTES = kRows * R * 2;
    static constexpr int RECV_BYTES = kRows * R * 4;
    static constexpr int SSQ_BYTES = kRows * 4;
    static constexpr int V_CHUNK_BYTES = R * 128;
    static constexpr int U_CHUNK_BYTES = 128 * KW * 2;
    static constexpr int SWZ_BITS = KW == 64 ? 3 : 2;
    static constexpr uint32_t U_LAYOUT = KW == 64 ? 2u : 4u;   // descriptor layout type
    static constexpr uint32_t U_SBO = 8 * KW * 2;              // bytes between 8-row groups
    static constexpr int FIXED_BYTES = S_BYTES + RECV_BYTES + SSQ_BYTES + 512 /*barriers*/ + 1024 /*alignment*/;
};

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

__device__ __forceinline__ void st_cluster_v2(uint32_t addr_cluster, uint32_t a, uint32_t b) {
    asm volatile("st.shared::cluster.v2.b32 [%0], {%1,%2};" ::"r"(addr_cluster), "r"(a), "r"(b) : "memory");
}

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

template <int R>
__global__ void __launch_bounds__(kThreads, 1)
dlr_cluster_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU,
                   ClusterParams p) {
    using C = CCfg<R>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int S = p.stages;
    uint8_t* ring = smem;
    uint8_t* sbuf = ring + size_t(S) * kStageBytes;
    float* recv = reinterpret_cast<float*>(sbuf + C::S_BYTES);
    float* ssqbuf = recv + kRows * R;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ssqbuf + kRows);
    uint64_t* ring_full = bars;                 // [kMaxStages]
    uint64_t* ring_empty = bars + kMaxStages;   // [kMaxStages]
    uint64_t* z_full = bars + 2 * kMaxStages;
    uint64_t* recv_full = z_full + 1;
    uint64_t* s_full = z_full + 2;
    uint64_t* dh_full = z_full + 3;             // [2]
    uint64_t* acc_empty = z_full + 5;           // [2]
    uint64_t* h_ready = z_full + 7;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(z_full + 8);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int CS = p.cs;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x / CS;
    const int num_clusters = gridDim.x / CS;
    const int rows_own = kRows / CS;
    const int stripe0 = int(rank) * kStripe;
    const Waiter w{abort_flag, p.spin_limit >> 2};

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(smem_u32(&ring_full[s]), 1);
            mbar_init(smem_u32(&ring_empty[s]), 1);
        }
        mbar_init(smem_u32(z_full), 1);
        mbar_init(smem_u32(recv_full), CS * (rows_own >= 32 ? rows_own / 32 : 1));
        mbar_init(smem_u32(s_full), CS * 4);
        mbar_init(smem_u32(&dh_full[0]), 1);
        mbar_init(smem_u32(&dh_full[1]), 1);
        mbar_init(smem_u32(&acc_empty[0]), 128);
        mbar_init(smem_u32(&acc_empty[1]), 128);
        mbar_init(smem_u32(h_ready), 128);
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

    int err = 0;
    int err_layer = 0;

    if (warp == 0) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            uint32_t n = 0;
            for (int tile = cluster_id; tile < p.num_tiles && !err; tile += num_clusters) {
                for (int l = 0; l < p.L && !err; ++l) {
                    for (int i = 0; i < kKT + kNCH * C::UK; ++i, ++n) {
                        const uint32_t st = n % uint32_t(S);
                        const uint32_t ph = (n / uint32_t(S)) & 1u;
                        if (!w.cta(smem_u32(&ring_empty[st]), ph ^ 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; err_layer = l; break; }
                        const uint32_t bar = smem_u32(&ring_full[st]);
                        const uint32_t dst = ring_s + st * kStageBytes;
                        if (i < kKT) {
                            mbar_arrive_expect_tx(bar, C::V_CHUNK_BYTES);
                            tma_load_2d(dst, &tmV, stripe0 + 64 * i, l * R, bar);
                        } else {
                            const int j = i - kKT;
                            const int nc = j / C::UK, kh = j % C::UK;
                            mbar_arrive_expect_tx(bar, C::U_CHUNK_BYTES);
                            tma_load_2d(dst, &tmU, kh * C::KW, l * p.d + stripe0 + 128 * nc, bar);
                        }
                    }
                }
            }
            if (err) {
                // the copies issued before giving up still land in this CTA's
                // ring: wait (bounded) until the consumers have drained them or
                // they have at least completed.
                for (uint32_t back = 1; back <= uint32_t(S) && back <= n; ++back) {
                    const uint32_t m = n - back;
                    mbar_wait(smem_u32(&ring_full[m % uint32_t(S)]), (m / uint32_t(S)) & 1u, p.spin_limit >> 6);
                }
            }
        }
    } else if (warp == 1) {
        // =============================== MMA issuer =================================
        if (lane == 0) {
            const uint32_t idesc_v = umma_idesc_bf16(128, R);
            const uint32_t idesc_u = umma_idesc_bf16(128, 128);
            uint32_t n = 0, c_h = 0, c_s = 0, c_e0 = 0, c_e1 = 0;
            for (int tile = cluster_id; tile < p.num_tiles && !err; tile += num_clusters) {
                for (int l = 0; l < p.L && !err; ++l) {
                    err_layer = l;
                    if (!w.cta(smem_u32(h_ready), c_h & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_h;
                    tc_fence_after();
                    // ---- V contraction: acc0 = h . V'^T over the 8 K tiles of the stripe
                    for (int kt = 0; kt < kKT && !err; ++kt, ++n) {
                        const uint32_t st = n % uint32_t(S);
                        if (!w.cta(smem_u32(&ring_full[st]), (n / uint32_t(S)) & 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                        tc_fence_after();
                        const uint64_t bdesc = umma_desc_sw128(ring_s + st * kStageBytes);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_ts(tmem_base + kAcc0, tmem_base + kH0 + uint32_t(kt * 32 + k * 8), bdesc + uint64_t(2 * k),
                                    idesc_v, (kt | k) ? 1u : 0u);
                        umma_commit(smem_u32(&ring_empty[st]));
                    }
                    if (err) break;
                    umma_commit(smem_u32(z_full));
                    // ---- U contraction: four 128-column chunks, accumulators alternate
                    if (!w.cluster(smem_u32(s_full), c_s & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_s;
                    tc_fence_after();
                    for (int nc = 0; nc < kNCH && !err; ++nc) {
                        const int b = nc & 1;
                        if (nc != 1) {
                            uint32_t& c_e = b ? c_e1 : c_e0;
                            if (!w.cta(smem_u32(&acc_empty[b]), c_e & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                            ++c_e;
                            tc_fence_after();
                        }
                        const uint32_t acc = tmem_base + (b ? kAcc1 : kAcc0);
                        for (int kh = 0; kh < C::UK && !err; ++kh, ++n) {
                            const uint32_t st = n % uint32_t(S);
                            if (!w.cta(smem_u32(&ring_full[st]), (n / uint32_t(S)) & 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                            tc_fence_after();
                            const uint64_t adesc = umma_desc(sbuf_s + kh * C::S_TILE_BYTES, C::U_LAYOUT, C::U_SBO);
                            const uint64_t bdesc = umma_desc(ring_s + st * kStageBytes, C::U_LAYOUT, C::U_SBO);
#pragma unroll
                            for (int k = 0; k < C::KW / 16; ++k)
                                umma_ss(acc, adesc + uint64_t(2 * k), bdesc + uint64_t(2 * k), idesc_u, (kh | k) ? 1u : 0u);
                            umma_commit(smem_u32(&ring_empty[st]));
                        }
                        if (err) break;
                        umma_commit(smem_u32(&dh_full[b]));
                    }
                }
            }
        }
    } else {
        // =============================== epilogue warps =============================
        const int et = threadIdx.x - 64;             // 0..127
        const int q = warp & 3;                      // tensor-memory lane quadrant of this warp
        const int er = 32 * q + lane;                // row of the tile this thread owns
        const uint32_t tl = tmem_base + (uint32_t(32 * q) << 16);
        const uint32_t recv_s = smem_u32(recv);
        const uint32_t ssq_s = smem_u32(ssqbuf);
        const int owner = er / rows_own;
        const int lr = er % rows_own;
        const int o_first = (32 * q) / rows_own;
        const int o_last = (32 * q + 31) / rows_own;
        const int cpt = R / CS;                      // columns of s per thread in the reduce
        const int lr2 = et / CS;
        const int cseg = et % CS;
        uint32_t c_z = 0, c_recv = 0, c_dh0 = 0, c_dh1 = 0;

        for (int tile = cluster_id; tile < p.num_tiles && !err; tile += num_clusters) {
            const int grow = tile * kRows + er;
            const bool valid = grow < p.M;
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
                tmem_st8(tl + kH0 + uint32_t(8 * c), v);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(smem_u32(h_ready));

            for (int l = 0; l < p.L && !err; ++l) {
                err_layer = l;
                // ---- partial z of this row -> owner CTA (reduce-scatter by rows)
                if (!__all_sync(0xffffffffu, w.cta(smem_u32(z_full), c_z & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                ++c_z;
                tc_fence_after();
                {
                    const uint32_t dst = mapa(recv_s + uint32_t((int(rank) * rows_own + lr) * R) * 4u, uint32_t(owner));
#pragma unroll
                    for (int c = 0; c < R / 16; ++c) {
                        uint32_t v[16];
                        tmem_ld16(tl + kAcc0 + uint32_t(16 * c), v);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            st_cluster_v4(dst + uint32_t(c * 64 + j * 16), v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    }
                    st_cluster_f32(mapa(ssq_s + uint32_t(int(rank) * rows_own + lr) * 4u, uint32_t(owner)), ssq);
                }
                tc_fence_before();
                mbar_arrive(smem_u32(&acc_empty[0]));   // z has left accumulator 0
                __syncwarp();
                if (lane == 0)
                    for (int o = o_first; o <= o_last; ++o) mbar_arrive_remote(mapa(smem_u32(recv_full), uint32_t(o)));

                // ---- owner: sum the CS partials of its rows, normalise, SiLU, all-gather
                if (!__all_sync(0xffffffffu, w.cluster(smem_u32(recv_full), c_recv & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                ++c_recv;
                {
                    float tot = 0.f;
                    for (int src = 0; src < CS; ++src) tot += ssqbuf[src * rows_own + lr2];
                    const float rstd = rsqrtf(tot * p.inv_d + p.eps);
                    const int srow = int(rank) * rows_own + lr2;      // row inside the 128-row tile
                    for (int c0 = 0; c0 < cpt; c0 += 8) {
                        const int col = cseg * cpt + c0;
                        const int nval = cpt - c0 < 8 ? cpt - c0 : 8;   // 8, or 4 when cpt == 4
                        float a[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) a[j] = 0.f;
                        for (int src = 0; src < CS; ++src) {
                            const float* rp = recv + (src * rows_own + lr2) * R + col;
                            const float4 u0 = *reinterpret_cast<const float4*>(rp);
                            a[0] += u0.x; a[1] += u0.y; a[2] += u0.z; a[3] += u0.w;
                            if (nval == 8) {
                                const float4 u1 = *reinterpret_cast<const float4*>(rp + 4);
                                a[4] += u1.x; a[5] += u1.y; a[6] += u1.z; a[7] += u1.w;
                            }
                        }
                        uint32_t pk[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) pk[j] = pack_bf16x2(silu_f(a[2 * j] * rstd), silu_f(a[2 * j + 1] * rstd));
                        const int kh = col / C::KW;
                        const uint32_t off = uint32_t(kh) * C::S_TILE_BYTES +
                                             swz(uint32_t(srow) * (C::KW * 2) + uint32_t(col % C::KW) * 2u, C::SWZ_BITS);
                        for (int dstc = 0; dstc < CS; ++dstc) {
                            const uint32_t da = mapa(sbuf_s + off, uint32_t(dstc));
                            if (nval == 8) st_cluster_v4(da, pk[0], pk[1], pk[2], pk[3]);
                            else st_cluster_v2(da, pk[0], pk[1]);
                        }
                    }
                }
                fence_proxy_async_all();
                __syncwarp();
                if (lane == 0)
                    for (int dstc = 0; dstc < CS; ++dstc) mbar_arrive_remote(mapa(smem_u32(s_full), uint32_t(dstc)));

                // ---- fused epilogue of the U contraction: h += dh, new sum of squares
                float ssq_new = 0.f;
                for (int nc = 0; nc < kNCH && !err; ++nc) {
                    const int b = nc & 1;
                    uint32_t& c_dh = b ? c_dh1 : c_dh0;
                    if (!__all_sync(0xffffffffu, w.cta(smem_u32(&dh_full[b]), c_dh & 1u))) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_dh;
                    tc_fence_after();
                    const uint32_t acc = tl + (b ? kAcc1 : kAcc0);
#pragma unroll 2
                    for (int c = 0; c < 8; ++c) {
                        uint32_t dh[16], hp[8];
                        tmem_ld16(acc + uint32_t(16 * c), dh);
                        tmem_ld8(tl + kH0 + uint32_t(64 * nc + 8 * c), hp);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float lo = bf16lo_to_f(hp[j]) + __uint_as_float(dh[2 * j]);
                            const float hi = bf16hi_to_f(hp[j]) + __uint_as_float(dh[2 * j + 1]);
                            const uint32_t pk = pack_bf16x2(lo, hi);
                            const float rl = bf16lo_to_f(pk), rh = bf16hi_to_f(pk);
                            ssq_new += rl * rl + rh * rh;
                            hp[j] = pk;
                        }
                        tmem_st8(tl + kH0 + uint32_t(64 * nc + 8 * c), hp);
                    }
                    if (nc + 2 < kNCH) {
                        tc_fence_before();
                        mbar_arrive(smem_u32(&acc_empty[b]));
                    }
                }
                if (err) break;
                ssq = ssq_new;
                tmem_wait_st();
                if (l + 1 < p.L) {
                    tc_fence_before();
                    mbar_arrive(smem_u32(h_ready));
                }
            }
            if (err) break;
            // ---- final activation stripe -> global
            __nv_bfloat16* yrow = p.y + size_t(valid ? grow : 0) * p.d + stripe0;
#pragma unroll 4
            for (int c = 0; c < kStripe / 16; ++c) {
                uint32_t v[8];
                tmem_ld8(tl + kH0 + uint32_t(8 * c), v);
                tmem_wait_ld();
                if (valid) {
                    *reinterpret_cast<uint4*>(yrow + 16 * c) = make_uint4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<uint4*>(yrow + 16 * c + 8) = make_uint4(v[4], v[5], v[6], v[7]);
                }
            }
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

template <int R>
int launch_cluster(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int L, float eps,
                   int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
                   dlrb200_plan* plan_only) {
    using C = CCfg<R>;
    auto kern = dlr_cluster_kernel<R>;
    const int cs = d / kStripe;
    int stages = (smem_optin - C::FIXED_BYTES) / kStageBytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 3) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    const int smem = stages * kStageBytes + C::FIXED_BYTES;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return DLRB200_ERR_CUDA;

    const int num_tiles = (M + kRows - 1) / kRows;
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
    const int clusters = num_tiles < max_clusters ? num_tiles : max_clusters;
    cfg.gridDim = dim3(cs * clusters);
    if (plan_only) {
        plan_only->path = DLRB200_PATH_CLUSTER;
        plan_only->grid = cs * clusters;
        plan_only->cluster = cs;
        plan_only->stripe_cols = kStripe;
        plan_only->rows_per_pass = kRows;
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
    p.num_tiles = num_tiles;
    p.cs = cs;
    CUtensorMap tmV, tmU;
    if (!encode_2d_bf16(enc, &tmV, Vp, uint64_t(d), uint64_t(L) * R, 64, R, 128) ||
        !encode_2d_bf16(enc, &tmU, Up, uint64_t(R), uint64_t(L) * d, C::KW, 128, C::KW * 2))
        return DLRB200_ERR_CUDA;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, tmV, tmU, p);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

int dispatch(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L, float eps,
             int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
             dlrb200_plan* plan_only) {
    switch (r) {
        case 32: return launch_cluster<32>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only);
        case 64: return launch_cluster<64>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only);
        case 128: return launch_cluster<128>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace

bool cluster_supported(int d, int r, int L) {
    (void)L;
    return d % kStripe == 0 && d / kStripe >= 1 && d / kStripe <= 8 && (r == 32 || r == 64 || r == 128) &&
           (r / (d / kStripe)) >= 4;
}

size_t cluster_workspace_bytes(int, int, int, int) { return 0; }

int cluster_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan) {
    const size_t ws = plan->workspace_bytes;
    const int rc = dispatch(nullptr, nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, num_sms,
                            smem_optin, 0, plan);
    plan->workspace_bytes = ws;
    return rc;
}

int cluster_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                    int L, float eps, void* workspace, int* status_dev, cudaStream_t stream, int num_sms,
                    int smem_optin, unsigned int spin_limit) {
    (void)workspace;
    return dispatch(encode_fn_ptr, x, y, Vp, Up, M, d, r, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit,
                    nullptr);
}

}  // namespace dlr
