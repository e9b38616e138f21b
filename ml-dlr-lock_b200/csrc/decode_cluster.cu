// Small-batch ("decode") DLR-Net forward: one thread-block cluster per PAIR of
// token rows, CUDA-core dot products, per-layer exchange in distributed shared
// memory.
//
// Why.  A small batch is one dependency chain of L layers; each layer needs the
// sum over the whole width d of the partial z.  Spreading the width over all
// SMs makes that sum a round trip through global memory per layer (about 3 us
// measured on the striped kernel); inside a cluster it is one hop of
// asynchronous stores into the peers' shared memory (about 260 cycles
// measured).  With one or two rows there is nothing for a tensor core to do:
// the legacy mma.sync path cost about 150 cycles per dependent k-step here.
// So this kernel follows the classic GEMV recipe: 128-bit loads of the weights
// (from the TMA-filled, swizzled ring in shared memory), fp32 FMAs, a
// warp-shuffle reduce-scatter, fp32 everywhere.
//
// Work split.  Rows 2c and 2c+1 of the batch are served by cluster c of
// CS = d/256 CTAs (1..16); CTA `rank` owns columns [256*rank, 256*rank+256) for
// both contractions (K-stripe = N-stripe, as in
// kernels/kernels/cuda/cooperative.cu:10-16).  Thread j keeps column j of the
// stripe of h for both rows in registers for all L layers.  More rows take more
// clusters; they share the weights through L2 and never talk to each other.
//
// Per layer (dlr_lock/model.py:96-100 on folded weights):
//   V   warp w: rows [w*R/8, (w+1)*R/8) of V'; lane = 8 consecutive columns; a
//       butterfly reduce-scatter leaves one (r, row) sum per lane
//   X   the partial z and the partial sums of squares go to ALL CTAs of the cluster
//       (st.async, bytes counted on the receiver's mbarrier, receive buffer
//       double-buffered by layer parity); every CTA adds up the CS partials
//   s   = silu(z * rsqrt(sumsq/d + eps)), fp32
//   U   thread j: dot of row j of the U' slice with s for both rows; h += dh
//
// All waits are bounded; a wait that gives up records a status word, and the
// CTA barriers are still reached by every thread so that nothing hangs.
#include <cstring>

#include "cluster.h"
#include "decode_cluster.h"
#include "ptx.cuh"

namespace dlr {

namespace {

constexpr int kStage = 16384;
constexpr int kMaxStages = 12;
constexpr int kCompute = 256;          // 8 compute warps; warp 8 is the TMA producer
constexpr int kThreadsDC = 288;
constexpr int kMaxCS = 16;
constexpr int kSC = 256;               // columns per CTA
constexpr int kNR = 2;                 // rows per cluster
constexpr int kVT = kSC / 64;          // V tiles per layer: R rows x 64 columns

struct DCParams {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int M, d, L;
    float eps, inv_d;
    int* status;
    unsigned int spin_limit;
    int stages;
    int cs;
    unsigned long long* prof;   // optional phase cycle counters of CTA 0 (debug), or null
};

template <int R>
struct DCfg {
    static constexpr int KW = R < 64 ? R : 64;          // K columns per U tile
    static constexpr int UK = R / KW;
    static constexpr int UT = (kSC / 128) * UK;         // U tiles per layer: 128 rows x KW columns
    static constexpr int V_TILE_BYTES = R * 128;
    static constexpr int U_TILE_BYTES = 128 * KW * 2;
    static constexpr int UBITS = KW == 64 ? 3 : 2;
    static constexpr int ZF = R * kNR;                  // floats of partial z per CTA
    static constexpr int SRC_FLOATS = ZF + 4;           // + partial sums of squares (2, padded to 4)
    static constexpr int RW = R / 8;                    // V' rows per warp
    static constexpr int NV = RW * kNR;                 // partial sums per lane before the reduce-scatter
    static constexpr int FIXED_BYTES = 2 * kMaxCS * SRC_FLOATS * 4 /*recv*/ + ZF * 4 /*zp*/ + ZF * 4 /*s*/ +
                                       kNR * kSC * 4 /*h copy*/ + 1024 /*barriers, partial sums*/ + 1024 /*alignment*/;
};

struct DCBars {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t recv[2];
};

__device__ __forceinline__ void st_async_v4f(uint32_t dst_cluster, float a, float b, float c, float d, uint32_t bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1,%2,%3,%4}, [%5];" ::"r"(
                     dst_cluster),
                 "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)), "r"(__float_as_uint(d)),
                 "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void st_async_v2f(uint32_t dst_cluster, float a, float b, uint32_t bar) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1,%2}, [%3];" ::"r"(dst_cluster),
                 "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__device__ __forceinline__ void fma8(float (&acc), const uint4& w, const float4& h0, const float4& h1) {
    acc = fmaf(bf16lo_to_f(w.x), h0.x, acc);
    acc = fmaf(bf16hi_to_f(w.x), h0.y, acc);
    acc = fmaf(bf16lo_to_f(w.y), h0.z, acc);
    acc = fmaf(bf16hi_to_f(w.y), h0.w, acc);
    acc = fmaf(bf16lo_to_f(w.z), h1.x, acc);
    acc = fmaf(bf16hi_to_f(w.z), h1.y, acc);
    acc = fmaf(bf16lo_to_f(w.w), h1.z, acc);
    acc = fmaf(bf16hi_to_f(w.w), h1.w, acc);
}

// Butterfly reduce-scatter over the 32 lanes of a warp: every lane enters with NV
// partial sums (same meaning in every lane) and leaves with the complete sum of
// entry (lane >> log2(32/NV)) in v[0].
template <int NV>
__device__ __forceinline__ void warp_reduce_scatter(float (&v)[NV], int lane) {
    int cnt = NV;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) {
        if (cnt > 1) {
            const int half = cnt / 2;
            const bool up = (lane & s) != 0;
#pragma unroll
            for (int j = 0; j < NV / 2; ++j) {
                if (j < half) {
                    const float send = up ? v[j] : v[j + half];
                    const float keep = up ? v[j + half] : v[j];
                    v[j] = keep + __shfl_xor_sync(0xffffffffu, send, s);
                }
            }
            cnt = half;
        } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], s);
        }
    }
}

template <int R>
__global__ void __launch_bounds__(kThreadsDC, 1)
dlr_decode_cluster_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU,
                          DCParams p) {
    using C = DCfg<R>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int S = p.stages;
    const int CS = p.cs;
    uint8_t* ring = smem;
    float* recv = reinterpret_cast<float*>(ring + size_t(S) * kStage);   // [2][kMaxCS][SRC_FLOATS]
    float* zp = recv + 2 * kMaxCS * C::SRC_FLOATS;                       // [R][2] this CTA's partial z
    float* ssm = zp + C::ZF;                                             // [R][2] silu(z * rstd)
    float* hs = ssm + C::ZF;                                             // [2][256] copy of h for the V phase
    float* wsum = hs + kNR * kSC;                                        // [8 warps][2] partial sums of squares
    DCBars* bars = reinterpret_cast<DCBars*>(wsum + 16);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster_id = blockIdx.x / CS;
    const int stripe0 = int(rank) * kSC;
    const int row0 = cluster_id * kNR;
    const int rows = (p.M - row0) < kNR ? (p.M - row0) : kNR;
    const uint32_t ring_s = smem_u32(ring);
    const uint32_t recv_s = smem_u32(recv);
    const uint32_t wlimit = p.spin_limit >> 2;

    if (tid == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 8);
        }
        mbar_init(smem_u32(&bars->recv[0]), 1);
        mbar_init(smem_u32(&bars->recv[1]), 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmU);
    }
    __syncthreads();
    cluster_arrive_release();
    cluster_wait_acquire();

    auto wait_cta = [&](uint32_t bar, uint32_t parity) -> bool {
        for (uint32_t i = 0; i < wlimit; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            if ((i & 63u) == 63u && *abort_flag) return false;
        }
        return false;
    };
    int err = 0;
    int l = 0;
    if (warp == 8) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            // The V' tiles of a layer complete one barrier (that of the group's first stage), the U' tiles
            // another: the compute warps wait twice per layer instead of once per tile (a wait on a landed tile
            // still costs each of them about 200 cycles).  A stage's `full` barrier therefore advances only when
            // the stage leads a group; `lead` holds its next parity per stage, and the compute warps keep the same
            // bits.
            RingPos rp;
            uint32_t lead = 0;
            uint32_t last_bar[2] = {0, 0}, last_par[2] = {0, 0};   // the two youngest groups, for the drain below
            bool any[2] = {false, false};
            for (l = 0; l < p.L && !err; ++l) {
                uint32_t bar = 0;
                for (int i = 0; i < kVT + C::UT; ++i, rp.step(uint32_t(S))) {
                    const uint32_t st = rp.st;
                    if (!wait_cta(smem_u32(&bars->empty[st]), rp.ph ^ 1u)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                    const uint32_t dst = ring_s + st * kStage;
                    if (i == 0 || i == kVT) {
                        const int grp = i == 0 ? 0 : 1;
                        bar = smem_u32(&bars->full[st]);
                        mbar_arrive_expect_tx(bar, i == 0 ? kVT * C::V_TILE_BYTES : C::UT * C::U_TILE_BYTES);
                        last_bar[grp] = bar;
                        last_par[grp] = (lead >> st) & 1u;
                        any[grp] = true;
                        lead ^= 1u << st;
                    }
                    if (i < kVT) {
                        tma_load_2d(dst, &tmV, stripe0 + 64 * i, l * R, bar);
                    } else {
                        const int j = i - kVT;
                        tma_load_2d(dst, &tmU, (j % C::UK) * C::KW, l * p.d + stripe0 + 128 * (j / C::UK), bar);
                    }
                }
            }
            if (err) {
                if (!*abort_flag) {
                    *abort_flag = 1;
                    atomicCAS(p.status, 0, err | (l << 8));
                }
                // tiles already requested still land in this CTA's ring: wait (bounded) before leaving.  A group
                // cut short by the error never completes its byte count; older groups have been consumed.
                for (int g = 0; g < 2; ++g)
                    if (any[g]) mbar_wait(last_bar[g], last_par[g], kDrainPolls);
            }
        }
    } else {
        // =============================== compute warps ==============================
        // thread `tid` owns column `tid` of the stripe for both rows
        float h0 = 0.f, h1 = 0.f;
        if (rows > 0) h0 = __bfloat162float(p.x[size_t(row0) * p.d + stripe0 + tid]);
        if (rows > 1) h1 = __bfloat162float(p.x[size_t(row0 + 1) * p.d + stripe0 + tid]);
        auto publish_h = [&]() {
            hs[tid] = h0;
            hs[kSC + tid] = h1;
            float q0 = h0 * h0, q1 = h1 * h1;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                q0 += __shfl_xor_sync(0xffffffffu, q0, o);
                q1 += __shfl_xor_sync(0xffffffffu, q1, o);
            }
            if (lane == 0) { wsum[warp * 2] = q0; wsum[warp * 2 + 1] = q1; }
        };
        publish_h();
        bar_compute();

        const int kcol0 = (lane >> 3) * 64 + (lane & 7) * 8;   // this lane's 8 columns in the V phase
        const int urow = tid & 127;                            // this thread's row inside a U tile
        const int urb = tid >> 7;                              // which 128-row block of the U slice
        RingPos rp;
        uint32_t lead = 0;                   // next parity of each stage's `full` barrier (see the producer)
        bool ok = true;
        long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define DC_CLK() (p.prof ? clock64() : 0ll)
        for (l = 0; l < p.L; ++l) {
            long long q0c = DC_CLK(), q1c;
            const int buf = l & 1;
            const uint32_t rph = uint32_t(l >> 1) & 1u;
            const float* recvb = recv + buf * kMaxCS * C::SRC_FLOATS;
            const uint32_t rbar_local = smem_u32(&bars->recv[buf]);
            if (tid == 0) mbar_arrive_expect_tx(rbar_local, uint32_t(CS) * (C::ZF * 4 + 8));   // arm this layer's receive

            // ---- V phase: rows [warp*RW, warp*RW+RW) of V', this lane's 8 columns, both token rows
            const float4 ha0 = *reinterpret_cast<const float4*>(hs + kcol0);
            const float4 ha1 = *reinterpret_cast<const float4*>(hs + kcol0 + 4);
            const float4 hb0 = *reinterpret_cast<const float4*>(hs + kSC + kcol0);
            const float4 hb1 = *reinterpret_cast<const float4*>(hs + kSC + kcol0 + 4);
            uint32_t vst[kVT];
#pragma unroll
            for (int kt = 0; kt < kVT; ++kt, rp.step(uint32_t(S))) vst[kt] = rp.st;
            ok = wait_cta(smem_u32(&bars->full[vst[0]]), (lead >> vst[0]) & 1u) && ok;   // all V' tiles of the layer
            lead ^= 1u << vst[0];
            { const long long qq = DC_CLK(); pc[5] += qq - q0c; }
            float v[C::NV];
#pragma unroll
            for (int i = 0; i < C::NV; ++i) v[i] = 0.f;
            if (ok) {
                const int q = lane >> 3;
                const uint8_t* tptr = ring + size_t(q == 0 ? vst[0] : q == 1 ? vst[1] : q == 2 ? vst[2] : vst[3]) * kStage;
#pragma unroll
                for (int i = 0; i < C::RW; ++i) {
                    const int rr = warp * C::RW + i;
                    const uint4 wv = *reinterpret_cast<const uint4*>(tptr + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
                    fma8(v[2 * i], wv, ha0, ha1);
                    fma8(v[2 * i + 1], wv, hb0, hb1);
                }
            }
            { const long long qq = DC_CLK(); pc[6] += qq - q0c; }
            __syncwarp();
            if (lane == 0)
                for (int kt = 0; kt < kVT; ++kt) mbar_arrive(smem_u32(&bars->empty[vst[kt]]));
            warp_reduce_scatter<C::NV>(v, lane);
            {
                constexpr int SH = C::NV == 32 ? 0 : (C::NV == 16 ? 1 : 2);
                if ((lane & ((1 << SH) - 1)) == 0) zp[warp * C::NV + (lane >> SH)] = v[0];
            }
            { const long long qq = DC_CLK(); pc[7] += qq - q0c; }
            if (!ok) *abort_flag = 1;
            bar_compute();
            if (*abort_flag) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
            q1c = DC_CLK(); pc[0] += q1c - q0c; q0c = q1c;

            // ---- exchange: partial z and partial sums of squares to every CTA of the cluster
            {
                const uint32_t base = uint32_t((buf * kMaxCS + int(rank)) * C::SRC_FLOATS) * 4u;
                if (tid < C::ZF / 4) {
                    const float4 z4 = *reinterpret_cast<const float4*>(zp + 4 * tid);
                    for (int dc = 0; dc < CS; ++dc)
                        st_async_v4f(mapa(recv_s + base + uint32_t(tid) * 16u, uint32_t(dc)), z4.x, z4.y, z4.z, z4.w,
                                     mapa(rbar_local, uint32_t(dc)));
                } else if (tid == kCompute - 1) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int w8 = 0; w8 < 8; ++w8) { s0 += wsum[2 * w8]; s1 += wsum[2 * w8 + 1]; }
                    for (int dc = 0; dc < CS; ++dc)
                        st_async_v2f(mapa(recv_s + base + uint32_t(C::ZF) * 4u, uint32_t(dc)), s0, s1,
                                     mapa(rbar_local, uint32_t(dc)));
                }
            }
            q1c = DC_CLK(); pc[1] += q1c - q0c; q0c = q1c;
            {
                int got = 0;
                if (lane == 0) {
                    for (uint32_t i = 0; i < wlimit && !got; ++i) {
                        got = mbar_try_wait_cluster(rbar_local, rph) ? 1 : 0;
                        if (!got && (i & 63u) == 63u && *abort_flag) break;
                    }
                }
                ok = ok && __shfl_sync(0xffffffffu, got, 0) != 0;
            }
            q1c = DC_CLK(); pc[2] += q1c - q0c; q0c = q1c;
            // ---- add up the CS partials, normalise, SiLU
            if (ok && tid < C::ZF) {
                float z = 0.f, q = 0.f;
#pragma unroll 4
                for (int src = 0; src < CS; ++src) {
                    z += recvb[src * C::SRC_FLOATS + tid];
                    q += recvb[src * C::SRC_FLOATS + C::ZF + (tid & 1)];
                }
                ssm[tid] = silu_f(z * rsqrtf(q * p.inv_d + p.eps));
            }
            if (!ok) *abort_flag = 1;
            bar_compute();
            if (*abort_flag) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
            q1c = DC_CLK(); pc[3] += q1c - q0c; q0c = q1c;

            // ---- U phase: column `tid` of the stripe: dot of its U' row with s, both token rows
            // four partial sums per token row: the products of a chunk are independent, one accumulator each would
            // make the phase a chain of dependent FMAs
            float d0 = 0.f, d1 = 0.f, e0 = 0.f, e1 = 0.f, f0 = 0.f, f1 = 0.f, g0 = 0.f, g1 = 0.f;
            ok = wait_cta(smem_u32(&bars->full[rp.st]), (lead >> rp.st) & 1u) && ok;            // all U' tiles of the layer
            lead ^= 1u << rp.st;
#pragma unroll 1
            for (int j = 0; j < C::UT; ++j, rp.step(uint32_t(S))) {
                const int rb = j / C::UK, kh = j % C::UK;
                const uint32_t st = rp.st;
                if (ok && rb == urb) {
                    const uint8_t* tptr = ring + size_t(st) * kStage;
#pragma unroll
                    for (int ch = 0; ch < C::KW / 8; ++ch) {
                        const uint32_t off = swz(uint32_t(urow) * (C::KW * 2) + ch * 16, C::UBITS);
                        const uint4 wv = *reinterpret_cast<const uint4*>(tptr + off);
                        const float* sp = ssm + (kh * C::KW + 8 * ch) * 2;
                        const float4 a = *reinterpret_cast<const float4*>(sp);
                        const float4 b = *reinterpret_cast<const float4*>(sp + 4);
                        const float4 c = *reinterpret_cast<const float4*>(sp + 8);
                        const float4 e = *reinterpret_cast<const float4*>(sp + 12);
                        const float w0 = bf16lo_to_f(wv.x), w1 = bf16hi_to_f(wv.x), w2 = bf16lo_to_f(wv.y), w3 = bf16hi_to_f(wv.y);
                        const float w4 = bf16lo_to_f(wv.z), w5 = bf16hi_to_f(wv.z), w6 = bf16lo_to_f(wv.w), w7 = bf16hi_to_f(wv.w);
                        d0 = fmaf(w0, a.x, d0); d1 = fmaf(w0, a.y, d1);
                        e0 = fmaf(w1, a.z, e0); e1 = fmaf(w1, a.w, e1);
                        f0 = fmaf(w2, b.x, f0); f1 = fmaf(w2, b.y, f1);
                        g0 = fmaf(w3, b.z, g0); g1 = fmaf(w3, b.w, g1);
                        d0 = fmaf(w4, c.x, d0); d1 = fmaf(w4, c.y, d1);
                        e0 = fmaf(w5, c.z, e0); e1 = fmaf(w5, c.w, e1);
                        f0 = fmaf(w6, e.x, f0); f1 = fmaf(w6, e.y, f1);
                        g0 = fmaf(w7, e.z, g0); g1 = fmaf(w7, e.w, g1);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->empty[st]));
            }
            h0 += (d0 + e0) + (f0 + g0);
            h1 += (d1 + e1) + (f1 + g1);
            publish_h();
            if (!ok) *abort_flag = 1;
            bar_compute();
            if (*abort_flag) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
            q1c = DC_CLK(); pc[4] += q1c - q0c;
        }
        if (p.prof && tid == 0 && blockIdx.x == 0)
            for (int k = 0; k < 8; ++k) p.prof[k] = (unsigned long long)pc[k];
        if (err) {
            if (tid == 0) atomicCAS(p.status, 0, err | (l << 8));
        } else {
            if (rows > 0) p.y[size_t(row0) * p.d + stripe0 + tid] = __float2bfloat16_rn(h0);
            if (rows > 1) p.y[size_t(row0 + 1) * p.d + stripe0 + tid] = __float2bfloat16_rn(h1);
        }
    }
    __syncwarp();
    __syncthreads();
    // no CTA may leave while a peer can still write into its shared memory
    cluster_arrive_release();
    cluster_wait_acquire();
}

template <int R>
int launch_dc(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int L, float eps,
              int* status_dev, cudaStream_t stream, int smem_optin, unsigned int spin_limit, dlrb200_plan* plan_only,
              unsigned long long* prof) {
    using C = DCfg<R>;
    auto kern = dlr_decode_cluster_kernel<R>;
    const int cs = d / kSC;
    int stages = (smem_optin - C::FIXED_BYTES) / kStage;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < kVT + 1) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    const int smem = stages * kStage + C::FIXED_BYTES;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return DLRB200_ERR_CUDA;
    if (cs > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
        return DLRB200_ERR_CUDA;
    const int clusters = (M + kNR - 1) / kNR;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(kThreadsDC);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(cs * clusters);
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) return DLRB200_ERR_CUDA;
    if (max_clusters < 1) return DLRB200_ERR_OCCUPANCY;
    if (plan_only) {
        plan_only->path = DLRB200_PATH_CLUSTER_SMALL;
        plan_only->grid = cs * clusters;
        plan_only->cluster = cs;
        plan_only->stripe_cols = kSC;
        plan_only->rows_per_pass = kNR;
        plan_only->passes = 1;
        plan_only->stages = stages;
        plan_only->smem_bytes = size_t(smem);
        return DLRB200_OK;
    }
    DCParams p;
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.y = static_cast<__nv_bfloat16*>(y);
    p.M = M; p.d = d; p.L = L; p.eps = eps; p.inv_d = 1.0f / float(d);
    p.status = status_dev;
    p.spin_limit = spin_limit;
    p.stages = stages;
    p.cs = cs;
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

int dispatch_dc(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L, float eps,
                int* status_dev, cudaStream_t stream, int smem_optin, unsigned int spin_limit, dlrb200_plan* plan_only,
                unsigned long long* prof) {
    switch (r) {
        case 32: return launch_dc<32>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, smem_optin, spin_limit, plan_only, prof);
        case 64: return launch_dc<64>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, smem_optin, spin_limit, plan_only, prof);
        case 128: return launch_dc<128>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, smem_optin, spin_limit, plan_only, prof);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace

bool decode_cluster_supported(int d, int r) {
    return (r == 32 || r == 64 || r == 128) && d % kSC == 0 && d / kSC >= 1 && d / kSC <= kMaxCS;
}

int decode_cluster_plan(int M, int d, int r, int L, int smem_optin, dlrb200_plan* plan) {
    const size_t ws = plan->workspace_bytes;
    const int rc = dispatch_dc(nullptr, nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, smem_optin, 0,
                               plan, nullptr);
    plan->workspace_bytes = ws;
    return rc;
}

int decode_cluster_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d,
                           int r, int L, float eps, int* status_dev, cudaStream_t stream, int smem_optin,
                           unsigned int spin_limit, unsigned long long* prof) {
    return dispatch_dc(encode_fn_ptr, x, y, Vp, Up, M, d, r, L, eps, status_dev, stream, smem_optin, spin_limit, nullptr,
                       prof);
}

}  // namespace dlr
