// Small-batch ("decode") DLR-Net forward for up to 64 token rows, two-level exchange: the width-striped
// grid of decode.cu (CTA c owns columns [c*DC, (c+1)*DC) for both contractions of a layer, the activation
// never leaves its CTA: the idea of kernels/kernels/cuda/cooperative.cu:10-16; per-layer math of
// dlr_lock/model.py:96-100 on folded weights) launched as clusters of eight CTAs.
//
// Why.  With more than a few rows the per-layer exchange of decode.cu is what a layer costs: every CTA adds
// its partial z (rows x r values) into the same words of L2, 64 atomics per word and layer, and reads all of
// them back.  Here the eight CTAs of a cluster first reduce among themselves through distributed shared
// memory and only the cluster sums go through L2:
//   1. every CTA computes its partial z over its stripe (mma.sync, weights as the 16-row operand) into
//      shared memory;
//   2. reduce-scatter inside the cluster: z's columns are dealt out to the eight CTAs (r/8 each), every CTA
//      sends each owner its slice with st.async (16-byte stores whose bytes are counted on the owner's
//      mbarrier: no fences); the partial sums of squares go to rank 0;
//   3. the owner adds the eight partials in rank order and adds the result, in fixed point with an arrival
//      count in the top bits of the word (see decode.cu), into words of L2 that belong to this layer alone:
//      one atomic per word and CLUSTER, nothing to clear or to subtract;
//   4. it polls just its own words until every cluster has arrived, every CTA polls the sums of squares,
//      the owner applies 1/rms and SiLU to its slice and
//   5. all-gathers s (bf16) into the operand tile of every CTA of the cluster, again with st.async;
//   6. every CTA updates its stripe (h += s . U'^T), as in decode.cu.
// L2 sees (rows x r) / 8 atomics per CTA instead of rows x r, and (rows x r) / 8 words read back instead
// of all of them.  The sums are integers: the result does not depend on the order of arrival.
//
// All waits are bounded; a wait that gives up records a status word and the CTA drains and leaves; the
// cluster leaves together.
#include <cstring>

#include "decode_tl.h"
#include "ptx.cuh"

namespace dlr {

namespace {

constexpr int kThreadsT = 256;
constexpr int kWarpsT = kThreadsT / 32;
constexpr int kCS = 8;                            // CTAs per cluster
constexpr double kZScaleT = 16777216.0;           // 2^24: partial z, scaled by the row's 1/rms of the layer before
constexpr double kQScaleT = 65536.0;              // 2^16: sums of squares, scaled alike
constexpr unsigned long long kOneArrivalT = 1ull << 48;

__device__ __forceinline__ void red_add_u64_t(unsigned long long* p, unsigned long long v) {
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_volatile_u64_t(const unsigned long long* p) {
    unsigned long long a;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return a;
}
__device__ __forceinline__ unsigned int word_count_t(unsigned long long w) { return unsigned((w + (1ull << 47)) >> 48) & 0xffffu; }
__device__ __forceinline__ long long word_sum_t(unsigned long long w) {
    return static_cast<long long>(w - (((w + (1ull << 47)) >> 48) << 48));
}
__device__ __forceinline__ void st_async_b64(uint32_t dst_cluster, uint32_t lo, uint32_t hi, uint32_t bar_cluster) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(dst_cluster),
                 "r"(lo), "r"(hi), "r"(bar_cluster)
                 : "memory");
}

template <int R, int DC, int NT>
struct TLCfg {
    static constexpr int MP = 8 * NT;                 // padded rows
    static constexpr int RP = R + 4;                  // words per row of the layer's accumulator; [R] = sum of squares
    static constexpr int SW = R / kCS;                // columns of z per owner
    static constexpr int KW = R < 64 ? R : 64;        // columns per U tile (one swizzle span)
    static constexpr int UT = R / KW;
    static constexpr int VBITS = DC == 16 ? 1 : (DC == 32 ? 2 : 3);
    static constexpr int UBITS = KW == 16 ? 1 : (KW == 32 ? 2 : 3);
    static constexpr int V_BYTES = R * DC * 2;
    static constexpr int U_TILE_BYTES = DC * KW * 2;
    static constexpr int STAGE_BYTES = 4 * R * DC;
    static constexpr int HS = DC + 4;                 // fp32 row stride of h
    static constexpr int HBS = DC + 8;                // bf16 row stride of the bf16 copy of h
    static constexpr int SS = R + 8;                  // bf16 row stride of silu(z)
    static constexpr int ZS = R + 4;                  // fp32 row stride of the partial z
    static constexpr int MT_V = R / 16;
    static constexpr int MT_U = DC / 16;
    static constexpr int KS_V = DC / 16;
    static constexpr int KS_U = R / 16;
    static constexpr int KSPLIT_RAW = kWarpsT / (MT_U * NT) > 0 ? kWarpsT / (MT_U * NT) : 1;
    static constexpr int KSPLIT = KSPLIT_RAW > KS_U ? KS_U : KSPLIT_RAW;
    static constexpr int H_BYTES = MP * HS * 4;
    static constexpr int DHP_BYTES = KSPLIT * MP * HS * 4;
    static constexpr int ZP_BYTES = MP * ZS * 4;
    static constexpr int SCR_BYTES = DHP_BYTES > ZP_BYTES ? DHP_BYTES : ZP_BYTES;   // partial z, then the partial dh
    static constexpr int HB_BYTES = MP * HBS * 2;
    static constexpr int S_BYTES = MP * SS * 2;
    static constexpr int RECV_BYTES = kCS * MP * SW * 4;                  // [rank][row][SW] partial z of this owner's slice
    static constexpr int RECVQ_BYTES = kCS * MP * 4;                      // [rank][row] partial sums of squares (rank 0 owns them)
    static constexpr int FIXED_BYTES = H_BYTES + SCR_BYTES + HB_BYTES + S_BYTES + RECV_BYTES + RECVQ_BYTES + 3 * MP * 4 +
                                       1024 /*barriers+flags*/ + 1024 /*alignment slack*/;
};

template <int R, int DC, int NT>
__global__ void __launch_bounds__(kThreadsT, 1)
dlr_decode_tl_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU, DecodeTLParams p) {
    using C = TLCfg<R, DC, NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int S = p.stages;
    uint8_t* ring = smem;
    float* h = reinterpret_cast<float*>(ring + size_t(S) * C::STAGE_BYTES);
    float* scr = h + C::MP * C::HS;                                       // zp [MP][ZS] in the V phase, dhp in the U phase
    __nv_bfloat16* hb = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(scr) + C::SCR_BYTES);
    __nv_bfloat16* sb = hb + C::MP * C::HBS;
    float* recv = reinterpret_cast<float*>(sb + C::MP * C::SS);           // [kCS][MP][SW]
    float* recvq = recv + kCS * C::MP * C::SW;                            // [kCS][MP]
    float* qpart = recvq + kCS * C::MP;                                   // [MP] this CTA's partial sums of squares
    float* rs_sh = qpart + C::MP;                                         // [2][MP] 1/rms per row: layer before / this layer
    uint64_t* full = reinterpret_cast<uint64_t*>(rs_sh + 2 * C::MP);      // [32] weight stages
    uint64_t* rbar = full + 32;                                           // partial z of my slice has arrived (bytes)
    uint64_t* sbar = rbar + 1;                                            // s of all slices has arrived (bytes)
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sbar + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;   // mma "group" index
    const int t = lane & 3;    // thread in group
    const int cta = blockIdx.x;
    const int G = gridDim.x;
    const int NC = G / kCS;                                               // clusters: arrivals per word and layer
    const int M = p.M;
    const int col0 = cta * DC;
    const uint32_t rank = cluster_ctarank();
    const uint32_t ring_s = smem_u32(ring);
    unsigned long long* words = p.words;                                  // [L][MP][RP], zero on entry
    float* pre = p.pre;                                                   // [G][64]: every CTA's sums of squares of the input

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(&full[s]), 1);
        mbar_init(smem_u32(rbar), 1);
        mbar_init(smem_u32(sbar), 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmU);
    }
    __syncthreads();
    // the peers' barriers must exist before anyone sends to them
    cluster_arrive_release();
    cluster_wait_acquire();

    auto issue_layer = [&](int layer, int st) {   // st == layer % S, kept by stepping (no division in the loop)
        const uint32_t bar = smem_u32(&full[st]);
        const uint32_t dst = ring_s + uint32_t(st) * C::STAGE_BYTES;
        mbar_arrive_expect_tx(bar, C::STAGE_BYTES);
        tma_load_2d(dst, &tmV, col0, layer * R, bar);
#pragma unroll
        for (int ut = 0; ut < C::UT; ++ut)
            tma_load_2d(dst + C::V_BYTES + ut * C::U_TILE_BYTES, &tmU, ut * C::KW, layer * p.d + col0, bar);
    };
    if (tid == 0) {
        const int ahead = S < p.L ? S : p.L;
        for (int l = 0; l < ahead; ++l) issue_layer(l, l);
    }

    // ---- load the input stripe: h (fp32), its bf16 copy, partial sum of squares
    constexpr int GPR = DC / 4;              // threads per row (4 columns each)
    constexpr int RPP = kThreadsT / GPR;     // rows per pass
#pragma unroll 1
    for (int row0 = 0; row0 < C::MP; row0 += RPP) {
        const int row = row0 + tid / GPR;
        const int cg = tid % GPR;
        if (row < C::MP) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            uint2 raw = make_uint2(0u, 0u);
            if (row < M) {
                raw = *reinterpret_cast<const uint2*>(p.x + size_t(row) * p.d + col0 + 4 * cg);
                v.x = bf16lo_to_f(raw.x); v.y = bf16hi_to_f(raw.x);
                v.z = bf16lo_to_f(raw.y); v.w = bf16hi_to_f(raw.y);
            }
            *reinterpret_cast<uint2*>(hb + row * C::HBS + 4 * cg) = raw;
            *reinterpret_cast<float4*>(h + row * C::HS + 4 * cg) = v;
            float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
            for (int o = GPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (cg == 0 && row < M) pre[cta * 64 + row] = ss;      // summed in a fixed order below: repeatable
        }
    }
    // rows past the batch never receive s: keep their operand rows at zero
    for (int i = tid; i < C::MP * C::SS / 2; i += kThreadsT) reinterpret_cast<uint32_t*>(sb)[i] = 0u;

    int err = 0;
    int l = 0;
    bool nothing_consumed = false;           // gave up before the first layer's weights were waited for
    {
        // ---- the sums of squares of the input, once, through a plain grid barrier: every later layer scales
        // its partials by the 1/rms before it
        __threadfence();
        __syncthreads();
        bool failed = false;
        if (tid == 0) {
            red_release_add_u32(p.counter, 1u);
            unsigned int spins = 0;
            while (ld_acquire_u32(p.counter) < unsigned(G)) {
                if (++spins > p.spin_limit) { failed = true; break; }
            }
        }
        if (__syncthreads_or(failed)) { err = DLRB200_ERR_TIMEOUT_BARRIER; nothing_consumed = true; }
        if (tid < C::MP) {
            float q = 0.f;
            if (tid < M && !err)
                for (int c = 0; c < G; ++c) q += __ldcg(pre + c * 64 + tid);
            rs_sh[tid] = rsqrtf(q * p.inv_d + p.eps);
        }
        __syncthreads();
    }

    // this owner's slice of (row, column) values: 4 consecutive columns per thread
    constexpr int SLICE = C::MP * C::SW;                 // values of one slice
    constexpr int VPT = 4;                               // (eight per thread, one 16-byte store of s per destination, measured slower)
    constexpr int SL_ITERS = (SLICE / VPT + kThreadsT - 1) / kThreadsT;
    const uint32_t rbar_s = smem_u32(rbar), sbar_s = smem_u32(sbar);
    const uint32_t z_bytes = uint32_t(kCS * M * C::SW * 4);              // into an owner per layer
    const uint32_t q_bytes = uint32_t(kCS * M * 4);                      // into rank 0 per layer (not for layer 0)
    const uint32_t s_bytes = uint32_t(M * R * 2);                        // s into every CTA per layer

    RingPos rpos;
#pragma unroll 1
    for (; l < p.L && !err; ++l, rpos.step(uint32_t(S))) {
        const int st = int(rpos.st);
        const uint32_t ph = rpos.ph;
        const uint32_t lpar = uint32_t(l) & 1u;
        const uint32_t vbase = ring_s + uint32_t(st) * C::STAGE_BYTES;
        const uint32_t ubase = vbase + C::V_BYTES;
        const float* nrm = rs_sh + (l & 1) * C::MP;                      // 1/rms of the layer before (of the input at l = 0)
        float* rnext = rs_sh + ((l + 1) & 1) * C::MP;
        unsigned long long* wl = words + size_t(l) * C::MP * C::RP;

        // (A) weights of this layer have landed; also orders the previous layer's writes of hb before the reads below
        const bool landed = mbar_wait(smem_u32(&full[st]), ph, p.spin_limit >> 4);
        if (__syncthreads_or(!landed)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
        if (tid == 0) {
            mbar_arrive_expect_tx(rbar_s, z_bytes + ((rank == 0 && l > 0) ? q_bytes : 0u));
            mbar_arrive_expect_tx(sbar_s, s_bytes);
        }

        // ---- V phase: z_part[row][r] over this stripe -> shared memory.  A warp keeps one 16-row tile of the
        // weights and walks its share of the 8-row token tiles with it: one ldmatrix per k-step feeds up to eight
        // independent MMAs (a chain of dependent mma.sync costs its latency per step).
        float* zp = scr;
        {
            constexpr int WPM = C::MT_V >= kWarpsT ? 1 : kWarpsT / C::MT_V;        // warps that share a weight tile
            constexpr int NPW = (NT + WPM - 1) / WPM;                              // token tiles per warp
#pragma unroll 1
            for (int mt = warp % C::MT_V; mt < C::MT_V; mt += (C::MT_V >= kWarpsT ? kWarpsT : C::MT_V)) {
                const int sub = C::MT_V >= kWarpsT ? 0 : warp / C::MT_V;
                float c[NPW][4];
#pragma unroll
                for (int i = 0; i < NPW; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < C::KS_V; ++ks) {
                    const int arow = 16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const uint32_t off = uint32_t(arow) * (DC * 2) + ks * 32 + (lane >> 4) * 16;
                    uint32_t a0, a1, a2, a3;
                    ldmatrix_x4(vbase + swz(off, C::VBITS), a0, a1, a2, a3);
#pragma unroll
                    for (int i = 0; i < NPW; ++i) {
                        const int nt = sub + i * WPM;
                        if (nt < NT) {
                            const __nv_bfloat16* bp = hb + (8 * nt + g) * C::HBS + 16 * ks + 2 * t;
                            mma_bf16_16816(c[i], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(bp),
                                           *reinterpret_cast<const uint32_t*>(bp + 8));
                        }
                    }
                }
                // c[0], c[2]: token row n0, z columns rr, rr+8;  c[1], c[3]: token row n0+1
                const int rr = 16 * mt + g;
#pragma unroll
                for (int i = 0; i < NPW; ++i) {
                    const int nt = sub + i * WPM;
                    if (nt < NT) {
                        const int n0 = 8 * nt + 2 * t;
                        zp[n0 * C::ZS + rr] = c[i][0];
                        zp[n0 * C::ZS + rr + 8] = c[i][2];
                        zp[(n0 + 1) * C::ZS + rr] = c[i][1];
                        zp[(n0 + 1) * C::ZS + rr + 8] = c[i][3];
                    }
                }
            }
        }
        __syncthreads();  // (B) the partial z of this CTA is complete

        // ---- reduce-scatter: slice k of every row goes to CTA k of the cluster (its own slice too, the same way)
        {
            constexpr int VEC_PER_ROW = C::SW / 4;                       // 16-byte stores per row and owner
            const int total = kCS * M * VEC_PER_ROW;
            for (int i = tid; i < total; i += kThreadsT) {
                const int k = i / (M * VEC_PER_ROW);
                const int rem = i - k * (M * VEC_PER_ROW);
                const int row = rem / VEC_PER_ROW;
                const int j4 = rem - row * VEC_PER_ROW;
                const float4 v = *reinterpret_cast<const float4*>(zp + row * C::ZS + k * C::SW + 4 * j4);
                const uint32_t dst = mapa(smem_u32(recv + (int(rank) * C::MP + row) * C::SW + 4 * j4), uint32_t(k));
                st_async_v4(dst, __float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w),
                            mapa(rbar_s, uint32_t(k)));
            }
            if (l > 0 && tid < M)      // the sums of squares after layer l-1, to rank 0
                st_async_b32(mapa(smem_u32(recvq + int(rank) * C::MP + tid), 0u), __float_as_uint(qpart[tid]), mapa(rbar_s, 0u));
        }

        // ---- owner: the eight partials of my slice, added in rank order, go to this layer's words in L2
        bool failed = !mbar_wait_cluster(rbar_s, lpar, p.spin_limit >> 4);
        if (!failed) {
#pragma unroll
            for (int it = 0; it < SL_ITERS; ++it) {
                const int v0 = VPT * (tid + it * kThreadsT);
                if (v0 < SLICE) {
                    const int row = v0 / C::SW, j = v0 % C::SW;
                    if (row < M) {
                        const double sc = double(nrm[row]) * kZScaleT;
#pragma unroll
                        for (int q4 = 0; q4 < VPT / 4; ++q4) {
                            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int k = 0; k < kCS; ++k) {
                                const float4 v = *reinterpret_cast<const float4*>(recv + (k * C::MP + row) * C::SW + j + 4 * q4);
                                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                            }
                            unsigned long long* w = wl + size_t(row) * C::RP + int(rank) * C::SW + j + 4 * q4;
                            red_add_u64_t(w + 0, static_cast<unsigned long long>(__double2ll_rn(double(acc.x) * sc)) + kOneArrivalT);
                            red_add_u64_t(w + 1, static_cast<unsigned long long>(__double2ll_rn(double(acc.y) * sc)) + kOneArrivalT);
                            red_add_u64_t(w + 2, static_cast<unsigned long long>(__double2ll_rn(double(acc.z) * sc)) + kOneArrivalT);
                            red_add_u64_t(w + 3, static_cast<unsigned long long>(__double2ll_rn(double(acc.w) * sc)) + kOneArrivalT);
                        }
                    }
                }
            }
            if (rank == 0 && l > 0 && tid < M) {
                float q = 0.f;
#pragma unroll
                for (int k = 0; k < kCS; ++k) q += recvq[k * C::MP + tid];
                const double sc = double(nrm[tid]) * double(nrm[tid]) * kQScaleT;
                red_add_u64_t(wl + size_t(tid) * C::RP + R, static_cast<unsigned long long>(__double2ll_rn(double(q) * sc)) + kOneArrivalT);
            }
        }

        // ---- every CTA: this layer's 1/rms per row, from the sums of squares of all clusters
        if (!failed && tid < C::MP) {
            float rstd = nrm[tid];                              // layer 0: the input's 1/rms, known already
            if (l > 0 && tid < M) {
                const unsigned long long* wq = wl + size_t(tid) * C::RP + R;
                unsigned long long w = 0;
                bool ok = false;
                for (unsigned int spins = 0; spins < p.spin_limit; ++spins) {
                    w = ld_volatile_u64_t(wq);
                    if (word_count_t(w) == unsigned(NC)) { ok = true; break; }
                    if ((spins & 0x3ffu) == 0x3ffu && *reinterpret_cast<volatile int*>(p.status) != 0) break;
                }
                if (!ok) failed = true;
                const float rp = nrm[tid];
                const float q = float(double(word_sum_t(w)) * (1.0 / kQScaleT)) / (rp * rp);
                rstd = rsqrtf(q * p.inv_d + p.eps);
            }
            rnext[tid] = rstd;
        }
        if (__syncthreads_or(failed)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }   // (C) rnext visible

        // ---- owner: my slice of z is complete once every cluster has arrived; s = silu(z * rstd) to every CTA
#pragma unroll
        for (int it = 0; it < SL_ITERS; ++it) {
            const int v0 = VPT * (tid + it * kThreadsT);
            if (v0 < SLICE) {
                const int row = v0 / C::SW, j = v0 % C::SW;
                if (row < M) {
                    const unsigned long long* w = wl + size_t(row) * C::RP + int(rank) * C::SW + j;
                    unsigned long long wv[VPT];
                    bool ok = false;
                    for (unsigned int spins = 0; spins < p.spin_limit; ++spins) {
                        bool all = true;
#pragma unroll
                        for (int e = 0; e < VPT; ++e) {
                            wv[e] = ld_volatile_u64_t(w + e);
                            all = all && word_count_t(wv[e]) == unsigned(NC);
                        }
                        if (all) { ok = true; break; }
                        if ((spins & 0x3ffu) == 0x3ffu && *reinterpret_cast<volatile int*>(p.status) != 0) break;
                    }
                    if (!ok) failed = true;
                    const float sc = rnext[row] / nrm[row] * float(1.0 / kZScaleT);
                    uint32_t pk[VPT / 2];
#pragma unroll
                    for (int e = 0; e < VPT / 2; ++e)
                        pk[e] = pack_bf16x2(silu_f(float(word_sum_t(wv[2 * e])) * sc), silu_f(float(word_sum_t(wv[2 * e + 1])) * sc));
                    const uint32_t dst_local = smem_u32(sb + row * C::SS + int(rank) * C::SW + j);
#pragma unroll
                    for (int k = 0; k < kCS; ++k) {
                        if constexpr (VPT == 8) st_async_v4(mapa(dst_local, uint32_t(k)), pk[0], pk[1], pk[2], pk[3], mapa(sbar_s, uint32_t(k)));
                        else st_async_b64(mapa(dst_local, uint32_t(k)), pk[0], pk[1], mapa(sbar_s, uint32_t(k)));
                    }
                }
            }
        }
        // ---- s of all eight slices has arrived in my operand tile
        if (!failed) failed = !mbar_wait_cluster(sbar_s, lpar, p.spin_limit >> 4);
        if (__syncthreads_or(failed)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }   // (D) also: zp is free for dh

        // ---- U phase: dh[stripe col][row]; same reuse of the weight fragment across token tiles, and a split
        // over k when there are fewer (weight tile, token tile) pairs than warps
        float* dhp = scr;
        {
            constexpr int WPM = kWarpsT / C::MT_U;                                  // warps that share a weight tile (2 or 4)
            constexpr int WN = C::KSPLIT > 1 ? WPM / C::KSPLIT : WPM;               // of which along the token tiles
            constexpr int NPW = (NT + WN - 1) / WN;                                 // token tiles per warp
            const int mt = warp % C::MT_U;
            const int sub = warp / C::MT_U;
            const int kp = C::KSPLIT > 1 ? sub / WN : 0;
            const int sn = C::KSPLIT > 1 ? sub % WN : sub;
            float c[NPW][4];
#pragma unroll
            for (int i = 0; i < NPW; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < C::KS_U / C::KSPLIT; ++kk) {
                const int ks = kp * (C::KS_U / C::KSPLIT) + kk;
                const int tile = (16 * ks) / C::KW;
                const int kin = (16 * ks) % C::KW;
                const int arow = 16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8;
                const uint32_t off = uint32_t(arow) * (C::KW * 2) + kin * 2 + (lane >> 4) * 16;
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(ubase + tile * C::U_TILE_BYTES + swz(off, C::UBITS), a0, a1, a2, a3);
#pragma unroll
                for (int i = 0; i < NPW; ++i) {
                    const int nt = sn + i * WN;
                    if (nt < NT) {
                        const __nv_bfloat16* bp = sb + (8 * nt + g) * C::SS + 16 * ks + 2 * t;
                        mma_bf16_16816(c[i], a0, a1, a2, a3, *reinterpret_cast<const uint32_t*>(bp),
                                       *reinterpret_cast<const uint32_t*>(bp + 8));
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < NPW; ++i) {
                const int nt = sn + i * WN;
                if (nt < NT) {
                    float* o = dhp + (kp * C::MP + 8 * nt + 2 * t) * C::HS + 16 * mt + g;
                    o[0] = c[i][0];
                    o[C::HS] = c[i][1];
                    o[8] = c[i][2];
                    o[C::HS + 8] = c[i][3];
                }
            }
        }
        __syncthreads();  // (E) stage fully consumed, dh partials visible

        if (tid == 0 && l + S < p.L) issue_layer(l + S, st);

        // ---- h += dh ; partial sum of squares and bf16 copy for the next layer
        const bool last = (l + 1 == p.L);
#pragma unroll 1
        for (int row0 = 0; row0 < C::MP; row0 += RPP) {
            const int row = row0 + tid / GPR;
            const int cg = tid % GPR;
            if (row < C::MP) {
                float4 v = *reinterpret_cast<float4*>(h + row * C::HS + 4 * cg);
#pragma unroll
                for (int kp = 0; kp < C::KSPLIT; ++kp) {
                    const float4 a = *reinterpret_cast<const float4*>(dhp + (kp * C::MP + row) * C::HS + 4 * cg);
                    v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
                }
                *reinterpret_cast<float4*>(h + row * C::HS + 4 * cg) = v;
                uint2 packed;
                packed.x = pack_bf16x2(v.x, v.y);
                packed.y = pack_bf16x2(v.z, v.w);
                if (!last) {
                    *reinterpret_cast<uint2*>(hb + row * C::HBS + 4 * cg) = packed;
                    float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
                    for (int o = GPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                    if (cg == 0) qpart[row] = ss;
                } else if (row < M) {
                    *reinterpret_cast<uint2*>(p.y + size_t(row) * p.d + col0 + 4 * cg) = packed;
                }
            }
        }
        // (the barrier at (A) of the next layer orders qpart and hb before their readers)
    }

    if (err != 0) {
        // Give up: record why and where, then wait (bounded) for the copies still in flight into this CTA's
        // shared memory before leaving.
        if (tid == 0) {
            atomicCAS(p.status, 0, err | (l << 8));
            const int hi = (l + S < p.L) ? l + S : p.L;
            const int lo = (err == DLRB200_ERR_TIMEOUT_COPY || nothing_consumed) ? l : l + 1;
            for (int j = lo; j < hi; ++j) mbar_wait(smem_u32(&full[j % S]), (j / S) & 1, kDrainPolls);
        }
        __syncthreads();
    }
    // no CTA leaves while a peer may still send into its shared memory
    cluster_arrive_release();
    cluster_wait_acquire();
}

template <int R, int DC, int NT>
int launch_tl(const DecodeTLLaunch& a, dlrb200_plan* plan_only) {
    using C = TLCfg<R, DC, NT>;
    auto kern = dlr_decode_tl_kernel<R, DC, NT>;
    const int G = a.d / DC;
    if (G % kCS != 0 || G > a.num_sms) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    const int budget = a.smem_optin - C::FIXED_BYTES;
    int stages = budget / C::STAGE_BYTES;
    if (stages > 32) stages = 32;
    if (stages > a.L) stages = a.L;
    if (stages < 2 && a.L > 1) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    if (stages < 1) stages = 1;
    const int smem = stages * C::STAGE_BYTES + C::FIXED_BYTES;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return DLRB200_ERR_CUDA;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;      // every CTA of the grid resident at once: they wait for each other
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cfg.blockDim = dim3(kThreadsT);
    cfg.gridDim = dim3(G);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = a.stream;
    int max_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) return DLRB200_ERR_CUDA;
    if (max_clusters * kCS < G) return DLRB200_ERR_OCCUPANCY;
    if (plan_only) {
        plan_only->path = DLRB200_PATH_STRIPED_CLUSTERS;
        plan_only->grid = G;
        plan_only->cluster = kCS;
        plan_only->stripe_cols = DC;
        plan_only->rows_per_pass = a.p.M;
        plan_only->passes = 1;
        plan_only->stages = stages;
        plan_only->smem_bytes = size_t(smem);
        return DLRB200_OK;
    }
    DecodeTLParams p = a.p;
    p.stages = stages;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, a.tmV, a.tmU, p);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

template <int R, int DC>
int launch_tl_nt(const DecodeTLLaunch& a, dlrb200_plan* plan_only) {
    const int M = a.p.M;
    if (M <= 8) return launch_tl<R, DC, 1>(a, plan_only);
    if (M <= 16) return launch_tl<R, DC, 2>(a, plan_only);
    if (M <= 32) return launch_tl<R, DC, 4>(a, plan_only);
    return launch_tl<R, DC, 8>(a, plan_only);
}

template <int R>
int launch_tl_dc(const DecodeTLLaunch& a, dlrb200_plan* plan_only) {
    switch (a.dc) {
        case 32: return launch_tl_nt<R, 32>(a, plan_only);
        case 64: return launch_tl_nt<R, 64>(a, plan_only);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace

// one word per (layer, row, column of z or the sum of squares), then every CTA's sums of squares of the input
// (up to 160 CTAs x 64 rows), after 256 bytes of control words
size_t decode_tl_workspace_bytes(int M, int r, int L) {
    if (M > 64) return 0;
    const int mp = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    return 256 + size_t(L) * mp * (r + 4) * 8 + size_t(160) * 64 * 4;
}

size_t decode_tl_clear_bytes(int M, int r, int L) {
    const int mp = M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    return 256 + size_t(L) * mp * (r + 4) * 8;
}

bool decode_tl_supported(int d, int r, int dc) {
    return (r == 32 || r == 64 || r == 128 || r == 256) && (dc == 32 || dc == 64) && d % dc == 0 && (d / dc) % kCS == 0;
}

int decode_tl_launch(const DecodeTLLaunch& a, dlrb200_plan* plan_only) {
    switch (a.r) {
        case 32: return launch_tl_dc<32>(a, plan_only);
        case 64: return launch_tl_dc<64>(a, plan_only);
        case 128: return launch_tl_dc<128>(a, plan_only);
        case 256: return launch_tl_dc<256>(a, plan_only);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace dlr
