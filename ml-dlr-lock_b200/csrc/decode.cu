// Small-batch ("decode") DLR-Net forward: one launch walks all L layers for up
// to 64 token rows.
//
// Work split.  The model width d is cut into G stripes of DC columns; CTA c
// owns columns [c*DC, (c+1)*DC) for BOTH contractions of a layer:
//   z_part[row][0..r)  = h[row][stripe] . V'[:, stripe]^T      (K-stripe)
//   h[row][stripe]    += silu(z*rstd)[row][:] . U'[stripe, :]^T (N-stripe)
// so the activation never leaves its CTA (kept in shared memory in fp32 for
// all layers) and a layer needs exactly ONE cross-CTA exchange: the sum of the
// partial z and of the partial row sums of squares (same idea as the
// reference's cooperative kernels, kernels/kernels/cuda/cooperative.cu:10-16,
// 312-388; per-layer math of dlr_lock/model.py:96-100 on folded weights as in
// kernels/README.md:5-7).
//
// Exchange.  Partials are added with fp32 reductions into a small accumulator
// in global memory (three rotating slots so that no slot is cleared while a
// straggler still reads it), followed by a release-increment of an arrival
// counter; one thread per CTA polls the counter with acquire loads, with a
// poll limit.  The launch is cooperative, so all G CTAs are co-resident.
//
// Exchange for up to 16 rows (the latency-critical case).  The scheme above costs
// about three round trips to L2 per layer (reductions performed, counter seen,
// sums read).  With few rows every accumulator word is instead a 64-bit integer
// that carries its own arrival count: bits 48-63 count the CTAs that have added,
// bits 0-47 hold the sum in fixed point (values are first scaled by the row's
// 1/rms of the layer before, so the format does not depend on the scale of the
// input).  One red.add.u64 per value and CTA, then every thread polls just the
// words it needs until their counts are complete: about one and a half round
// trips, no counter, no fence.  Slots are never cleared: a CTA that adds into a
// slot again (three layers later) subtracts what it added then, exactly, since
// integer addition commutes; for the same reason the result does not depend on
// the order of arrival (the fp32 reductions do).
//
// Weight streaming.  Weights do not depend on activations, so each CTA keeps a
// ring of S layers of its weight slices in flight with TMA tiled loads that
// complete on mbarriers; the ring is refilled as soon as a layer is consumed.
// HBM traffic therefore runs ahead of the dependency chain.
//
// Tensor cores.  Both contractions use mma.sync m16n8k16 (bf16 in, fp32 out)
// with the WEIGHTS as the 16-row operand (ldmatrix from the swizzled TMA tile)
// and the token rows as the 8-wide operand, so one instruction shape covers
// 1..64 rows.
#include "decode.h"
#include "ptx.cuh"

namespace dlr {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// ---- counted 64-bit accumulator words (see "Exchange for up to 16 rows") ----
constexpr double kZScale = 16777216.0;      // 2^24: normalised partial z
constexpr double kQScale = 65536.0;         // 2^16: normalised partial sums of squares
constexpr unsigned long long kOneArrival = 1ull << 48;

__device__ __forceinline__ void red_add_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void ld_volatile_2xu64(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
    unsigned long long a;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
    return a;
}
// arrivals recorded in a word (the sum may be negative and borrow from the count: round to the nearest count)
__device__ __forceinline__ unsigned int word_count(unsigned long long w) { return unsigned((w + (1ull << 47)) >> 48) & 0xffffu; }
__device__ __forceinline__ long long word_sum(unsigned long long w) {
    return static_cast<long long>(w - (((w + (1ull << 47)) >> 48) << 48));
}

template <int R, int DC, int NT>
struct DecodeCfg {
    static constexpr int MP = 8 * NT;                 // padded rows
    static constexpr int RP = R + 4;                  // floats per accumulator row; [R] = sum of squares
    static constexpr int KW = R < 64 ? R : 64;        // columns per U tile (one swizzle span)
    static constexpr int UT = R / KW;                 // U tiles per stage
    static constexpr int VBITS = DC == 16 ? 1 : (DC == 32 ? 2 : 3);
    static constexpr int UBITS = KW == 16 ? 1 : (KW == 32 ? 2 : 3);
    static constexpr int V_BYTES = R * DC * 2;
    static constexpr int U_TILE_BYTES = DC * KW * 2;
    static constexpr int STAGE_BYTES = 4 * R * DC;
    static constexpr int HS = DC + 4;                 // fp32 row stride of h
    static constexpr int HBS = DC + 8;                // bf16 row stride of the bf16 copy of h
    static constexpr int SS = R + 8;                  // bf16 row stride of silu(z)
    static constexpr int MT_V = R / 16;
    static constexpr int MT_U = DC / 16;
    static constexpr int KS_V = DC / 16;
    static constexpr int KS_U = R / 16;
    static constexpr int KSPLIT_RAW = kWarps / (MT_U * NT) > 0 ? kWarps / (MT_U * NT) : 1;
    static constexpr int KSPLIT = KSPLIT_RAW > KS_U ? KS_U : KSPLIT_RAW;
    static constexpr int H_BYTES = MP * HS * 4;
    static constexpr int DHP_BYTES = KSPLIT * MP * HS * 4;
    static constexpr int HB_BYTES = MP * HBS * 2;
    static constexpr int S_BYTES = MP * SS * 2;
    static constexpr int FIXED_BYTES = H_BYTES + DHP_BYTES + HB_BYTES + S_BYTES + 1024 /*barriers+flags*/ +
                                       1024 /*alignment slack*/;
};

template <int R, int DC, int NT>
__global__ void __launch_bounds__(kThreads, 1)
dlr_decode_kernel(const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU,
                  DecodeParams p) {
    using C = DecodeCfg<R, DC, NT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

    const int S = p.stages;
    uint8_t* ring = smem;
    float* h = reinterpret_cast<float*>(ring + size_t(S) * C::STAGE_BYTES);
    float* dhp = h + C::MP * C::HS;
    __nv_bfloat16* hb = reinterpret_cast<__nv_bfloat16*>(dhp + C::KSPLIT * C::MP * C::HS);
    __nv_bfloat16* sb = hb + C::MP * C::HBS;
    uint64_t* full = reinterpret_cast<uint64_t*>(sb + C::MP * C::SS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(full + 32);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;   // mma "group" index
    const int t = lane & 3;    // thread in group
    const int cta = blockIdx.x;
    const int G = gridDim.x;
    const int M = p.M;
    const int col0 = cta * DC;
    const uint32_t ring_s = smem_u32(ring);
    // counted 64-bit exchange, up to 16 rows: beyond that a thread updates several rows per layer and the
    // bookkeeping of what it added (oldz, oldq) no longer fits
    constexpr bool CNT = NT <= 2;
    constexpr int VI = CNT ? (C::MT_V * NT + kWarps - 1) / kWarps : 1;   // V-phase items per warp
    unsigned long long* zs64 = reinterpret_cast<unsigned long long*>(p.zacc);   // [3][MP][RP]
    float* pre = reinterpret_cast<float*>(zs64 + 3 * C::MP * C::RP);  // [G][32]: every CTA's sums of squares of the input
    __shared__ float rs_sh[2][32];                                     // 1/rms per row: of the layer before / of this layer

    if (tid == 0) {
        for (int s = 0; s < S; ++s) mbar_init(smem_u32(&full[s]), 1);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmU);
    }
    __syncthreads();

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
        const int pre = S < p.L ? S : p.L;
        for (int l = 0; l < pre; ++l) issue_layer(l, l);
    }

    // ---- load the input stripe: h (fp32), its bf16 copy, partial sum of squares
    float* zacc = p.zacc;
    constexpr int GPR = DC / 4;              // threads per row (4 columns each)
    constexpr int RPP = kThreads / GPR;      // rows per pass
    {
#pragma unroll 1
        for (int row0 = 0; row0 < C::MP; row0 += RPP) {
            const int row = row0 + tid / GPR;
            const int cg = tid % GPR;
            if (row < C::MP) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (row < M) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(p.x + size_t(row) * p.d + col0 + 4 * cg);
                    v.x = bf16lo_to_f(raw.x); v.y = bf16hi_to_f(raw.x);
                    v.z = bf16lo_to_f(raw.y); v.w = bf16hi_to_f(raw.y);
                    *reinterpret_cast<uint2*>(hb + row * C::HBS + 4 * cg) = raw;
                } else {
                    *reinterpret_cast<uint2*>(hb + row * C::HBS + 4 * cg) = make_uint2(0u, 0u);
                }
                *reinterpret_cast<float4*>(h + row * C::HS + 4 * cg) = v;
                float ss = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
                for (int o = GPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (cg == 0 && row < M) {
                    if constexpr (CNT) pre[cta * 32 + row] = ss;       // summed in a fixed order below: repeatable
                    else red_add_f32(zacc + size_t(row) * C::RP + R, ss);
                }
            }
        }
    }

    int err = 0;
    int l = 0;
    bool nothing_consumed = false;           // gave up before the first layer's weights were waited for
    if constexpr (CNT) {
        // ---- the sums of squares of the input, once, through a plain barrier: every later layer scales by the
        // 1/rms before it
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
                for (int c = 0; c < G; ++c) q += __ldcg(pre + c * 32 + tid);
            rs_sh[0][tid] = rsqrtf(q * p.inv_d + p.eps);
            // an arrival without a value in the first slot's sum-of-squares words: every word of a slot then
            // counts the same number of arrivals per use
            if (tid < M) red_add_u64(zs64 + size_t(tid) * C::RP + R, kOneArrival);
        }
        __syncthreads();
    }
    long long oldz[3][VI][4];                // what this thread added to a slot the last three times (front = [0])
    long long oldq[3] = {0, 0, 0};
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int b = 0; b < VI; ++b)
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) oldz[a][b][c4] = 0;
    RingPos rpos;
#pragma unroll 1
    for (; l < p.L && !err; ++l, rpos.step(uint32_t(S))) {
        const int st = int(rpos.st);
        const uint32_t ph = rpos.ph;
        const int slot = l % 3;
        float* zs = zacc + size_t(slot) * C::MP * C::RP;
        const uint32_t vbase = ring_s + uint32_t(st) * C::STAGE_BYTES;
        const uint32_t ubase = vbase + C::V_BYTES;

        // (A) weights of this layer have landed; also orders the previous
        // layer's writes of hb before the reads below.
        const bool landed = mbar_wait(smem_u32(&full[st]), ph, p.spin_limit >> 4);
        if (__syncthreads_or(!landed)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }

        // ---- V phase: z_part[r][row] over this stripe, added into the accumulator
        if constexpr (CNT) {
            const float* nrm = rs_sh[l & 1];                       // 1/rms of the layer before (of the input at l = 0)
            unsigned long long* zw = zs64 + size_t(slot) * C::MP * C::RP;
#pragma unroll
            for (int vi = 0; vi < VI; ++vi) {
                const int item = warp + kWarps * vi;
                const int mt = item % C::MT_V;
                const int nt = item / C::MT_V;
                if (item < C::MT_V * NT) {
                    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int ks = 0; ks < C::KS_V; ++ks) {
                        const int arow = 16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8;
                        const uint32_t off = uint32_t(arow) * (DC * 2) + ks * 32 + (lane >> 4) * 16;
                        uint32_t a0, a1, a2, a3;
                        ldmatrix_x4(vbase + swz(off, C::VBITS), a0, a1, a2, a3);
                        const __nv_bfloat16* bp = hb + (8 * nt + g) * C::HBS + 16 * ks + 2 * t;
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bp);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(bp + 8);
                        mma_bf16_16816(c, a0, a1, a2, a3, b0, b1);
                    }
                    const int n0 = 8 * nt + 2 * t;
                    const int rr = 16 * mt + g;
                    // c[0], c[2]: row n0, columns rr, rr+8;  c[1], c[3]: row n0+1
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int row = n0 + (q & 1);
                        if (row < M) {
                            const long long e = __double2ll_rn(double(c[q]) * double(nrm[row]) * kZScale);
                            red_add_u64(zw + size_t(row) * C::RP + rr + 8 * (q >> 1),
                                        static_cast<unsigned long long>(e - oldz[0][vi][q]) + kOneArrival);
                            oldz[0][vi][q] = oldz[1][vi][q];
                            oldz[1][vi][q] = oldz[2][vi][q];
                            oldz[2][vi][q] = e;
                        }
                    }
                }
            }
        } else {
#pragma unroll 1
        for (int item = warp; item < C::MT_V * NT; item += kWarps) {
            const int mt = item % C::MT_V;
            const int nt = item / C::MT_V;
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < C::KS_V; ++ks) {
                const int arow = 16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8;
                const uint32_t off = uint32_t(arow) * (DC * 2) + ks * 32 + (lane >> 4) * 16;
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(vbase + swz(off, C::VBITS), a0, a1, a2, a3);
                const __nv_bfloat16* bp = hb + (8 * nt + g) * C::HBS + 16 * ks + 2 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bp);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(bp + 8);
                mma_bf16_16816(c, a0, a1, a2, a3, b0, b1);
            }
            const int n0 = 8 * nt + 2 * t;
            const int rr = 16 * mt + g;
            if (n0 < M) {
                red_add_f32(zs + size_t(n0) * C::RP + rr, c[0]);
                red_add_f32(zs + size_t(n0) * C::RP + rr + 8, c[2]);
            }
            if (n0 + 1 < M) {
                red_add_f32(zs + size_t(n0 + 1) * C::RP + rr, c[1]);
                red_add_f32(zs + size_t(n0 + 1) * C::RP + rr + 8, c[3]);
            }
        }
        __syncthreads();  // (B) every thread's reductions are issued

        // ---- arrive, then wait for all G stripes of this layer
        bool failed = false;
        if (tid == 0) {
            red_release_add_u32(p.counter, 1u);
            const unsigned int target = unsigned(G) * unsigned(l + 1);
            unsigned int spins = 0;
            while (ld_acquire_u32(p.counter) < target) {
                if (++spins > p.spin_limit) { failed = true; break; }
                if ((spins & 0x3ffu) == 0 && *reinterpret_cast<volatile int*>(p.status) != 0) {
                    failed = true;
                    break;
                }
            }
        }
        if (__syncthreads_or(failed)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }  // (C)
        }

        // ---- s = silu(z * rstd) as the 8-wide operand of the U phase
        if constexpr (CNT) {
            // every thread polls the words it needs until all G stripes have added to them
            const unsigned int target = (unsigned(l / 3 + 1) * unsigned(G)) & 0xffffu;
            const unsigned long long* zw = zs64 + size_t(slot) * C::MP * C::RP;
            const float* nrm = rs_sh[l & 1];
            float* rnext = rs_sh[(l + 1) & 1];
            bool failed = false;
            // 256 threads of 128 CTAs polling the very lines the reductions go to would slow those down: one
            // lane per warp watches one word (with a short back-off); the others look only once it is complete,
            // when theirs almost always are too
            if (lane == 0) {
                const unsigned long long* watch = zw + size_t(warp % M) * C::RP + R;
                unsigned int spins = 0;
                while (word_count(ld_volatile_u64(watch)) != target) {
                    if (++spins > p.spin_limit) { failed = true; break; }
                    if ((spins & 0xffu) == 0xffu && *reinterpret_cast<volatile int*>(p.status) != 0) { failed = true; break; }
                    __nanosleep(40);
                }
            }
            __syncwarp();
#pragma unroll 1
            for (int e = tid; e < C::MP * (R / 4); e += kThreads) {
                const int row = e / (R / 4);
                const int k4 = e % (R / 4);
                uint2 out = make_uint2(0u, 0u);
                if (row < M) {
                    unsigned long long w0 = 0, w1 = 0, w2 = 0, w3 = 0, wq = 0;
                    bool ok = false;
                    for (unsigned int spins = 0; spins < p.spin_limit; ++spins) {
                        ld_volatile_2xu64(zw + size_t(row) * C::RP + 4 * k4, w0, w1);
                        ld_volatile_2xu64(zw + size_t(row) * C::RP + 4 * k4 + 2, w2, w3);
                        wq = ld_volatile_u64(zw + size_t(row) * C::RP + R);
                        if (word_count(w0) == target && word_count(w1) == target && word_count(w2) == target &&
                            word_count(w3) == target && word_count(wq) == target) { ok = true; break; }
                        if ((spins & 0x3ffu) == 0x3ffu && *reinterpret_cast<volatile int*>(p.status) != 0) break;
                    }
                    if (!ok) failed = true;
                    const float rprev = nrm[row];
                    float rstd = rprev;                         // layer 0: the input's 1/rms, known already
                    if (l > 0) {
                        const float q = float(double(word_sum(wq)) * (1.0 / kQScale)) / (rprev * rprev);
                        rstd = rsqrtf(q * p.inv_d + p.eps);
                    }
                    if (k4 == 0) rnext[row] = rstd;
                    const float sc = rstd / rprev * float(1.0 / kZScale);
                    out.x = pack_bf16x2(silu_f(float(word_sum(w0)) * sc), silu_f(float(word_sum(w1)) * sc));
                    out.y = pack_bf16x2(silu_f(float(word_sum(w2)) * sc), silu_f(float(word_sum(w3)) * sc));
                }
                *reinterpret_cast<uint2*>(sb + row * C::SS + 4 * k4) = out;
            }
            if (__syncthreads_or(failed)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }  // (D)
        } else {
#pragma unroll 1
        for (int e = tid; e < C::MP * (R / 4); e += kThreads) {
            const int row = e / (R / 4);
            const int k4 = e % (R / 4);
            uint2 out = make_uint2(0u, 0u);
            if (row < M) {
                const float4 z = __ldcg(reinterpret_cast<const float4*>(zs + size_t(row) * C::RP + 4 * k4));
                const float ssq = __ldcg(zs + size_t(row) * C::RP + R);
                const float rstd = rsqrtf(ssq * p.inv_d + p.eps);
                out.x = pack_bf16x2(silu_f(z.x * rstd), silu_f(z.y * rstd));
                out.y = pack_bf16x2(silu_f(z.z * rstd), silu_f(z.w * rstd));
            }
            *reinterpret_cast<uint2*>(sb + row * C::SS + 4 * k4) = out;
        }
        // clear the slot that layer l+2 will use; every CTA has finished reading
        // it (it held layer l-1) before it arrived at this layer's barrier.
        {
            float* zclr = zacc + size_t((l + 2) % 3) * C::MP * C::RP;
            const int total = M * C::RP;
            const int per = (total + G - 1) / G;
            for (int i = tid; i < per; i += kThreads) {
                const int idx = cta * per + i;
                if (idx < total) zclr[idx] = 0.f;
            }
        }
        __syncthreads();  // (D)
        }

        // ---- U phase: dh[stripe col][row], split over k when there are few tiles
#pragma unroll 1
        for (int item = warp; item < C::MT_U * NT * C::KSPLIT; item += kWarps) {
            const int mt = item % C::MT_U;
            const int nt = (item / C::MT_U) % NT;
            const int kp = item / (C::MT_U * NT);
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int kk = 0; kk < C::KS_U / C::KSPLIT; ++kk) {
                const int ks = kp * (C::KS_U / C::KSPLIT) + kk;
                const int tile = (16 * ks) / C::KW;
                const int kin = (16 * ks) % C::KW;
                const int arow = 16 * mt + (lane & 7) + ((lane >> 3) & 1) * 8;
                const uint32_t off = uint32_t(arow) * (C::KW * 2) + kin * 2 + (lane >> 4) * 16;
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4(ubase + tile * C::U_TILE_BYTES + swz(off, C::UBITS), a0, a1, a2, a3);
                const __nv_bfloat16* bp = sb + (8 * nt + g) * C::SS + 16 * ks + 2 * t;
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bp);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(bp + 8);
                mma_bf16_16816(c, a0, a1, a2, a3, b0, b1);
            }
            float* o = dhp + (kp * C::MP + 8 * nt + 2 * t) * C::HS + 16 * mt + g;
            o[0] = c[0];
            o[C::HS] = c[1];
            o[8] = c[2];
            o[C::HS + 8] = c[3];
        }
        __syncthreads();  // (E) stage fully consumed, dh partials visible

        if (tid == 0 && l + S < p.L) issue_layer(l + S, st);

        // ---- h += dh ; partial sum of squares and bf16 copy for the next layer
        float* znext = zacc + size_t((l + 1) % 3) * C::MP * C::RP;
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
                    if (cg == 0 && row < M) {
                        if constexpr (CNT) {
                            const float rcur = rs_sh[(l + 1) & 1][row];          // this layer's 1/rms
                            const long long e = __double2ll_rn(double(ss) * double(rcur) * double(rcur) * kQScale);
                            red_add_u64(zs64 + (size_t((l + 1) % 3) * C::MP + row) * C::RP + R,
                                        static_cast<unsigned long long>(e - oldq[0]) + kOneArrival);
                            oldq[0] = oldq[1];
                            oldq[1] = oldq[2];
                            oldq[2] = e;
                        } else {
                            red_add_f32(znext + size_t(row) * C::RP + R, ss);
                        }
                    }
                } else if (row < M) {
                    *reinterpret_cast<uint2*>(p.y + size_t(row) * p.d + col0 + 4 * cg) = packed;
                }
            }
        }
    }

    if (err != 0) {
        // Give up: record why and where, then wait (bounded) for the copies
        // still in flight into this CTA's shared memory before leaving.
        if (tid == 0) {
            atomicCAS(p.status, 0, err | (l << 8));
            const int hi = (l + S < p.L) ? l + S : p.L;
            const int lo = (err == DLRB200_ERR_TIMEOUT_COPY || nothing_consumed) ? l : l + 1;
            for (int j = lo; j < hi; ++j) mbar_wait(smem_u32(&full[j % S]), (j / S) & 1, kDrainPolls);
        }
        __syncthreads();
    }
}

template <int R, int DC, int NT>
int launch_one(const DecodeLaunch& a) {
    using C = DecodeCfg<R, DC, NT>;
    auto kern = dlr_decode_kernel<R, DC, NT>;
    const int G = a.d / DC;
    // Ring depth: as many layers as fit; when the grid needs two CTAs per SM
    // each gets half of the shared memory.
    const int budget = (G > a.num_sms ? a.smem_optin / 2 - 2048 : a.smem_optin) - C::FIXED_BYTES;
    int stages = budget / C::STAGE_BYTES;
    if (stages > 32) stages = 32;
    if (stages > a.L) stages = a.L;
    if (a.max_stages > 0 && stages > a.max_stages) stages = a.max_stages;
    if (stages < 2 && a.L > 1) return DLRB200_ERR_UNSUPPORTED_SHAPE;
    if (stages < 1) stages = 1;
    const int smem = stages * C::STAGE_BYTES + C::FIXED_BYTES;
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (ce != cudaSuccess) return DLRB200_ERR_CUDA;
    int per_sm = 0;
    ce = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
    if (ce != cudaSuccess) return DLRB200_ERR_CUDA;
    if (per_sm * a.num_sms < G) return DLRB200_ERR_OCCUPANCY;

    DecodeParams p = a.p;
    p.stages = stages;
    CUtensorMap tmV = a.tmV, tmU = a.tmU;
    void* args[] = {&tmV, &tmU, &p};
    ce = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kern), dim3(G), dim3(kThreads), args, smem,
                                     a.stream);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

template <int R, int DC>
int launch_nt(const DecodeLaunch& a) {
    const int M = a.p.M;
    if (M <= 8) return launch_one<R, DC, 1>(a);
    if (M <= 16) return launch_one<R, DC, 2>(a);
    if (M <= 32) return launch_one<R, DC, 4>(a);
    return launch_one<R, DC, 8>(a);
}

template <int R>
int launch_dc(const DecodeLaunch& a) {
    switch (a.dc) {
        case 16: return launch_nt<R, 16>(a);
        case 32: return launch_nt<R, 32>(a);
        case 64: return launch_nt<R, 64>(a);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace

// three slots of 64 rows x (r + 4) fp32 words (or 32 rows of 64-bit words), then every CTA's sums of squares of
// the input: up to 160 CTAs (one per SM) x 32 rows
size_t decode_zacc_floats(int r) { return size_t(3) * 64 * (r + 4) + size_t(160) * 32; }

bool decode_box_dims(int r, int dc, int* v_box_cols, int* v_box_rows, int* u_box_cols, int* u_box_rows,
                     int* v_swizzle_bytes, int* u_swizzle_bytes) {
    if (!(r == 16 || r == 32 || r == 64 || r == 128 || r == 256)) return false;
    if (!(dc == 16 || dc == 32 || dc == 64)) return false;
    const int kw = r < 64 ? r : 64;
    *v_box_cols = dc; *v_box_rows = r;
    *u_box_cols = kw; *u_box_rows = dc;
    *v_swizzle_bytes = dc * 2;
    *u_swizzle_bytes = kw * 2;
    return true;
}

int decode_launch(const DecodeLaunch& a) {
    switch (a.r) {
        case 16: return launch_dc<16>(a);
        case 32: return launch_dc<32>(a);
        case 64: return launch_dc<64>(a);
        case 128: return launch_dc<128>(a);
        case 256: return launch_dc<256>(a);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace dlr
