// Large-batch ("prefill") DLR-Net forward, streamed path: one CTA (or a cluster
// of 2 or 4 that share the width) walks one 128-row tile of the batch through
// all L layers.  The activations stream chunk by chunk through a staging slot
// in shared memory and through tensor memory, in place in the output buffer;
// no cluster ever waits for another.
//
// Why.  Rows are independent (dlr_lock/model.py:96-100 acts on each token
// alone), so a CTA that owns whole rows needs no exchange.  A tile of 128 rows
// x d does not fit on chip, but it does not have to: the update of a layer is
// h[:, c] += s * U'[c, :]^T column chunk by column chunk, and the next layer's
// contraction z = h * V'^T can take a chunk as soon as it is updated.  The two
// contractions of neighbouring layers therefore run interleaved on the tensor
// core, and the only serial point per layer is the normalise + SiLU step.
//
// What bounds it.  With 128 rows per SM every weight byte is written to shared
// memory once (TMA) and read from it once (the MMA's B operand); at the tensor
// core's rate that alone is the whole 128 B/clk of the shared-memory port.  So
// as little else as possible goes through shared memory: both A operands (s
// and the updated chunk) are bf16 in tensor memory (tcgen05.mma with A in
// TMEM).  The activations do pass through a staging slot: the old values of a
// chunk come in by TMA, the epilogue threads update them in place, and a TMA
// store writes the slot back (a thread owns a row, so plain loads and stores
// would touch 32 cache lines per instruction, and an SM writes to L2 at only
// about 32 bytes per clock: threads that store themselves stall on it).
//
// Per chunk c of layer l (steady state), 128 rows x 128 columns, on one of two
// tensor-memory accumulators of 128 columns (one at rank 256, see SCfg):
//   producer warp   TMA loads of the old chunk, of U'[l] rows of the chunk and
//                   of V'[l+1] columns of the chunk into three rings
//   U-MMA warp      dh = s(l) * U'[l][chunk]^T  -> buffer (fp32)
//   epilogue warps  h_new = h_old + dh (fp32 add, rounded once to bf16), in
//                   place in the staging slot and, packed bf16, into tensor
//                   memory; running sum of squares per row
//   store warp      TMA store of the slot to the output buffer
//   V-MMA warp      z(l+1) += h_new[chunk] * V'[l+1][:, chunk]^T  (A = buffer)
// After the last chunk z(l+1) is complete; the epilogue warps turn it into
// s(l+1) = silu(z * rsqrt(sumsq / d + eps)), bf16, into tensor memory.
//
// Layer 0 is preceded by a pass that only feeds x to the V-MMA warp.  Passes
// 0 and -1 read x, every pass >= 0 writes y and every pass >= 1 reads y, so x
// is never modified.  A chunk stored in one pass is loaded again in the next:
// the store warp counts the chunks whose bulk store is complete, and the
// producer waits for that count before it asks for the chunk.
//
// Split.  When there are fewer tiles than SMs, a cluster of sp = 2 or 4 CTAs
// shares a tile: each takes d / 128 / sp chunks, and once per layer they add
// up their partial z and partial sums of squares (published in global memory,
// signalled with one remote mbarrier arrive per warp).
//
// All waits are bounded; a wait that gives up raises an abort flag, records a
// status word and every role drains and leaves.
#include <cstdlib>
#include <cstring>

#include "ptx.cuh"
#include "stream.h"

namespace dlr {

namespace {

constexpr int kRowsS = 128;              // rows per tile
constexpr int kCW = 128;                 // columns per chunk
constexpr int kThreadsS = 384;           // 12 warps: producer, U-MMA, V-MMA, store (owns tensor memory), 8 epilogue
constexpr int kEpiWarps = 8;
constexpr int kMaxW = 8;                 // most stages of a weight ring
constexpr int kMaxNH = 3;                // most staging slots for chunks of activations
constexpr int kHBytes = 2 * 16384;       // one chunk: two tiles of 128 rows x 64 columns (128-byte swizzle)
constexpr uint32_t kZCol = 0;            // tensor-memory columns: z accumulator (R columns)

// Tensor-memory columns and shared-memory stages per rank.  Up to rank 128 there is room for two dh
// accumulators and a separate A operand: z [0,128) | s [128,192) | A [192,256) | dh0 [256,384) | dh1 [384,512).
// Rank 256 fills the 512 columns with z [0,256) | s [256,384) | one buffer [384,512) that holds dh and then,
// in place, the bf16 chunk (columns 0-31 of the buffer: chunk columns 0-63, columns 64-95: chunk columns
// 64-127); U-MMA, epilogue and V-MMA of a chunk then run one after the other.
template <int R>
struct SCfg {
    static constexpr bool ONE_BUF = R == 256;
    static constexpr uint32_t S_COL = ONE_BUF ? 256 : 128;
    static constexpr uint32_t BUF_COL = ONE_BUF ? 384 : 256;
    static constexpr uint32_t A_COL = ONE_BUF ? 384 : 192;
    static constexpr int NH = ONE_BUF ? 2 : 3;           // staging slots for chunks of activations
    // a U' stage: 128 rows x up to 128 K-columns (tiles of 64); a chunk takes USPC stages
    static constexpr int USPC = R == 256 ? 2 : 1;
    static constexpr int UT = R / 64 / USPC;             // tiles per stage
    static constexpr int U_BYTES = UT * 16384;
    // a V' stage: tiles of R rows x 64 K-columns; a chunk (128 K-columns) takes VSPC stages
    static constexpr int VSPC = R == 256 ? 2 : 1;
    static constexpr int V_TILE_BYTES = R * 128;
    static constexpr int VT = 2 / VSPC;                  // tiles per stage
    static constexpr int V_BYTES = VT * V_TILE_BYTES;
    static constexpr int NU = R == 256 ? 3 : (R == 128 ? 2 : 4);   // stages of the U' ring
    static constexpr int NV = R == 256 ? 2 : (R == 128 ? 2 : 4);   // stages of the V' ring
    static constexpr int SMEM_BYTES = NH * kHBytes + NU * U_BYTES + NV * V_BYTES + 1024 /*sums of squares*/ + 512 /*barriers*/ +
                                      1024 /*alignment*/;
};

struct SBars {
    uint64_t u_full[kMaxW], u_empty[kMaxW];
    uint64_t v_full[kMaxW], v_empty[kMaxW];
    uint64_t h_full[kMaxNH];     // old chunk has landed (TMA bytes)
    uint64_t h_written[kMaxNH];  // the 8 epilogue warps have updated it in place
    uint64_t h_empty[kMaxNH];    // the store warp's bulk copy has read it
    uint64_t dh_full[2];      // U-MMA warp: dh of the chunk is in the buffer
    uint64_t dh_empty[2];     // 8 epilogue warps: dh has been read
    uint64_t a_ready;         // 8 epilogue warps: the updated chunk (bf16) is in tensor memory
    uint64_t a_empty;         // V-MMA warp: the chunk has been read
    uint64_t z_full, s_ready;
    uint64_t xchg_bar;        // sp > 1: the other CTAs of the cluster have published their partial z
    uint64_t ssq_bar;         // the 8 epilogue warps have published their halves of the sums of squares
    uint64_t drain[2];        // all tensor-core work of an MMA warp is complete (waited for before leaving)
    uint32_t tmem_slot;
    int abort_flag;
    unsigned int stored;      // chunks of this CTA (all tiles, all passes) whose bulk store is complete
};
static_assert(sizeof(SBars) <= 512, "barrier block");

struct SParams {
    const __nv_bfloat16* x;
    __nv_bfloat16* y;
    int M, d, L;
    int nch;                  // chunks per row: d / 128
    int sp;                   // CTAs (one cluster) that share a row tile, each with nch / sp of the chunks
    int num_tiles;
    uint4* xchg;              // sp > 1: per-layer exchange of the partial z between the CTAs of a cluster
    float eps, inv_d;
    int* status;
    unsigned int spin_limit;
    unsigned long long* prof; // optional cycle counters (debug), or null
};

#define DLS_CLK() (p.prof ? clock64() : 0ll)

// Non-blocking test of an mbarrier phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

template <int R>
__global__ void __launch_bounds__(kThreadsS, 1)
dlr_stream_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU, SParams p) {
    using C = SCfg<R>;
    constexpr uint32_t NU = C::NU, NV = C::NV, kNH = C::NH;
    constexpr uint32_t kSCol = C::S_COL, kACol = C::A_COL, kBufCol = C::BUF_COL;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* hbuf = smem;
    uint8_t* ubuf = hbuf + kNH * kHBytes;
    uint8_t* vbuf = ubuf + NU * C::U_BYTES;
    float* ssqx = reinterpret_cast<float*>(vbuf + NV * C::V_BYTES);   // [2 halves][128 rows]
    SBars* bars = reinterpret_cast<SBars*>(ssqx + 2 * kRowsS);
    volatile int* abort_flag = &bars->abort_flag;
    volatile unsigned int* stored = &bars->stored;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Waiter w{abort_flag, p.spin_limit >> 2};

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxW; ++s) {
            mbar_init(smem_u32(&bars->u_full[s]), 1);
            mbar_init(smem_u32(&bars->u_empty[s]), 1);
            mbar_init(smem_u32(&bars->v_full[s]), 1);
            mbar_init(smem_u32(&bars->v_empty[s]), 1);
        }
        for (int s = 0; s < kMaxNH; ++s) {
            mbar_init(smem_u32(&bars->h_full[s]), 1);
            mbar_init(smem_u32(&bars->h_written[s]), kEpiWarps);
            mbar_init(smem_u32(&bars->h_empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->dh_full[b]), 1);
            mbar_init(smem_u32(&bars->dh_empty[b]), kEpiWarps);
        }
        mbar_init(smem_u32(&bars->a_ready), kEpiWarps);
        mbar_init(smem_u32(&bars->a_empty), 1);
        mbar_init(smem_u32(&bars->z_full), 1);
        mbar_init(smem_u32(&bars->s_ready), kEpiWarps);
        mbar_init(smem_u32(&bars->ssq_bar), kEpiWarps);
        mbar_init(smem_u32(&bars->xchg_bar), kEpiWarps * (p.sp > 1 ? p.sp - 1 : 1));
        mbar_init(smem_u32(&bars->drain[0]), 1);
        mbar_init(smem_u32(&bars->drain[1]), 1);
        bars->abort_flag = 0;
        bars->stored = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tmX);
        tma_prefetch_desc(&tmY);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmU);
    }
    if (warp == 3) {
        tmem_alloc(smem_u32(&bars->tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    if (p.sp > 1) {            // the peers' barriers must exist before anyone signals them
        cluster_arrive_release();
        cluster_wait_acquire();
    }
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;
    const uint32_t hbuf_s = smem_u32(hbuf), ubuf_s = smem_u32(ubuf), vbuf_s = smem_u32(vbuf);
    const int sp = p.sp;
    const int rank = sp > 1 ? int(cluster_ctarank()) : 0;
    const int cl = int(blockIdx.x) / sp, ncl = int(gridDim.x) / sp;   // this cluster, clusters in the grid
    const int nch = p.nch / sp;                                      // chunks of this CTA
    const int col0 = rank * nch * kCW;                               // its first column
    const int my_tiles = (p.num_tiles - cl + ncl - 1) / ncl;

    int err = 0;
    int err_layer = 0;

    // A pass q = -1 .. L-1 walks the nch chunks once.  Pass q >= 0 applies the update of layer q; pass q < L-1
    // feeds the V contraction of layer q+1.  Chunk number n (all tiles, all passes) uses buffer n & 1.
    if (warp == 0) {
        // =============================== TMA producer ===============================
        // The two rings advance independently: whichever has a free stage gets its next tile.
        if (lane == 0) {
            RingPos up, vp, hp;
            int uph[kMaxW], vph[kMaxW], hph[kMaxNH];   // parity of the last copy requested into each stage, -1: none
            for (int i = 0; i < kMaxW; ++i) uph[i] = vph[i] = -1;
            for (int i = 0; i < kMaxNH; ++i) hph[i] = -1;
            const long long total_u = (long long)my_tiles * p.L * nch * C::USPC;   // stages of each weight stream
            const long long total_v = (long long)my_tiles * p.L * nch * C::VSPC;
            const long long total_h = (long long)my_tiles * (p.L + 1) * nch;  // chunks of activations
            long long nu = 0, nv = 0, nh = 0;
            int uq = 0, uc = 0, vq = 0, vc = 0, us = 0, vs = 0;   // layer, chunk, stage within the chunk
            int ht = 0, hq = -1, hc = 0;
            uint32_t idle = 0;
            while ((nu < total_u || nv < total_v || nh < total_h) && !err) {
                bool did = false;
                // pass >= 1 reads what this CTA stored one pass (nch chunks) earlier
                if (nh < total_h && (hq < 1 || *stored + unsigned(nch) > unsigned(nh)) &&
                    mbar_test_wait(smem_u32(&bars->h_empty[hp.st]), hp.ph ^ 1u)) {
                    if (hq >= 1) asm volatile("fence.proxy.async.global;" ::: "memory");
                    const uint32_t bar = smem_u32(&bars->h_full[hp.st]);
                    const uint32_t dst = hbuf_s + hp.st * kHBytes;
                    const CUtensorMap* src = hq >= 1 ? &tmY : &tmX;
                    const int m0 = (cl + ht * ncl) * kRowsS;
                    mbar_arrive_expect_tx(bar, kHBytes);
                    tma_load_2d(dst, src, col0 + hc * kCW, m0, bar);
                    tma_load_2d(dst + 16384, src, col0 + hc * kCW + 64, m0, bar);
                    hph[hp.st] = int(hp.ph);
                    hp.step(kNH);
                    ++nh;
                    if (++hc == nch) { hc = 0; if (++hq == p.L) { hq = -1; ++ht; } }
                    did = true;
                }
                if (nu < total_u && mbar_test_wait(smem_u32(&bars->u_empty[up.st]), up.ph ^ 1u)) {
                    const uint32_t bar = smem_u32(&bars->u_full[up.st]);
                    const uint32_t dst = ubuf_s + up.st * C::U_BYTES;
                    mbar_arrive_expect_tx(bar, C::U_BYTES);
#pragma unroll
                    for (int t = 0; t < C::UT; ++t)
                        tma_load_2d(dst + t * 16384, &tmU, 64 * (us * C::UT + t), uq * p.d + col0 + uc * kCW, bar);
                    uph[up.st] = int(up.ph);
                    up.step(NU);
                    ++nu;
                    if (++us == C::USPC) { us = 0; if (++uc == nch) { uc = 0; if (++uq == p.L) uq = 0; } }
                    did = true;
                }
                if (nv < total_v && mbar_test_wait(smem_u32(&bars->v_empty[vp.st]), vp.ph ^ 1u)) {
                    const uint32_t bar = smem_u32(&bars->v_full[vp.st]);
                    const uint32_t dst = vbuf_s + vp.st * C::V_BYTES;
                    mbar_arrive_expect_tx(bar, C::V_BYTES);
#pragma unroll
                    for (int t = 0; t < C::VT; ++t)
                        tma_load_2d(dst + t * C::V_TILE_BYTES, &tmV, col0 + vc * kCW + 64 * (vs * C::VT + t), vq * R, bar);
                    vph[vp.st] = int(vp.ph);
                    vp.step(NV);
                    ++nv;
                    if (++vs == C::VSPC) { vs = 0; if (++vc == nch) { vc = 0; if (++vq == p.L) vq = 0; } }
                    did = true;
                }
                if (did) {
                    idle = 0;
                } else if (++idle > p.spin_limit || ((idle & 63u) == 63u && *abort_flag)) {
                    err = DLRB200_ERR_TIMEOUT_COPY;
                    err_layer = uq;
                }
            }
            if (err || *abort_flag) {
                // copies requested before giving up still land in this CTA's shared memory: wait for them
                for (int i = 0; i < int(kNH); ++i)
                    if (hph[i] >= 0) mbar_wait(smem_u32(&bars->h_full[i]), uint32_t(hph[i]), kDrainPolls);
                for (int i = 0; i < int(NU); ++i)
                    if (uph[i] >= 0) mbar_wait(smem_u32(&bars->u_full[i]), uint32_t(uph[i]), kDrainPolls);
                for (int i = 0; i < int(NV); ++i)
                    if (vph[i] >= 0) mbar_wait(smem_u32(&bars->v_full[i]), uint32_t(vph[i]), kDrainPolls);
            }
        }
    } else if (warp == 1) {
        // =============================== U-MMA warp ================================
        // buffer = s(q)[128 x R] * U'[q][chunk rows, :]^T, A from tensor memory
        if (lane == 0) {
            constexpr uint32_t idesc_u = umma_idesc_bf16(128, kCW);
            RingPos up;
            uint32_t n = 0;
            uint32_t c_s = 0;
            long long mw[3] = {0, 0, 0};
            for (int t = 0; t < my_tiles && !err; ++t) {
                if (C::ONE_BUF) n += uint32_t(nch);          // the pass over x goes through the one buffer too
                for (int q = 0; q < p.L && !err; ++q) {
                    err_layer = q;
                    long long t0 = DLS_CLK();
                    if (!w.cta(smem_u32(&bars->s_ready), c_s & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ++c_s;
                    tc_fence_after();
                    mw[0] += DLS_CLK() - t0;
                    for (int c = 0; c < nch; ++c, ++n) {
                        const uint32_t b = C::ONE_BUF ? 0u : (n & 1u);
                        t0 = DLS_CLK();
                        // the accumulator is free: two of them, released by the epilogue once dh is read, or the one
                        // buffer, released by the V-MMA warp once the chunk before has been read as its A operand
                        if (C::ONE_BUF) {
                            if (!w.cta(smem_u32(&bars->a_empty), (n & 1u) ^ 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        } else {
                            if (!w.cta(smem_u32(&bars->dh_empty[b]), ((n >> 1) & 1u) ^ 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        }
                        mw[2] += DLS_CLK() - t0;
                        const uint32_t acc = tmem_base + kBufCol + b * 128u;
#pragma unroll
                        for (int su = 0; su < C::USPC; ++su) {
                            t0 = DLS_CLK();
                            if (!w.cta(smem_u32(&bars->u_full[up.st]), up.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                            mw[1] += DLS_CLK() - t0;
                            tc_fence_after();
                            const uint32_t ub = ubuf_s + up.st * C::U_BYTES;
                            constexpr int KS = R / 16 / C::USPC;      // K steps per stage
#pragma unroll
                            for (int k = 0; k < KS; ++k) {
                                const uint64_t bdesc = umma_desc(ub + uint32_t(k / 4) * 16384u, 2u, 1024u) + uint64_t(2 * (k % 4));
                                umma_ts(acc, tmem_base + kSCol + uint32_t(8 * (su * KS + k)), bdesc, idesc_u, (su | k) ? 1u : 0u);
                            }
                            umma_commit(smem_u32(&bars->u_empty[up.st]));
                            up.step(NU);
                        }
                        if (err) break;
                        umma_commit(smem_u32(&bars->dh_full[b]));
                    }
                }
            }
            umma_commit(smem_u32(&bars->drain[0]));
            mbar_wait(smem_u32(&bars->drain[0]), 0, kDrainPolls);
            if (p.prof) for (int k = 0; k < 3; ++k) p.prof[blockIdx.x * 32 + 4 + k] = (unsigned long long)mw[k];
        }
    } else if (warp == 2) {
        // =============================== V-MMA warp ================================
        // z(q+1)[128 x R] += h_new[chunk][128 x 128] * V'[q+1][:, chunk]^T, A = the updated chunk in tensor memory
        if (lane == 0) {
            constexpr uint32_t idesc_v = umma_idesc_bf16(128, R);
            RingPos vp;
            uint32_t n = 0;
            long long mw[2] = {0, 0};
            for (int t = 0; t < my_tiles && !err; ++t) {
                for (int q = -1; q < p.L && !err; ++q) {
                    err_layer = q;
                    const bool feeds = q + 1 < p.L;
                    for (int c = 0; c < nch; ++c, ++n) {
                        long long t0 = DLS_CLK();
                        if (!w.cta(smem_u32(&bars->a_ready), n & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        mw[0] += DLS_CLK() - t0;
                        if (feeds) {
                            const uint32_t a0 = tmem_base + kACol;
#pragma unroll
                            for (int sv = 0; sv < C::VSPC; ++sv) {
                                t0 = DLS_CLK();
                                if (!w.cta(smem_u32(&bars->v_full[vp.st]), vp.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                                mw[1] += DLS_CLK() - t0;
                                tc_fence_after();
                                const uint32_t vb = vbuf_s + vp.st * C::V_BYTES;
                                constexpr int KS = kCW / 16 / C::VSPC;    // K steps per stage
#pragma unroll
                                for (int kk = 0; kk < KS; ++kk) {
                                    const int k = sv * KS + kk;          // K step of the chunk: 16 columns
                                    const uint64_t bdesc = umma_desc(vb + uint32_t(kk / 4) * C::V_TILE_BYTES, 2u, 1024u) + uint64_t(2 * (kk % 4));
                                    // the chunk as A operand: 8 columns per K step, contiguous, or in two runs of
                                    // 32 columns where it shares the buffer with dh
                                    const uint32_t acol = C::ONE_BUF ? uint32_t(64 * (k / 4) + 8 * (k % 4)) : uint32_t(8 * k);
                                    umma_ts(tmem_base + kZCol, a0 + acol, bdesc, idesc_v, (c | k) ? 1u : 0u);
                                }
                                umma_commit(smem_u32(&bars->v_empty[vp.st]));
                                vp.step(NV);
                            }
                            if (err) break;
                            umma_commit(smem_u32(&bars->a_empty));
                        } else {
                            mbar_arrive(smem_u32(&bars->a_empty));   // last layer: nothing reads the chunk here
                        }
                    }
                    if (err) break;
                    if (feeds) umma_commit(smem_u32(&bars->z_full));
                }
            }
            umma_commit(smem_u32(&bars->drain[1]));
            mbar_wait(smem_u32(&bars->drain[1]), 0, kDrainPolls);
            if (p.prof) for (int k = 0; k < 2; ++k) p.prof[blockIdx.x * 32 + 8 + k] = (unsigned long long)mw[k];
        }
    } else if (warp == 3) {
        // =============================== store warp ================================
        // updated chunk -> output buffer.  The slot is released when the copy has read it; the chunk counts as
        // stored (readable by the next pass) once its bulk group is complete, which is checked two chunks late
        // so that this warp never waits for a write in flight.
        if (lane == 0) {
            RingPos hp;
            unsigned int n = 0;              // chunks seen (all tiles, all passes): the producer counts the same way
            for (int t = 0; t < my_tiles && !err; ++t) {
                const int m0 = (cl + t * ncl) * kRowsS;
                for (int q = -1; q < p.L && !err; ++q) {
                    err_layer = q;
                    for (int c = 0; c < nch; ++c, ++n) {
                        if (!w.cta(smem_u32(&bars->h_written[hp.st]), hp.ph)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        if (q >= 0) {
                            const uint32_t src = hbuf_s + hp.st * kHBytes;
                            tma_store_2d(&tmY, col0 + c * kCW, m0, src);
                            tma_store_2d(&tmY, col0 + c * kCW + 64, m0, src + 16384);
                            bulk_commit_group();
                            bulk_wait_group_read<0>();
                            bulk_wait_group<2>();            // every group but the last two is complete
                            if (n + 1u > *stored + 2u) *stored = n + 1u - 2u;
                        } else {
                            // the pass over x stores nothing; also the point where the tile before is fully stored
                            bulk_wait_group<0>();
                            *stored = n + 1u;
                        }
                        mbar_arrive(smem_u32(&bars->h_empty[hp.st]));
                        hp.step(kNH);
                    }
                }
            }
            bulk_wait_group<0>();
        }
    } else if (warp >= 4) {
        // =============================== epilogue warps =============================
        // Two threads per row: thread (row er, half hh) owns 64 of the 128 columns of every chunk and half of
        // the columns of z.  Warp w reads tensor-memory lanes 32 * (w % 4) .. + 31.
        const int q4 = warp & 3;
        const int hh = (warp - 4) >> 2;
        const int er = 32 * q4 + lane;
        const uint32_t tl = tmem_base + (uint32_t(32 * q4) << 16);
        uint32_t n = 0;                      // chunks seen (all passes): phase of the A operand's barriers
        uint32_t nu = 0;                     // chunks of update passes: accumulator nu & 1
        uint32_t c_z = 0;
        long long ew[12] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};

        RingPos hp;
        const uint32_t x7 = uint32_t(er & 7);
        for (int t = 0; t < my_tiles && !err; ++t) {
            float ssq = 0.f;
            for (int q = -1; q < p.L && !err; ++q) {
                err_layer = q;
                for (int c = 0; c < nch; ++c, ++n) {
                    const uint32_t b = C::ONE_BUF ? 0u : (nu & 1u);
                    const uint32_t buf = tl + kBufCol + b * 128u + uint32_t(64 * hh);
                    // ---- old values of the chunk: this thread's 128 bytes of its row, from the staging slot
                    long long t0 = DLS_CLK();
                    if (!w.cta(smem_u32(&bars->h_full[hp.st]), hp.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                    ew[4] += DLS_CLK() - t0;
                    uint32_t cur[32];
                    {
                        const uint8_t* rowp = hbuf + hp.st * kHBytes + hh * 16384 + er * 128;
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch) {
                            const uint4 hv = *reinterpret_cast<const uint4*>(rowp + ((uint32_t(ch) ^ x7) << 4));
                            cur[4 * ch] = hv.x; cur[4 * ch + 1] = hv.y; cur[4 * ch + 2] = hv.z; cur[4 * ch + 3] = hv.w;
                        }
                    }
                    uint32_t out[32];
                    t0 = DLS_CLK();
                    if (q >= 0) {
                        if (!w.cta(smem_u32(&bars->dh_full[b]), (C::ONE_BUF ? nu : (nu >> 1)) & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        ++nu;
                        ew[1] += DLS_CLK() - t0;
                        tc_fence_after();
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            uint32_t dv[32];
                            tmem_ld32(buf + uint32_t(32 * g), dv);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const uint32_t hw = cur[16 * g + j];
                                const float f0 = bf16lo_to_f(hw) + __uint_as_float(dv[2 * j]);
                                const float f1 = bf16hi_to_f(hw) + __uint_as_float(dv[2 * j + 1]);
                                ssq = fmaf(f0, f0, ssq);
                                ssq = fmaf(f1, f1, ssq);
                                out[16 * g + j] = pack_bf16x2(f0, f1);
                            }
                        }
                        if (!C::ONE_BUF) {
                            // dh has been read: the U-MMA warp may overwrite the accumulator
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(smem_u32(&bars->dh_empty[b]));
                        }
                        ew[0] += DLS_CLK() - t0;
                    } else {
                        // pass over x: the chunk goes to the tensor core as it is
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float f0 = bf16lo_to_f(cur[j]), f1 = bf16hi_to_f(cur[j]);
                            ssq = fmaf(f0, f0, ssq);
                            ssq = fmaf(f1, f1, ssq);
                            out[j] = cur[j];
                        }
                    }
                    // ---- new values back into the staging slot, in place: the store warp copies the slot out
                    const long long t3 = DLS_CLK();
                    if (q >= 0) {
                        uint8_t* rowp = hbuf + hp.st * kHBytes + hh * 16384 + er * 128;
#pragma unroll
                        for (int ch = 0; ch < 8; ++ch)
                            *reinterpret_cast<uint4*>(rowp + ((uint32_t(ch) ^ x7) << 4)) =
                                make_uint4(out[4 * ch], out[4 * ch + 1], out[4 * ch + 2], out[4 * ch + 3]);
                        fence_async_smem();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->h_written[hp.st]));
                    ew[7] += DLS_CLK() - t3;
                    // ---- the chunk (bf16) becomes the A operand of the next layer's contraction
                    const long long t2 = DLS_CLK();
                    if (!w.cta(smem_u32(&bars->a_empty), (n & 1u) ^ 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ew[5] += DLS_CLK() - t2;
                    tc_fence_after();
                    constexpr uint32_t a_half = C::ONE_BUF ? 64u : 32u;   // in the shared buffer each thread writes over its own dh columns
                    tmem_st16(tl + kACol + a_half * uint32_t(hh), *reinterpret_cast<uint32_t(*)[16]>(&out[0]));
                    tmem_st16(tl + kACol + a_half * uint32_t(hh) + 16u, *reinterpret_cast<uint32_t(*)[16]>(&out[16]));
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->a_ready));
                    hp.step(kNH);
                    ew[6] += DLS_CLK() - t2;
                }
                if (err) break;
                if (q + 1 < p.L) {
                    // ---- z(q+1) is complete after the V-MMA warp's last chunk: s = silu(z * rstd) -> tensor memory
                    const long long t0 = DLS_CLK();
                    constexpr int NZ = R / 2;            // columns of z per thread, handled 32 at a time
                    constexpr int NQ = NZ / 8 + 1;       // 16-byte words a thread publishes: z as bf16 pairs, then its sum of squares
                    if (!w.cta(smem_u32(&bars->z_full), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    tc_fence_after();
                    const long long tb1 = DLS_CLK();
                    ew[8] += tb1 - t0;
                    const int et = int(threadIdx.x) - 128;
                    if (sp > 1) {
                        // Every CTA of the cluster holds the partial z of its own columns.  Each publishes its
                        // partial (rounded to bf16) and its partial sums of squares in global memory, signals the
                        // others, and adds up all sp partials in rank order, its own rounded like the rest, so that
                        // every CTA arrives at the same s.  Slots alternate with the layer's parity: a CTA can be at
                        // most one layer ahead of a peer that still reads.
                        uint4* mine = p.xchg + ((size_t(cl) * 2 + (c_z & 1u)) * sp + rank) * (NQ * 256) + et;
#pragma unroll
                        for (int g = 0; g < NZ / 32; ++g) {
                            uint32_t zv[32];
                            tmem_ld32(tl + kZCol + uint32_t(hh * NZ + 32 * g), zv);
                            tmem_wait_ld();
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float* f = reinterpret_cast<const float*>(&zv[8 * k]);
                                mine[(4 * g + k) * 256] = make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]),
                                                                     pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
                            }
                        }
                        mine[(NQ - 1) * 256] = make_uint4(__float_as_uint(ssq), 0u, 0u, 0u);
                        // the arrive below releases these stores at cluster scope and the peers' wait acquires them
                        __syncwarp();
                        if (lane == 0)
                            for (int o = 1; o < sp; ++o)
                                mbar_arrive_remote(mapa(smem_u32(&bars->xchg_bar), uint32_t((rank + o) % sp)));
                        const long long tb2 = DLS_CLK();
                        ew[9] += tb2 - tb1;
                        if (!w.cluster(smem_u32(&bars->xchg_bar), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        ew[10] += DLS_CLK() - tb2;
                        float qs = 0.f;
                        for (int o = 0; o < sp; ++o)
                            qs += __uint_as_float(__ldcg(p.xchg + ((size_t(cl) * 2 + (c_z & 1u)) * sp + o) * (NQ * 256) + et + (NQ - 1) * 256).x);
                        ssq = qs;
                    }
                    const long long tb3 = DLS_CLK();
                    ssqx[hh * kRowsS + er] = ssq;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->ssq_bar));
                    if (!w.cta(smem_u32(&bars->ssq_bar), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    ew[11] += DLS_CLK() - tb3;
                    const float tot = ssq + ssqx[(hh ^ 1) * kRowsS + er];
                    const float rstd = rsqrtf(tot * p.inv_d + p.eps);
                    ssq = 0.f;
                    ew[2] += DLS_CLK() - t0;
#pragma unroll
                    for (int g = 0; g < NZ / 32; ++g) {
                        float zf[32];
                        if (sp > 1) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) zf[j] = 0.f;
                            for (int o = 0; o < sp; ++o) {
                                const uint4* src = p.xchg + ((size_t(cl) * 2 + (c_z & 1u)) * sp + o) * (NQ * 256) + et;
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    const uint4 v = __ldcg(src + (4 * g + k) * 256);
                                    zf[8 * k] += bf16lo_to_f(v.x); zf[8 * k + 1] += bf16hi_to_f(v.x);
                                    zf[8 * k + 2] += bf16lo_to_f(v.y); zf[8 * k + 3] += bf16hi_to_f(v.y);
                                    zf[8 * k + 4] += bf16lo_to_f(v.z); zf[8 * k + 5] += bf16hi_to_f(v.z);
                                    zf[8 * k + 6] += bf16lo_to_f(v.w); zf[8 * k + 7] += bf16hi_to_f(v.w);
                                }
                            }
                        } else {
                            uint32_t zv[32];
                            tmem_ld32(tl + kZCol + uint32_t(hh * NZ + 32 * g), zv);
                            tmem_wait_ld();
#pragma unroll
                            for (int j = 0; j < 32; ++j) zf[j] = __uint_as_float(zv[j]);
                        }
                        uint32_t sv[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            sv[j] = pack_bf16x2(silu_tanh_f(zf[2 * j] * rstd), silu_tanh_f(zf[2 * j + 1] * rstd));
                        tmem_st16(tl + kSCol + uint32_t(hh * (NZ / 2) + 16 * g), sv);
                    }
                    ++c_z;
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->s_ready));
                    ew[3] += DLS_CLK() - t0;
                }
            }
        }
        if (p.prof && threadIdx.x == 128)
            for (int k = 0; k < 12; ++k) p.prof[blockIdx.x * 32 + 12 + k] = (unsigned long long)ew[k];
    }

    // ---- leave: report, let every role arrive, free tensor memory
    if (err) {
        if (!*abort_flag) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, err | ((err_layer & 0xffff) << 8));
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 3) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
    if (sp > 1) {              // no CTA may leave while a peer can still signal its barrier
        cluster_arrive_release();
        cluster_wait_acquire();
    }
}

constexpr size_t kXchgOffset = 65536;    // the exchange slots start here in the workspace (profiling counters come first)
constexpr size_t kXchgBytesPerCta = 2 * (256 / 16 + 1) * 256 * 16;   // two parities x 17 words x 256 threads at rank 256

// CTAs that share a row tile: as many as keep every tile resident at once, so that small batches still
// spread over the whole GPU.  Each CTA needs at least four chunks.
int pick_split(int num_tiles, int nch, int num_sms) {
    int forced = 0;
    if (const char* e = getenv("DLRB200_STREAM_SPLIT")) forced = atoi(e);
    for (int sp = 4; sp >= 2; sp >>= 1) {
        if (forced && forced != sp) continue;
        if (nch % sp == 0 && nch / sp >= 4 && num_tiles * sp <= num_sms - num_sms % sp) return sp;
    }
    return 1;
}

template <int R>
int launch_stream(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int L, float eps,
                  void* workspace, int* status_dev, cudaStream_t stream, int num_sms, int smem_optin,
                  unsigned int spin_limit, dlrb200_plan* plan_only, unsigned long long* prof) {
    using C = SCfg<R>;
    if (C::SMEM_BYTES > smem_optin) return DLRB200_ERR_OCCUPANCY;
    const int num_tiles = (M + kRowsS - 1) / kRowsS;
    int sp = pick_split(num_tiles, d / kCW, num_sms);
    auto kern = dlr_stream_kernel<R>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
        return DLRB200_ERR_CUDA;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    cfg.blockDim = dim3(kThreadsS);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    int clusters = num_tiles < num_sms ? num_tiles : num_sms;
    while (sp > 1) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = sp;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        cfg.gridDim = dim3(sp * (num_sms / sp));
        int max_clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) return DLRB200_ERR_CUDA;
        if (max_clusters >= num_tiles) { clusters = num_tiles; break; }
        sp >>= 1;                       // not all tiles resident at this split: use a smaller one
    }
    if (sp == 1) {
        cfg.attrs = nullptr;
        cfg.numAttrs = 0;
        clusters = num_tiles < num_sms ? num_tiles : num_sms;
    }
    const int grid = clusters * sp;
    cfg.gridDim = dim3(grid);
    if (plan_only) {
        plan_only->path = DLRB200_PATH_STREAMED;
        plan_only->grid = grid;
        plan_only->cluster = sp;
        plan_only->stripe_cols = kCW;
        plan_only->rows_per_pass = kRowsS;
        plan_only->passes = (num_tiles + clusters - 1) / clusters;
        plan_only->stages = C::NU + C::NV;
        plan_only->smem_bytes = size_t(C::SMEM_BYTES);
        return DLRB200_OK;
    }
    CUtensorMap tmX, tmY, tmV, tmU;
    if (!encode_2d_bf16(enc, &tmX, x, uint64_t(d), uint64_t(M), 64, kRowsS, 128) ||
        !encode_2d_bf16(enc, &tmY, y, uint64_t(d), uint64_t(M), 64, kRowsS, 128) ||
        !encode_2d_bf16(enc, &tmV, Vp, uint64_t(d), uint64_t(L) * R, 64, R, 128) ||
        !encode_2d_bf16(enc, &tmU, Up, uint64_t(R), uint64_t(L) * d, 64, 128, 128))
        return DLRB200_ERR_CUDA;
    SParams p;
    p.x = static_cast<const __nv_bfloat16*>(x);
    p.y = static_cast<__nv_bfloat16*>(y);
    p.M = M; p.d = d; p.L = L;
    p.nch = d / kCW;
    p.sp = sp;
    p.num_tiles = num_tiles;
    p.xchg = reinterpret_cast<uint4*>(static_cast<uint8_t*>(workspace) + kXchgOffset);
    p.eps = eps;
    p.inv_d = 1.0f / float(d);
    p.status = status_dev;
    p.spin_limit = spin_limit;
    p.prof = prof;
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, tmX, tmY, tmV, tmU, p);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

int dispatch_stream(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L,
                    float eps, void* workspace, int* status_dev, cudaStream_t stream, int num_sms, int smem_optin,
                    unsigned int spin_limit, dlrb200_plan* plan_only, unsigned long long* prof) {
    switch (r) {
        case 64: return launch_stream<64>(enc, x, y, Vp, Up, M, d, L, eps, workspace, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only, prof);
        case 128: return launch_stream<128>(enc, x, y, Vp, Up, M, d, L, eps, workspace, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only, prof);
        case 256: return launch_stream<256>(enc, x, y, Vp, Up, M, d, L, eps, workspace, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only, prof);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace

// The store warp reports a chunk as stored two chunks late, and the producer runs up to three chunks ahead of
// the epilogue: a CTA needs at least four chunks per pass for the next pass's first loads to be released.
bool stream_supported(int d, int r) { return (r == 64 || r == 128 || r == 256) && d % kCW == 0 && d >= 4 * kCW; }

// The activations move by TMA: 16-byte aligned bases (rows are d * 2 bytes, a multiple of 256).
bool stream_aligned(const void* x, const void* y) {
    return (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
}

int stream_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan) {
    const size_t ws = plan->workspace_bytes;
    const int rc = dispatch_stream(nullptr, nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, nullptr, num_sms,
                                   smem_optin, 0, plan, nullptr);
    plan->workspace_bytes = ws;
    return rc;
}

size_t stream_workspace_bytes(int M, int d, int r) {
    if (M <= 64 || !stream_supported(d, r)) return 0;
    return kXchgOffset + 160 * kXchgBytesPerCta;    // one slot set per CTA, at most one CTA per SM
}

int stream_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                   int L, float eps, void* workspace, int* status_dev, cudaStream_t stream, int num_sms, int smem_optin,
                   unsigned int spin_limit, unsigned long long* prof) {
    if (num_sms > 160) return DLRB200_ERR_OCCUPANCY;
    return dispatch_stream(encode_fn_ptr, x, y, Vp, Up, M, d, r, L, eps, workspace, status_dev, stream, num_sms, smem_optin,
                           spin_limit, nullptr, prof);
}

}  // namespace dlr
