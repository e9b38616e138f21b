// Large-batch ("prefill") DLR-Net forward, streamed path on CTA pairs: two CTAs
// walk one 256-row tile of the batch through all L layers with tensor-core
// instructions of M = 256 (tcgen05 cta_group::2); a cluster holds one pair, or
// two or four pairs that split the width.
//
// Same data flow as the one-CTA streamed kernel (stream.cu): rows are
// independent (dlr_lock/model.py:96-100 acts on each token alone), the
// activations stream chunk by chunk (128 columns) through a staging slot in
// shared memory and through tensor memory, in place in the output buffer, and
// the two contractions of neighbouring layers run interleaved,
//     dh        = s(l) * U'[l][chunk]^T          (U-MMA)
//     h[chunk] += dh                             (epilogue threads)
//     z(l+1)   += h[chunk] * V'[l+1][:, chunk]^T (V-MMA)
// with s(l+1) = silu(z(l+1) * rstd) once per layer.
//
// Why pairs.  The one-CTA kernel is bound by the shared-memory port of its SM:
// per chunk 64 KB of weights are written by TMA and read by the tensor core,
// and 32 KB of activations pass four times (TMA in, read, write, TMA out):
// 256 KB at 128 bytes per clock is twice the tensor core's own time.  In a
// pair each CTA keeps its own 128 rows (A operands and accumulators in its own
// tensor memory) but supplies only HALF of every weight tile: the instruction
// reads the other half from the partner's shared memory.  Weight bytes through
// each SM's port halve; nothing is multicast, each CTA loads its own half with
// a plain TMA load whose bytes are counted on the leader's barrier.
//
// Roles per CTA (640 threads): TMA producer, U-MMA issuer and V-MMA issuer
// (these two work in the leader, the even-ranked CTA of the pair, only), store
// warp (owns tensor memory), 16 epilogue warps.  The epilogue warps of the
// second CTA signal the leader's barriers with remote arrives; the leader's
// tcgen05.commit signals the barriers of both CTAs.
//
// Two or four pairs per cluster (when there are too few 256-row tiles to fill
// the GPU) split the width: pair i takes the i-th part of the chunks; once per
// layer the CTAs that hold the same rows add up their partial z and partial
// sums of squares in one or two exchange steps (partner: pair i ^ 1, then pair
// i ^ 2).  A step sends the running sum (rounded to bf16) straight into the
// partner's shared memory with st.async (bytes counted on the receiver's
// barrier: no fences, no trip through global memory), and both sides add own
// (rounded alike) + received: every CTA ends with the same bits.
//
// All waits are bounded; a wait that gives up raises an abort flag, records a
// status word and every role drains and leaves.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "ptx.cuh"
#include "stream_pair.h"

namespace dlr {

namespace {

constexpr int kRowsP = 128;              // rows per CTA (a pair: 256)
constexpr int kCWP = 128;                // columns per chunk
constexpr int kEpiWarpsP = 16;           // four threads per row: each owns 32 of a chunk's 128 columns
constexpr int kEpiThreadsP = kEpiWarpsP * 32;
constexpr int kThreadsP = 128 + kEpiThreadsP;   // 20 warps: producer, U-MMA, V-MMA, store (owns tensor memory), 16 epilogue
constexpr int kMaxWP = 4;                // most stages of a weight ring
constexpr int kNLP = 2;                  // slots the old values of a chunk are loaded into
constexpr int kNSP = 2;                  // slots the new values are written to and stored from
constexpr int kHBytesP = 2 * 16384;      // one chunk: two tiles of 128 rows x 64 columns (128-byte swizzle)

// Tensor-memory columns (per CTA): z [0, R) | s [128, 128 + R/2) | buffer 0 [256, 384) | buffer 1 [384, 512).
// A buffer first holds dh of a chunk (fp32, 128 columns); the epilogue thread that has read its 32 columns of
// dh writes its 32 updated values back as bf16 over the first 16 of them, and the V contraction reads the
// chunk from there (K step k: columns 32 (k / 2) + 8 (k % 2)).  The chunk therefore needs no buffer of its
// own, two chunks are in flight, and the epilogue never waits for the V contraction of the chunk before.
template <int R>
struct PCfg {
    static constexpr uint32_t Z_COL = 0, S_COL = 128, BUF_COL = 256;
    // this CTA's half of a chunk's U' rows: 64 rows x R K-columns, in tiles of 64 K-columns
    static constexpr int UT = R / 64;
    static constexpr int U_TILE_BYTES = 64 * 128;
    static constexpr int U_BYTES = UT * U_TILE_BYTES;
    // this CTA's half of V'[l]: R/2 rows x the chunk's 128 K-columns, in two tiles of 64 K-columns
    static constexpr int V_TILE_BYTES = (R / 2) * 128;
    static constexpr int V_BYTES = 2 * V_TILE_BYTES;
    static constexpr int NU = R == 128 ? 2 : 4;
    static constexpr int NV = R == 128 ? 2 : 4;
    // message of one thread to a partner pair: its R/4 columns of z as bf16 (NZW words of 16 bytes) and its
    // partial sum of squares (4 bytes)
    static constexpr int NZ = R / 4;
    static constexpr int NZW = NZ / 8;
    static constexpr int RECV_Z_BYTES = NZW * kEpiThreadsP * 16;
    static constexpr int RECV_BYTES = RECV_Z_BYTES + kEpiThreadsP * 4;
    // the partial sums of squares of this CTA are added in place onto the received ones: no array of their own
    static constexpr int SMEM_BYTES = (kNLP + kNSP) * kHBytesP + NU * U_BYTES + NV * V_BYTES + RECV_BYTES + 512 /*barriers*/;
};

struct PBars {
    uint64_t u_full[kMaxWP], u_empty[kMaxWP];   // full: in the leader, bytes of both CTAs; empty: commit, both CTAs
    uint64_t v_full[kMaxWP], v_empty[kMaxWP];
    uint64_t l_free[kNLP];       // the 16 epilogue warps have it in registers
    uint64_t s_written[kNSP];    // the 16 epilogue warps have written the new chunk
    // The one barrier an epilogue thread waits for per chunk (a look at an mbarrier costs a few hundred cycles even
    // when its phase is complete, and the epilogue is on the loop that bounds the time per chunk).  Chunk n uses
    // buffer, load slot and store slot n & 1, and barrier [n & 1] collects three arrivals: the commit of the U
    // contraction (both CTAs; in the pass over x an empty commit once the buffer is free), the producer's arrival
    // that carries the byte count of the old values, and the store warp's arrival when the bulk store of the chunk
    // two before has read the store slot.
    uint64_t dh_full[2];
    uint64_t a_ready[2];         // leader: the 32 epilogue warps have put the updated chunk (bf16) into the buffer
    uint64_t a_free[2];          // commit, both CTAs: the V contraction has read the chunk, the buffer is free
    uint64_t z_full;             // commit, both CTAs
    uint64_t s_ready;            // leader: 32 epilogue warps
    uint64_t xchg_bar[2];        // per exchange step: the partner's message has arrived (bytes)
    uint64_t xack_bar[2];        // per exchange step: the 16 epilogue warps of that step's partner have read their receive
                                 // buffer, this CTA may send its next message of that step
    uint64_t ssq_bar;            // the 16 epilogue warps have published their quarters of the sums of squares
    uint64_t drain[2];           // all tensor-core work of an MMA warp is complete (waited for before leaving)
    uint32_t tmem_slot;
    int abort_flag;
    unsigned int stored;         // chunks of this CTA (all tiles, all passes) whose bulk store is complete
};
static_assert(sizeof(PBars) <= 512, "barrier block");

struct PParams {
    int M, d, L;
    int nch;                  // chunks per row: d / 128
    int pp;                   // pairs per cluster (1, 2 or 4), each with nch / pp of the chunks
    int num_tiles;            // 256-row tiles
    float eps, inv_d;
    int* status;
    unsigned int spin_limit;
    unsigned long long* prof; // time stamps (profiling instantiation), or null
    int trace_layer;
    int exp;                  // profiling instantiation only: bits that leave out one piece of work each (timing experiments)
};

// Time stamps of one layer of the first pair of the grid, written only by the profiling instantiation:
// prof[(CTA * 8 + role) * 256 + chunk * 8 + event] = clock64().  Roles: 0-2 producer (activations, U', V'),
// 3 U-MMA, 4 V-MMA, 5 store, 6 and 7 the first and the last epilogue warp.
#define DLP_T(role, layer, chunk, event)                                                                   \
    do {                                                                                                   \
        if (PROF && blockIdx.x < 2 && (layer) == p.trace_layer && (chunk) < 32)                            \
            p.prof[((blockIdx.x * 8 + (role)) * 32 + (chunk)) * 8 + (event)] = (unsigned long long)clock64(); \
    } while (0)

template <int R, bool PROF>
__global__ void __launch_bounds__(kThreadsP, 1)
dlr_stream_pair_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmY,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmU, PParams p) {
    using C = PCfg<R>;
    constexpr uint32_t NU = C::NU, NV = C::NV;
    constexpr uint32_t kZCol = C::Z_COL, kSCol = C::S_COL, kBufCol = C::BUF_COL;
    // the swizzled tiles need a 1024-byte aligned base: asked for here, checked below
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* lbuf = smem;
    uint8_t* sbuf = lbuf + kNLP * kHBytesP;
    uint8_t* ubuf = sbuf + kNSP * kHBytesP;
    uint8_t* vbuf = ubuf + NU * C::U_BYTES;
    uint4* recv = reinterpret_cast<uint4*>(vbuf + NV * C::V_BYTES);                 // [NZW][512 threads]
    float* recv_q = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(recv) + C::RECV_Z_BYTES);   // [512 threads]
    float* ssqx = recv_q;                                                           // [4 column quarters][128 rows], same words
    PBars* bars = reinterpret_cast<PBars*>(recv_q + kEpiThreadsP);
    volatile int* abort_flag = &bars->abort_flag;
    volatile unsigned int* stored = &bars->stored;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const Waiter w{abort_flag, p.spin_limit >> 2};

    const int pp = p.pp;
    const uint32_t crank = cluster_ctarank();
    const int hf = int(crank & 1u);                 // 0: leader of the pair
    const int pi = int(crank >> 1);                 // pair within the cluster
    const uint32_t lead = crank & ~1u;              // cluster rank of this pair's leader
    const int nsteps = pp == 4 ? 2 : (pp == 2 ? 1 : 0);   // exchange steps per layer; step s: partner = pair pi ^ (1 << s)
    const uint16_t pair_mask = uint16_t(3u << lead);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxWP; ++s) {
            mbar_init(smem_u32(&bars->u_full[s]), 1);
            mbar_init(smem_u32(&bars->u_empty[s]), 1);
            mbar_init(smem_u32(&bars->v_full[s]), 1);
            mbar_init(smem_u32(&bars->v_empty[s]), 1);
        }
        for (int s = 0; s < kNLP; ++s) {
            mbar_init(smem_u32(&bars->l_free[s]), kEpiWarpsP);
        }
        for (int s = 0; s < kNSP; ++s) {
            mbar_init(smem_u32(&bars->s_written[s]), kEpiWarpsP);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->dh_full[b]), 3);
            mbar_init(smem_u32(&bars->a_ready[b]), 2 * kEpiWarpsP);
            mbar_init(smem_u32(&bars->a_free[b]), 1);
        }
        mbar_init(smem_u32(&bars->z_full), 1);
        mbar_init(smem_u32(&bars->s_ready), 2 * kEpiWarpsP);
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bars->xchg_bar[b]), 1);
            mbar_init(smem_u32(&bars->xack_bar[b]), kEpiWarpsP);
        }
        mbar_init(smem_u32(&bars->ssq_bar), kEpiWarpsP);
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
    __syncthreads();
    // the other CTAs' barriers must exist before anyone signals them, and both CTAs of a pair must be running
    // before tensor memory is allocated for the pair
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == 3) {
        tmem_alloc2(smem_u32(&bars->tmem_slot), 512);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_slot;
    const uint32_t lbuf_s = smem_u32(lbuf), sbuf_s = smem_u32(sbuf), ubuf_s = smem_u32(ubuf), vbuf_s = smem_u32(vbuf);
    const int cl = int(blockIdx.x) / (2 * pp), ncl = int(gridDim.x) / (2 * pp);   // this cluster, clusters in the grid
    const int nch = p.nch / pp;                                      // chunks of this pair
    const int col0 = pi * nch * kCWP;                                // its first column
    const int my_tiles = (p.num_tiles - cl + ncl - 1) / ncl;

    int err = (smem_u32(smem) & 1023u) ? DLRB200_ERR_ALIGNMENT : 0;   // every role skips its loops
    int err_layer = 0;

    // A pass q = -1 .. L-1 walks the nch chunks once.  Pass q >= 0 applies the update of layer q; pass q < L-1
    // feeds the V contraction of layer q+1.  Chunk number n (all tiles, all passes) uses buffer n & 1.
    if (warp == 0) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            RingPos up, vp, hp;
            int uph[kMaxWP], vph[kMaxWP], hph[kNLP];   // parity of the last copy requested into each stage, -1: none
            for (int i = 0; i < kMaxWP; ++i) uph[i] = vph[i] = -1;
            for (int i = 0; i < kNLP; ++i) hph[i] = -1;
            const long long total_w = (long long)my_tiles * p.L * nch;        // stages of each weight stream
            const long long total_h = (long long)my_tiles * (p.L + 1) * nch;  // chunks of activations
            long long nu = 0, nv = 0, nh = 0;
            int uq = 0, uc = 0, vq = 0, vc = 0;
            int ht = 0, hq = -1, hc = 0;
            uint32_t idle = 0;
            // the weight stages of both CTAs are counted on the leader's barriers
            const uint32_t ufull_lead = mapa(smem_u32(&bars->u_full[0]), lead);
            const uint32_t vfull_lead = mapa(smem_u32(&bars->v_full[0]), lead);
            // the weights pass through L2 once per cluster and layer, the activations come back every layer: tell
            // L2 which to keep (without the hints over half of every layer's output is written back to DRAM)
            const uint64_t pol_w = l2_policy_evict_first(), pol_h = l2_policy_evict_last();
            const bool hints = !(PROF && (p.exp & 32));
            while ((nu < total_w || nv < total_w || nh < total_h) && !err) {
                bool did = false;
                // The epilogue threads wait for one barrier per chunk (a look at an mbarrier costs them a few hundred
                // cycles): the bytes of the old values are counted on the chunk's own barrier (slot n & 1 = buffer n & 1).
                // pass >= 1 reads what this CTA stored one pass (nch chunks) earlier
                if (nh < total_h && (hq < 1 || *stored + unsigned(nch) > unsigned(nh)) &&
                    mbar_test(smem_u32(&bars->l_free[hp.st]), hp.ph ^ 1u)) {
                    if (hq >= 1) asm volatile("fence.proxy.async.global;" ::: "memory");
                    const uint32_t bar = smem_u32(&bars->dh_full[hp.st]);
                    const uint32_t dst = lbuf_s + hp.st * kHBytesP;
                    const CUtensorMap* src = hq >= 1 ? &tmY : &tmX;
                    const int m0 = (cl + ht * ncl) * 2 * kRowsP + hf * kRowsP;
                    DLP_T(0, hq, hc, 0);
                    mbar_arrive_expect_tx(bar, kHBytesP);
                    if (hints) {
                        const uint64_t pol = hq >= 1 ? pol_h : pol_w;      // x is read once
                        tma_load_2d_hint(dst, src, col0 + hc * kCWP, m0, bar, pol);
                        tma_load_2d_hint(dst + 16384, src, col0 + hc * kCWP + 64, m0, bar, pol);
                    } else {
                        tma_load_2d(dst, src, col0 + hc * kCWP, m0, bar);
                        tma_load_2d(dst + 16384, src, col0 + hc * kCWP + 64, m0, bar);
                    }
                    hph[hp.st] = int(hp.ph);
                    hp.step(kNLP);
                    ++nh;
                    if (++hc == nch) { hc = 0; if (++hq == p.L) { hq = -1; ++ht; } }
                    did = true;
                }
                if (nu < total_w && mbar_test(smem_u32(&bars->u_empty[up.st]), up.ph ^ 1u)) {
                    const uint32_t dst = ubuf_s + up.st * C::U_BYTES;
                    DLP_T(1, uq, uc, 0);
                    if (hf == 0) mbar_arrive_expect_tx(smem_u32(&bars->u_full[up.st]), 2 * C::U_BYTES);
#pragma unroll
                    for (int t = 0; t < C::UT; ++t)
                        if (hints)
                            tma_load_2d_pair_hint(dst + t * C::U_TILE_BYTES, &tmU, 64 * t, uq * p.d + col0 + uc * kCWP + 64 * hf,
                                                  ufull_lead + 8u * up.st, pol_w);
                        else
                            tma_load_2d_pair(dst + t * C::U_TILE_BYTES, &tmU, 64 * t, uq * p.d + col0 + uc * kCWP + 64 * hf,
                                             ufull_lead + 8u * up.st);
                    uph[up.st] = int(up.ph);
                    up.step(NU);
                    ++nu;
                    if (++uc == nch) { uc = 0; if (++uq == p.L) uq = 0; }
                    did = true;
                }
                if (nv < total_w && mbar_test(smem_u32(&bars->v_empty[vp.st]), vp.ph ^ 1u)) {
                    const uint32_t dst = vbuf_s + vp.st * C::V_BYTES;
                    DLP_T(2, vq - 1, vc, 0);
                    if (hf == 0) mbar_arrive_expect_tx(smem_u32(&bars->v_full[vp.st]), 2 * C::V_BYTES);
#pragma unroll
                    for (int t = 0; t < 2; ++t)
                        if (hints)
                            tma_load_2d_pair_hint(dst + t * C::V_TILE_BYTES, &tmV, col0 + vc * kCWP + 64 * t, vq * R + (R / 2) * hf,
                                                  vfull_lead + 8u * vp.st, pol_w);
                        else
                            tma_load_2d_pair(dst + t * C::V_TILE_BYTES, &tmV, col0 + vc * kCWP + 64 * t, vq * R + (R / 2) * hf,
                                             vfull_lead + 8u * vp.st);
                    vph[vp.st] = int(vp.ph);
                    vp.step(NV);
                    ++nv;
                    if (++vc == nch) { vc = 0; if (++vq == p.L) vq = 0; }
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
                // copies requested before giving up still land in shared memory: wait for them (the weight copies of
                // both CTAs are counted in the leader, which the second CTA outlasts through the cluster barrier)
                for (int i = 0; i < kNLP; ++i)
                    if (hph[i] >= 0) mbar_wait(smem_u32(&bars->dh_full[i]), uint32_t(hph[i]), kDrainPolls);
                if (hf == 0) {
                    for (int i = 0; i < int(NU); ++i)
                        if (uph[i] >= 0) mbar_wait_cluster(smem_u32(&bars->u_full[i]), uint32_t(uph[i]), kDrainPolls);
                    for (int i = 0; i < int(NV); ++i)
                        if (vph[i] >= 0) mbar_wait_cluster(smem_u32(&bars->v_full[i]), uint32_t(vph[i]), kDrainPolls);
                }
            }
        }
    } else if (warp == 1) {
        // =============================== U-MMA warp (leader) =======================
        // buffer = s(q)[256 x R] * U'[q][chunk rows, :]^T, A from tensor memory of both CTAs
        if (lane == 0 && hf == 0) {
            constexpr uint32_t idesc_u = umma_idesc_bf16(256, kCWP);
            RingPos up;
            uint32_t n = 0;
            uint32_t c_s = 0;
            for (int t = 0; t < my_tiles && !err; ++t) {
                // the pass over x goes through the buffers too (chunk n: buffer n & 1): nothing to multiply, but the
                // chunk's barrier gets its commit (which arrives at once) when the buffer is free
                for (int c = 0; c < nch && !err; ++c, ++n) {
                    const uint32_t b = n & 1u;
                    if (!w.cta(smem_u32(&bars->a_free[b]), ((n >> 1) & 1u) ^ 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    umma_commit2_mask(smem_u32(&bars->dh_full[b]), pair_mask);
                }
                for (int q = 0; q < p.L && !err; ++q) {
                    err_layer = q;
                    DLP_T(3, q, 0, 7);
                    if (!w.cluster(smem_u32(&bars->s_ready), c_s & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    DLP_T(3, q, 0, 0);
                    ++c_s;
                    tc_fence_after();
                    for (int c = 0; c < nch; ++c, ++n) {
                        const uint32_t b = n & 1u;
                        // the weights land early: wait for them first, off the critical path
                        if (!w.cluster(smem_u32(&bars->u_full[up.st]), up.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                        DLP_T(3, q, c, 1);
                        const uint32_t acc = tmem_base + kBufCol + b * 128u;
                        // the buffer is free once the V contraction of the chunk two before has read it
                        if (!w.cta(smem_u32(&bars->a_free[b]), ((n >> 1) & 1u) ^ 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        DLP_T(3, q, c, 2);
                        tc_fence_after();
                        const uint32_t ub = ubuf_s + up.st * C::U_BYTES;
#pragma unroll
                        for (int k = 0; k < R / 16; ++k) {
                            const uint64_t bdesc = umma_desc(ub + uint32_t(k / 4) * C::U_TILE_BYTES, 2u, 1024u) + uint64_t(2 * (k % 4));
                            umma_ts2(acc, tmem_base + kSCol + uint32_t(8 * k), bdesc, idesc_u, k ? 1u : 0u);
                        }
                        umma_commit2_mask(smem_u32(&bars->u_empty[up.st]), pair_mask);
                        up.step(NU);
                        umma_commit2_mask(smem_u32(&bars->dh_full[b]), pair_mask);
                        DLP_T(3, q, c, 3);
                    }
                }
            }
            umma_commit2(smem_u32(&bars->drain[0]));
            mbar_wait(smem_u32(&bars->drain[0]), 0, kDrainPolls);
        }
    } else if (warp == 2) {
        // =============================== V-MMA warp (leader) =======================
        // z(q+1)[256 x R] += h_new[chunk][256 x 128] * V'[q+1][:, chunk]^T, A = the updated chunk in tensor memory
        if (lane == 0 && hf == 0) {
            constexpr uint32_t idesc_v = umma_idesc_bf16(256, R);
            RingPos vp;
            uint32_t n = 0;
            for (int t = 0; t < my_tiles && !err; ++t) {
                for (int q = -1; q < p.L && !err; ++q) {
                    err_layer = q;
                    const bool feeds = q + 1 < p.L;
                    for (int c = 0; c < nch; ++c, ++n) {
                        const uint32_t b = n & 1u;
                        // the weights land early: wait for them first, off the critical path
                        if (feeds && !w.cluster(smem_u32(&bars->v_full[vp.st]), vp.ph)) { err = DLRB200_ERR_TIMEOUT_COPY; break; }
                        DLP_T(4, q, c, 1);
                        if (!w.cluster(smem_u32(&bars->a_ready[b]), (n >> 1) & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        DLP_T(4, q, c, 2);
                        tc_fence_after();
                        if (feeds) {
                            const uint32_t a0 = tmem_base + kBufCol + b * 128u;
                            const uint32_t vb = vbuf_s + vp.st * C::V_BYTES;
#pragma unroll
                            for (int k = 0; k < kCWP / 16; ++k) {
                                const uint64_t bdesc = umma_desc(vb + uint32_t(k / 4) * C::V_TILE_BYTES, 2u, 1024u) + uint64_t(2 * (k % 4));
                                umma_ts2(tmem_base + kZCol, a0 + uint32_t(32 * (k / 2) + 8 * (k % 2)), bdesc, idesc_v, (c | k) ? 1u : 0u);
                            }
                            umma_commit2_mask(smem_u32(&bars->v_empty[vp.st]), pair_mask);
                            vp.step(NV);
                        }
                        // the chunk has been read (last layer: nothing reads it, the commit arrives at once)
                        umma_commit2_mask(smem_u32(&bars->a_free[b]), pair_mask);
                        DLP_T(4, q, c, 3);
                    }
                    if (err) break;
                    if (feeds) umma_commit2_mask(smem_u32(&bars->z_full), pair_mask);
                }
            }
            umma_commit2(smem_u32(&bars->drain[1]));
            mbar_wait(smem_u32(&bars->drain[1]), 0, kDrainPolls);
        }
    } else if (warp == 3) {
        // =============================== store warp ================================
        // new chunk -> output buffer.  A slot is released when the copy has read it; the chunk counts as
        // stored (readable by the next pass) once its bulk group is complete, which is checked two chunks late
        // so that this warp never waits for a write in flight.
        if (lane == 0) {
            RingPos sp;
            const uint64_t pol_h = l2_policy_evict_last(), pol_out = l2_policy_evict_first();
            const bool hints = !(PROF && (p.exp & 32));
            unsigned int n = 0;              // chunks seen (all tiles, all passes): the producer counts the same way
            // the store slots of the first two chunks are free from the start
            mbar_arrive(smem_u32(&bars->dh_full[0]));
            mbar_arrive(smem_u32(&bars->dh_full[1]));
            for (int t = 0; t < my_tiles && !err; ++t) {
                const int m0 = (cl + t * ncl) * 2 * kRowsP + hf * kRowsP;
                // (the pass over x stores nothing but walks the slots like the others: chunk n uses slot n & 1, as it
                // uses buffer n & 1)
                for (int q = -1; q < p.L && !err; ++q) {
                    err_layer = q;
                    for (int c = 0; c < nch; ++c, ++n) {
                        if (!w.cta(smem_u32(&bars->s_written[sp.st]), sp.ph)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        DLP_T(5, q, c, 0);
                        if (q >= 0 && m0 < p.M && !(PROF && (p.exp & 8))) {   // a CTA whose rows lie wholly past the batch stores nothing
                            const uint32_t src = sbuf_s + sp.st * kHBytesP;
                            if (hints) {       // the last layer's output is not read again here: first to leave L2
                                const uint64_t pol = q + 1 < p.L ? pol_h : pol_out;
                                tma_store_2d_hint(&tmY, col0 + c * kCWP, m0, src, pol);
                                tma_store_2d_hint(&tmY, col0 + c * kCWP + 64, m0, src + 16384, pol);
                            } else {
                                tma_store_2d(&tmY, col0 + c * kCWP, m0, src);
                                tma_store_2d(&tmY, col0 + c * kCWP + 64, m0, src + 16384);
                            }
                        }
                        bulk_commit_group();
                        bulk_wait_group_read<0>();
                        DLP_T(5, q, c, 1);
                        // the slot is free for the chunk after next: one of the three arrivals its barrier waits for
                        mbar_arrive(smem_u32(&bars->dh_full[sp.st]));
                        sp.step(kNSP);
                        bulk_wait_group<2>();            // every group but the last two is complete
                        if (n + 1u > *stored + 2u) *stored = n + 1u - 2u;
                    }
                }
            }
            bulk_wait_group<0>();
        }
    } else if (warp >= 4) {
        // =============================== epilogue warps =============================
        // Four threads per row: thread (row er, quarter cq) owns 32 of the 128 columns of every chunk and a
        // quarter of the columns of z.  Warp w reads tensor-memory lanes 32 * (w % 4) .. + 31.  Sixteen warps,
        // four per scheduler: the per-chunk chain of one warp (wait, tensor-memory load, add, pack, store,
        // signal) is latency-bound, and the other three fill its gaps.
        const int q4 = warp & 3;
        const int cq = (warp - 4) >> 2;
        const int er = 32 * q4 + lane;
        const int et = int(threadIdx.x) - 128;            // = cq * 128 + er
        const uint32_t tl = tmem_base + (uint32_t(32 * q4) << 16);
        uint32_t n = 0;                      // chunks seen (all passes): phase of the A operand's barriers
        uint32_t c_z = 0;
        // barriers of the leader that this warp signals: its own if this CTA leads, else through the cluster window
        const uint32_t l_a_ready = hf ? mapa(smem_u32(&bars->a_ready[0]), lead) : smem_u32(&bars->a_ready[0]);
        const uint32_t l_s_ready = hf ? mapa(smem_u32(&bars->s_ready), lead) : smem_u32(&bars->s_ready);
        auto arrive_lead = [&](uint32_t bar) {
            if (hf) mbar_arrive_remote_light(bar);
            else mbar_arrive(bar);
        };

        RingPos lp, sp;
        const int trole = (warp == 4 && lane == 0) ? 6 : ((warp == 19 && lane == 0) ? 7 : -1);
#define DLP_TE(layer, chunk, event) do { if (PROF && trole >= 0) DLP_T(trole, layer, chunk, event); } while (0)
        const uint32_t x7 = uint32_t(er & 7);
        // this thread's 64 bytes of its row inside a staging slot: tile cq / 2, 16-byte pieces 4 (cq % 2) .. + 3
        const uint32_t row_off = uint32_t((cq >> 1) * 16384 + er * 128);
        const uint32_t piece0 = uint32_t((cq & 1) * 4);
        for (int t = 0; t < my_tiles && !err; ++t) {
            float ssq0 = 0.f, ssq1 = 0.f;
            for (int q = -1; q < p.L && !err; ++q) {
                err_layer = q;
                for (int c = 0; c < nch; ++c, ++n) {
                    const uint32_t b = n & 1u;
                    const uint32_t buf = tl + kBufCol + b * 128u + uint32_t(32 * cq);   // this thread's 32 columns of the buffer
                    // ---- old values of the chunk: this thread's 64 bytes of its row, from the staging slot
                    DLP_TE(q, c, 0);
                    // ---- the one wait of a chunk: dh is in the buffer (in the pass over x: the buffer is free), the old
                    // values of the chunk have landed in their slot and the store slot is free
                    if (!w.cta(smem_u32(&bars->dh_full[b]), (n >> 1) & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    tc_fence_after();
                    DLP_TE(q, c, 1);
                    uint32_t cur[16];
                    {
                        const uint8_t* rowp = lbuf + lp.st * kHBytesP + row_off;
                        if (PROF && (p.exp & 1)) rowp = lbuf + lane * 16;     // experiment: no bank-spread reads
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            if (PROF && (p.exp & 2)) { cur[4 * j] = cur[4 * j + 1] = cur[4 * j + 2] = cur[4 * j + 3] = 0x3f803f80u; continue; }
                            const uint4 hv = *reinterpret_cast<const uint4*>(rowp + (((piece0 + uint32_t(j)) ^ x7) << 4));
                            cur[4 * j] = hv.x; cur[4 * j + 1] = hv.y; cur[4 * j + 2] = hv.z; cur[4 * j + 3] = hv.w;
                        }
                    }
                    if (q >= 0) {
                        DLP_TE(q, c, 2);
                        uint32_t dv[32];
                        tmem_ld32(buf, dv);
                        tmem_wait_ld();
                        // the old values are in registers (the loads above have returned by now): the slot can take the
                        // next chunk
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->l_free[lp.st]));
                        DLP_TE(q, c, 3);
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (PROF && (p.exp & 16)) { cur[j] ^= dv[2 * j] & dv[2 * j + 1]; continue; }
                            // two columns at a time with the packed fp32 instructions (one add, one fma per pair)
                            const uint32_t hw = cur[j];
                            float f0, f1;
                            add_f32x2(f0, f1, bf16lo_to_f(hw), bf16hi_to_f(hw), __uint_as_float(dv[2 * j]), __uint_as_float(dv[2 * j + 1]));
                            fma_f32x2(ssq0, ssq1, f0, f1, f0, f1, ssq0, ssq1);
                            cur[j] = pack_bf16x2(f0, f1);
                        }
                    } else {
                        // pass over x: the chunk goes to the tensor core as it is
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->l_free[lp.st]));
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const float f0 = bf16lo_to_f(cur[j]), f1 = bf16hi_to_f(cur[j]);
                            ssq0 = fmaf(f0, f0, ssq0);
                            ssq1 = fmaf(f1, f1, ssq1);
                        }
                    }
                    lp.step(kNLP);
                    // ---- the chunk (bf16) becomes the A operand of the next layer's contraction, over this thread's own
                    // columns of dh: first, because the tensor core waits for it
                    DLP_TE(q, c, 4);
                    tmem_st16(buf, cur);
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) arrive_lead(l_a_ready + 8u * b);
                    DLP_TE(q, c, 6);
                    // ---- new values into a store slot: the store warp copies the slot out
                    {
                        if (q >= 0) {
                            uint8_t* rowp = sbuf + sp.st * kHBytesP + row_off;
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (!(PROF && (p.exp & 4))) *reinterpret_cast<uint4*>(rowp + (((piece0 + uint32_t(j)) ^ x7) << 4)) =
                                    make_uint4(cur[4 * j], cur[4 * j + 1], cur[4 * j + 2], cur[4 * j + 3]);
                            fence_async_smem();
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&bars->s_written[sp.st]));
                        sp.step(kNSP);
                    }
                    DLP_TE(q, c, 7);
                }
                if (err) break;
                if (q + 1 < p.L) {
                    // ---- z(q+1) is complete after the last chunk's V contraction: s = silu(z * rstd) -> tensor memory
                    constexpr int NZ = C::NZ;            // columns of z per thread: 32 (rank 128) or 16 (rank 64)
                    float ssq = ssq0 + ssq1;
                    ssq0 = ssq1 = 0.f;
                    DLP_TE(q, 24, 0);
                    if (!w.cluster(smem_u32(&bars->z_full), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    DLP_TE(q, 24, 1);
                    tc_fence_after();
                    uint32_t zv[NZ];
                    if constexpr (NZ == 32) tmem_ld32(tl + kZCol + uint32_t(cq * NZ), zv);
                    else tmem_ld16(tl + kZCol + uint32_t(cq * NZ), zv);
                    tmem_wait_ld();
                    // The pairs hold partial z over their parts of the width.  In step s each CTA sends its running
                    // sum (rounded to bf16) and its sum of squares so far to the CTA with the same rows in pair
                    // pi ^ (1 << s), and both add own (rounded alike) + received: the same s on all sides.  All steps
                    // of a CTA receive into one buffer: a message is sent once the receiver has read the one before.
                    for (int step = 0; step < nsteps; ++step) {
                        const uint32_t partner = crank ^ (2u << step);
                        if (step == 0) {
                            // the first partner acknowledged the last message of the layer before
                            if (c_z > 0 && !w.cluster(smem_u32(&bars->xack_bar[0]), (c_z - 1u) & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        } else {
                            // this CTA has read the message of the step before: the partner of this step may send; and
                            // that partner must have read its own
                            __syncwarp();
                            if (lane == 0) mbar_arrive_remote_light(mapa(smem_u32(&bars->xack_bar[step]), partner));
                            if (!w.cluster(smem_u32(&bars->xack_bar[step]), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        }
                        const uint32_t p_recv = mapa(smem_u32(recv), partner);
                        const uint32_t p_recv_q = mapa(smem_u32(recv_q), partner);
                        const uint32_t p_xchg = mapa(smem_u32(&bars->xchg_bar[step]), partner);
                        if (et == 0) mbar_arrive_expect_tx(smem_u32(&bars->xchg_bar[step]), C::RECV_BYTES);
#pragma unroll
                        for (int k = 0; k < C::NZW; ++k) {
                            const float* f = reinterpret_cast<const float*>(&zv[8 * k]);
                            const uint32_t o0 = pack_bf16x2(f[0], f[1]), o1 = pack_bf16x2(f[2], f[3]);
                            const uint32_t o2 = pack_bf16x2(f[4], f[5]), o3 = pack_bf16x2(f[6], f[7]);
                            st_async_v4(p_recv + uint32_t((k * kEpiThreadsP + et) * 16), o0, o1, o2, o3, p_xchg);
                            // own running sum, rounded like the one that was sent
                            zv[8 * k] = o0 << 16; zv[8 * k + 1] = o0 & 0xffff0000u;
                            zv[8 * k + 2] = o1 << 16; zv[8 * k + 3] = o1 & 0xffff0000u;
                            zv[8 * k + 4] = o2 << 16; zv[8 * k + 5] = o2 & 0xffff0000u;
                            zv[8 * k + 6] = o3 << 16; zv[8 * k + 7] = o3 & 0xffff0000u;
                        }
                        st_async_b32(p_recv_q + uint32_t(et * 4), __float_as_uint(ssq), p_xchg);
                        DLP_TE(q, 24, 2);
                        if (!w.cluster(smem_u32(&bars->xchg_bar[step]), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                        DLP_TE(q, 24, 3);
                        ssq += recv_q[et];
#pragma unroll
                        for (int k = 0; k < C::NZW; ++k) {
                            const uint4 v = recv[k * kEpiThreadsP + et];
                            float* f = reinterpret_cast<float*>(&zv[8 * k]);
                            f[0] += bf16lo_to_f(v.x); f[1] += bf16hi_to_f(v.x);
                            f[2] += bf16lo_to_f(v.y); f[3] += bf16hi_to_f(v.y);
                            f[4] += bf16lo_to_f(v.z); f[5] += bf16hi_to_f(v.z);
                            f[6] += bf16lo_to_f(v.w); f[7] += bf16hi_to_f(v.w);
                        }
                    }
                    if (err) break;
                    ssqx[cq * kRowsP + er] = ssq;              // index et: the word this thread's received partial came in
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&bars->ssq_bar));
                    if (!w.cta(smem_u32(&bars->ssq_bar), c_z & 1u)) { err = DLRB200_ERR_TIMEOUT_BARRIER; break; }
                    // the four quarters in a fixed order: every thread of a row gets the same total
                    const float tot = (ssqx[er] + ssqx[kRowsP + er]) + (ssqx[2 * kRowsP + er] + ssqx[3 * kRowsP + er]);
                    const float rstd = rsqrtf(tot * p.inv_d + p.eps);
                    DLP_TE(q, 24, 4);
                    if (nsteps > 0) {
                        // the last message and the words shared with it have been read: the first partner may send again
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote_light(mapa(smem_u32(&bars->xack_bar[0]), crank ^ 2u));
                    }
                    uint32_t sv[NZ / 2];
#pragma unroll
                    for (int j = 0; j < NZ / 2; ++j)
                        sv[j] = pack_bf16x2(silu_tanh_f(__uint_as_float(zv[2 * j]) * rstd), silu_tanh_f(__uint_as_float(zv[2 * j + 1]) * rstd));
                    if constexpr (NZ == 32) tmem_st16(tl + kSCol + uint32_t(cq * (NZ / 2)), sv);
                    else tmem_st8(tl + kSCol + uint32_t(cq * (NZ / 2)), sv);
                    ++c_z;
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) arrive_lead(l_s_ready);
                    DLP_TE(q, 24, 5);
                }
            }
        }
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
    // no CTA may free the pair's tensor memory, or leave, while another can still use it or signal its barriers
    cluster_arrive_release();
    cluster_wait_acquire();
    if (warp == 3) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
    }
}

// Shape of a launch: pairs per cluster (1, 2 or 4: they split the width) and clusters in the grid.  For each
// number of pairs that fits, estimated time = rounds x (chunks per pair x time per chunk + the pause at the end
// of a layer, which grows with the exchange steps), where the clusters of a round are as many as can be resident
// and no more than keep the rows in flight inside L2: every layer rewrites its tile in place, and once the tiles
// of a round outgrow L2 each layer's traffic goes to DRAM (measured at d = 4096: 16384 rows at once 8.2 ms, in
// two rounds of 8448 rows 6.6 ms).  Every pair keeps at least four chunks (the store warp reports a chunk as
// stored two chunks late and the producer runs up to three chunks ahead).
struct PairShape { int pp, clusters; };
PairShape pick_shape(int num_tiles, int d, int r, const int (&max_clusters)[3], size_t l2_bytes) {
    int forced = 0;
    if (const char* e = getenv("DLRB200_PAIR_SPLIT")) forced = atoi(e);
    const int nch = d / kCWP;
    const double t_chunk = r == 128 ? 1.09 : 0.80;
    const size_t tile_bytes = size_t(2 * kRowsP) * d * 2;
    int fit = int(double(l2_bytes) * 0.62 / double(tile_bytes));      // tiles whose rows stay in L2 beside the weight stream
    if (fit < 1) fit = 1;
    PairShape best{0, 0};
    double best_t = 1e30;
    for (int pp = 1, i = 0; pp <= 4; pp *= 2, ++i) {
        if (forced && pp != forced) continue;
        if (nch % pp || nch / pp < 4 || max_clusters[i] < 1) continue;
        int clusters = max_clusters[i] < fit ? max_clusters[i] : fit;
        if (clusters > num_tiles) clusters = num_tiles;
        const int rounds = (num_tiles + clusters - 1) / clusters;
        const double pause = (r == 128 ? 3.4 : 2.0) + (pp == 4 ? 2.8 : (pp == 2 ? 1.0 : 0.0));
        const double t = rounds * ((nch / pp) * t_chunk + pause);
        if (t < best_t) { best_t = t; best = PairShape{pp, clusters}; }
    }
    return best;
}

template <int R>
int launch_pair(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int L, float eps,
                int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
                dlrb200_plan* plan_only, unsigned long long* prof) {
    using C = PCfg<R>;
    if (C::SMEM_BYTES > smem_optin) return DLRB200_ERR_OCCUPANCY;
    const int num_tiles = (M + 2 * kRowsP - 1) / (2 * kRowsP);
    auto kern = prof ? dlr_stream_pair_kernel<R, true> : dlr_stream_pair_kernel<R, false>;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cudaLaunchAttribute attr[1];
    cfg.blockDim = dim3(kThreadsP);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // per process (one device per process) and kernel: shared-memory opt-in, clusters of 2, 4 and 8 CTAs that can
    // be resident at once, size of L2
    struct DeviceFacts { bool known; int max_clusters[3]; size_t l2_bytes; };
    static DeviceFacts facts[2] = {{false, {0, 0, 0}, 0}, {false, {0, 0, 0}, 0}};
    static std::mutex facts_mutex;
    DeviceFacts f;
    {
        std::lock_guard<std::mutex> lock(facts_mutex);
        DeviceFacts& slot = facts[prof ? 1 : 0];
        if (!slot.known) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
                return DLRB200_ERR_CUDA;
            for (int i = 0; i < 3; ++i) {
                const int cs = 2 << i;
                attr[0].val.clusterDim.x = cs;
                cfg.gridDim = dim3(cs * (num_sms / cs));
                int mc = 0;
                if (cudaOccupancyMaxActiveClusters(&mc, kern, &cfg) != cudaSuccess) mc = 0;
                slot.max_clusters[i] = mc;
            }
            int dev = 0, l2 = 0;
            if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) != cudaSuccess)
                return DLRB200_ERR_CUDA;
            slot.l2_bytes = size_t(l2);
            slot.known = true;
        }
        f = slot;
    }
    const PairShape sh = pick_shape(num_tiles, d, R, f.max_clusters, f.l2_bytes);
    if (sh.pp < 1) return DLRB200_ERR_OCCUPANCY;
    const int pp = sh.pp, clusters = sh.clusters;
    attr[0].val.clusterDim.x = 2 * pp;
    const int grid = clusters * 2 * pp;
    cfg.gridDim = dim3(grid);
    if (plan_only) {
        plan_only->path = DLRB200_PATH_STREAMED_PAIRS;
        plan_only->grid = grid;
        plan_only->cluster = 2 * pp;
        plan_only->stripe_cols = kCWP;
        plan_only->rows_per_pass = 2 * kRowsP;
        plan_only->passes = (num_tiles + clusters - 1) / clusters;
        plan_only->stages = C::NU + C::NV;
        plan_only->smem_bytes = size_t(C::SMEM_BYTES);
        return DLRB200_OK;
    }
    CUtensorMap tmX, tmY, tmV, tmU;
    if (!encode_2d_bf16(enc, &tmX, x, uint64_t(d), uint64_t(M), 64, kRowsP, 128) ||
        !encode_2d_bf16(enc, &tmY, y, uint64_t(d), uint64_t(M), 64, kRowsP, 128) ||
        !encode_2d_bf16(enc, &tmV, Vp, uint64_t(d), uint64_t(L) * R, 64, R / 2, 128) ||
        !encode_2d_bf16(enc, &tmU, Up, uint64_t(R), uint64_t(L) * d, 64, 64, 128))
        return DLRB200_ERR_CUDA;
    PParams p;
    p.M = M; p.d = d; p.L = L;
    p.nch = d / kCWP;
    p.pp = pp;
    p.num_tiles = num_tiles;
    p.eps = eps;
    p.inv_d = 1.0f / float(d);
    p.status = status_dev;
    p.spin_limit = spin_limit;
    p.prof = prof;
    p.trace_layer = L / 2;
    p.exp = 0;
    if (prof) {
        if (const char* e = getenv("DLRB200_EXP")) p.exp = atoi(e);
    }
    const cudaError_t ce = cudaLaunchKernelEx(&cfg, kern, tmX, tmY, tmV, tmU, p);
    return ce == cudaSuccess ? DLRB200_OK : DLRB200_ERR_CUDA;
}

int dispatch_pair(void* enc, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r, int L, float eps,
                  int* status_dev, cudaStream_t stream, int num_sms, int smem_optin, unsigned int spin_limit,
                  dlrb200_plan* plan_only, unsigned long long* prof) {
    switch (r) {
        case 64: return launch_pair<64>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only, prof);
        case 128: return launch_pair<128>(enc, x, y, Vp, Up, M, d, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit, plan_only, prof);
    }
    return DLRB200_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace

bool stream_pair_supported(int d, int r) { return (r == 64 || r == 128) && d % kCWP == 0 && d >= 4 * kCWP; }

int stream_pair_plan(int M, int d, int r, int L, int num_sms, int smem_optin, dlrb200_plan* plan) {
    const size_t ws = plan->workspace_bytes;
    const int rc = dispatch_pair(nullptr, nullptr, nullptr, nullptr, nullptr, M, d, r, L, 0.f, nullptr, nullptr, num_sms, smem_optin, 0,
                                 plan, nullptr);
    plan->workspace_bytes = ws;
    return rc;
}

int stream_pair_forward(void* encode_fn_ptr, const void* x, void* y, const void* Vp, const void* Up, int M, int d, int r,
                        int L, float eps, int* status_dev, cudaStream_t stream, int num_sms, int smem_optin,
                        unsigned int spin_limit, unsigned long long* prof) {
    if (num_sms > 160) return DLRB200_ERR_OCCUPANCY;
    return dispatch_pair(encode_fn_ptr, x, y, Vp, Up, M, d, r, L, eps, status_dev, stream, num_sms, smem_optin, spin_limit, nullptr,
                         prof);
}

}  // namespace dlr
