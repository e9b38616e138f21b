// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk/TMA copies, proxy
// fences, cluster addressing, legacy warp MMA (ldmatrix + mma.sync) and the
// tcgen05 / tensor-memory instructions.  Every wait helper here is bounded:
// it gives up after a fixed number of polls and reports failure to the caller,
// which records a status word and drains; nothing in this library spins
// forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dlr {

// ---------------------------------------------------------------------------
// addresses
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// shared::cta address of this CTA -> shared::cluster address of the same
// offset inside CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

// Arrive (release at cluster scope) on an mbarrier that lives in another CTA
// of the cluster; `bar_cluster` is a shared::cluster address from mapa().
__device__ __forceinline__ void mbar_arrive_remote(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster)
                 : "memory");
}

// Arrive on a barrier of another CTA without the cluster-scope release: for signals whose payload is not
// ordinary memory (tensor memory already made consistent with tcgen05.wait and tcgen05.fence, or registers
// already consumed).  The cluster-scope release above costs the issuing thread about a thousand cycles.
__device__ __forceinline__ void mbar_arrive_remote_light(uint32_t bar_cluster) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Acquire at cluster scope: needed when the arrivals come from other CTAs.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when `limit` polls went by without the phase
// completing (each try_wait itself blocks for a hardware-chosen short time).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    return false;
}

// Polls granted to the waits that run only when a kernel is giving up: copies and
// tensor-core work already requested must finish before the CTA leaves (they write
// into its shared memory), whatever limit the caller set for the ordinary waits.
constexpr uint32_t kDrainPolls = 1u << 20;

// Position in a ring of `S` stages (S known only at run time): stage index and
// phase parity, moved by stepping.  Never divide by S in a kernel loop: an
// integer division by a run-time value is a dependent chain of a few hundred
// cycles, and in a one-thread producer or MMA loop nothing hides it.
struct RingPos {
    uint32_t st = 0, ph = 0;
    __device__ __forceinline__ void step(uint32_t S) {
        if (++st == S) { st = 0; ph ^= 1u; }
    }
    __device__ __forceinline__ void advance(uint32_t k, uint32_t S) {
        st += k;
        while (st >= S) { st -= S; ph ^= 1u; }
    }
    __device__ __forceinline__ RingPos at(uint32_t k, uint32_t S) const {
        RingPos r = *this;
        r.advance(k, S);
        return r;
    }
};

// ---------------------------------------------------------------------------
// proxy fences
// ---------------------------------------------------------------------------
// Make generic-proxy writes to shared memory visible to the async proxy (TMA,
// tcgen05.mma operand reads).
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA: tiled 2-D load global -> shared, completion on an mbarrier.  No
// multicast anywhere in this library.  c0 (inner coordinate) times the element
// size must be a multiple of 16 bytes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---------------------------------------------------------------------------
// global-memory synchronisation primitives
// ---------------------------------------------------------------------------
__device__ __forceinline__ void red_release_add_u32(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void red_add_f32(float* p, float v) {
    asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}

// ---------------------------------------------------------------------------
// legacy warp MMA (used by the small-batch path: weights are the 16-row
// operand, token rows are the 8-wide operand)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Byte-offset swizzle shared by TMA (CU_TENSOR_MAP_SWIZZLE_32B/64B/128B) and
// the tcgen05 shared-memory descriptors: the 16-byte chunk index inside a
// span of 32/64/128 bytes is XORed with the row bits that start at bit 7.
// `bits` = 1, 2, 3 for the 32-, 64- and 128-byte modes; 0 = no swizzle.  The
// tile base must be 1024-byte aligned for the formula to depend on the offset
// alone.
__device__ __forceinline__ uint32_t swz(uint32_t off, int bits) {
    return off ^ (((off >> 7) & ((1u << bits) - 1u)) << 4);
}

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + __expf(-z)); }

// SiLU through the hardware tanh: z * sigmoid(z) = 0.5 z (1 + tanh(z / 2)).  One special-function
// operation per value instead of two (exp and reciprocal); tanh.approx is good to about 2^-11, far
// below the bf16 rounding the result gets.
__device__ __forceinline__ float silu_tanh_f(float z) {
    float t;
    const float hz = 0.5f * z;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(hz));
    return fmaf(hz, t, hz);
}

// Packed fp32 arithmetic (two lanes per instruction, each rounded like the scalar form).
__device__ __forceinline__ void add_f32x2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void fma_f32x2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16lo_to_f(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16hi_to_f(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ---------------------------------------------------------------------------
// cluster: remote shared-memory stores
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_cluster_v4(uint32_t addr_cluster, uint32_t a, uint32_t b, uint32_t c,
                                              uint32_t d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr_cluster), "r"(a), "r"(b),
                 "r"(c), "r"(d)
                 : "memory");
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr_cluster, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr_cluster), "f"(v) : "memory");
}

__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------
// tcgen05 / tensor memory (cta_group::1 only)
// ---------------------------------------------------------------------------
// Allocate `ncols` (power of two, >= 32) tensor-memory columns; one full warp
// executes this.  The base address is written to `dst_smem`.
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Instruction descriptor for kind::f16 with bf16 operands, fp32 accumulate,
// both operands K-major: bit 4 D=f32, bits 7-9 A=bf16, bits 10-12 B=bf16,
// bits 17-22 N>>3, bits 24-28 M>>4.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory operand descriptor for a K-major tile whose rows are one
// 128-byte swizzle span (64 bf16): start address >> 4 in bits 0-13, leading
// byte offset (unused for swizzled K-major, set to 1) in bits 16-29, stride
// byte offset = 1024 (eight 128-byte rows) >> 4 in bits 32-45, descriptor
// version 1 in bits 46-47, layout type 2 (128-byte swizzle) in bits 61-63.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3ffffu) >> 4);
    d |= uint64_t(1) << 16;
    d |= uint64_t(1024 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A holds 128 rows (lanes) x 16 bf16 packed
// two per 32-bit column.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Make the mbarrier track completion of all tcgen05 ops issued so far by this
// thread (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32-bit, 16 consecutive columns -> 16 registers per thread.  The
// warp reads the 32 lanes starting at 32*(warp_id % 4).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
          "r"(v[15])
        : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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

// The same for one 32-bit word.
__device__ __forceinline__ void st_async_b32(uint32_t dst_cluster, uint32_t a, uint32_t bar_cluster) {
    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(dst_cluster), "r"(a),
                 "r"(bar_cluster)
                 : "memory");
}

// Bounded waits on mbarriers that also give up when another thread of the CTA has
// raised the abort flag (a word in shared memory).
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
    // Whole warp, every lane with a barrier and parity of its own (lanes may name the same one): one poll
    // covers several barriers at the latency of one.  Returns true once every lane's phase is complete.
    __device__ __forceinline__ bool warp(uint32_t bar, uint32_t parity) const {
        bool done = false;
        for (uint32_t i = 0; i < limit; ++i) {
            if (!done) done = mbar_try_wait(bar, parity);
            if (__all_sync(0xffffffffu, done)) return true;
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

// ---------------------------------------------------------------------------
// TMA store (shared -> global through a tensor map) and its bulk groups
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0),
                 "r"(c1), "r"(src)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all but the N most recent groups of this thread have finished READING shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// all but the N most recent groups of this thread are complete (writes performed)
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Order generic-proxy accesses (any state space) against later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---------------------------------------------------------------------------
// tcgen05 with cta_group::2: the two CTAs of a pair (cluster ranks 2k and 2k+1)
// drive one tensor-core instruction of M = 256 rows.  Each CTA keeps its own 128
// rows of the A operand and of the accumulator in its own tensor memory (same
// addresses in both) and supplies half of the B operand's N rows from its own
// shared memory (same offsets in both).  One thread of the even-ranked CTA (the
// leader) issues; completion is signalled to barriers at the same offset in
// either or both CTAs.  A kernel uses one cta_group for all its tcgen05
// instructions.
// ---------------------------------------------------------------------------
// One warp of EACH CTA of the pair executes alloc / relinquish / dealloc.
__device__ __forceinline__ void tmem_alloc2(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

// D[tmem, both CTAs] (+)= A[tmem, both CTAs] * B[smem halves of both CTAs]; M = 256.
__device__ __forceinline__ void umma_ts2(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem, both CTAs] (+)= A[smem of both CTAs: each its own 128 rows] * B[smem halves of both CTAs]; M = 256.
__device__ __forceinline__ void umma_ss2(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Completion of all tcgen05 work issued so far by this thread arrives on the barrier
// at this shared-memory offset in every CTA of `cta_mask` (bit = rank in the cluster).
__device__ __forceinline__ void umma_commit2_mask(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(cta_mask)
                 : "memory");
}
// ... on this CTA's barrier only.
__device__ __forceinline__ void umma_commit2(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// Tiled 2-D load into THIS CTA's shared memory whose bytes are counted on a barrier
// that may live in the other CTA of the pair (`bar_cluster`: a shared::cluster address
// from mapa()).  One destination, no multicast: each CTA fetches its own half.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster)
        : "memory");
}

// L2 eviction priorities for TMA copies.  A stream that is read once per consumer (weights) should leave L2
// first; data that is re-read soon (the activations, re-read every layer) should stay.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                      uint32_t bar_cluster, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, int c0, int c1, uint32_t src, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;" ::"l"(map),
                 "r"(c0), "r"(c1), "r"(src), "l"(policy)
                 : "memory");
}

// Non-blocking test of an mbarrier phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
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

}  // namespace dlr
