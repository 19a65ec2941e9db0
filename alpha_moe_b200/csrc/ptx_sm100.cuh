// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), cp.async,
// tcgen05 (TMEM alloc, UMMA issue/commit, TMEM loads) and bf16x2 global reductions.
//
// This header takes the place of the reference's Hopper helper layer
// (csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:41-633: wgmma wrappers,
// Hopper smem descriptors, TMA/mbarrier helpers, stmatrix); none of that layer can be
// assembled for sm_100a, so everything here is written against the Blackwell
// instructions instead.  Every wait is bounded: a wait that runs out records a status
// word and returns false, it never spins forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace amoe {

// ---------------------------------------------------------------------------------------------
// status word written by a kernel whose bounded wait ran out (0 = healthy)
struct KernelStatus {
    int code;     // 0 ok, otherwise WAIT_* below
    int block;    // blockIdx.x of the first CTA that gave up
    int where;    // role-specific tag (which barrier)
    int iter;     // pipeline iteration
};
enum : int { ST_OK = 0, ST_WAIT_TIMEOUT = 1, ST_SMEM_MISALIGNED = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// --------------------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrival without release ordering: for hand-offs where the arriving thread has written nothing the
// waiter will read (e.g. "TMEM has been read", "ring slot is free").  A default (release) arrive would
// also wait for this thread's outstanding global reductions to be acknowledged by L2.
__device__ __forceinline__ void mbar_arrive_relaxed(uint64_t* bar) {
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_relaxed_n(uint64_t* bar, uint32_t n) {
    asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Limit of one wait, in SM clock cycles (about a second at B200 clocks).
constexpr long long kWaitLimitCycles = 2000000000LL;

// Bounded wait.  `abort_flag` is a CTA-shared word: once any thread of the CTA gives up, every
// other waiter of that CTA returns false at its next poll, so the CTA unwinds as a whole.
// (Kept inline: a device function call inside a role that has resized its register allotment with
// setmaxnreg does not get through register allocation.)
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                KernelStatus* status, int where, int iter, long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1;
            if (atomicCAS(&status->code, ST_OK, ST_WAIT_TIMEOUT) == ST_OK) {
                status->block = blockIdx.x;
                status->where = where;
                status->iter = iter;
            }
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          KernelStatus* status, int where, int iter) {
    return mbar_wait_limit(bar, parity, abort_flag, status, where, iter, kWaitLimitCycles);
}

// --------------------------------------------------------------------------------------------- clusters / DSMEM
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Hardware barrier over all threads of all CTAs of the cluster (used once, right after barrier set-up,
// where every CTA arrives unconditionally).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cta address -> address of the same location in the shared memory of CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that CTAs of the cluster arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  KernelStatus* status, int where, int iter) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitLimitCycles) {
            *abort_flag = 1;
            if (atomicCAS(&status->code, ST_OK, ST_WAIT_TIMEOUT) == ST_OK) {
                status->block = blockIdx.x;
                status->where = where;
                status->iter = iter;
            }
            return false;
        }
    }
}

// --------------------------------------------------------------------------------------------- proxies
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// --------------------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// --------------------------------------------------------------------------------------------- cp.async (16 B)
// src_bytes = 16 copies, src_bytes = 0 writes 16 zero bytes (src must still be a valid address).
__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}
// The mbarrier receives one arrival from this thread once all cp.async copies it has issued so far have
// landed (asynchronously: the thread does not wait).  .noinc: the arrival is part of the barrier's
// expected count, so a phase cannot complete before every gathering thread's copies are in.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t n) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// --------------------------------------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor, K-major operand stored as rows of 128 bytes with the 128-byte
// swizzle (what TMA writes with CU_TENSOR_MAP_SWIZZLE_128B); the leading offset is unused for this
// layout, descriptor version 1, layout type 2.
// `sbo` is the distance between consecutive 8-row groups of the operand: 1024 for a dense tile, 2048
// to take every other 8-row group of a tile (how the gate / up halves of the interleaved `w` rows are
// picked apart without moving any data).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t sbo = 1024u) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);        // start address  [0,14)
    d |= static_cast<uint64_t>(sbo >> 4) << 32;                     // stride byte offset [32,46)
    d |= static_cast<uint64_t>(1) << 46;                            // version [46,48)
    d |= static_cast<uint64_t>(2) << 61;                            // SWIZZLE_128B [61,64)
    return d;
}
// Instruction descriptor for kind::f8f6f4, e4m3 x e4m3 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// One 128-deep K chunk (four K=32 steps) of two independent accumulators:
//   D0 = A0 * B0, D1 = A1 * B1   (fresh accumulation: the first step overwrites D).
// All eight instructions sit in one asm block so that the issuing thread spends no instructions
// between them; descriptors advance by 32 bytes (2 in units of 16 B) per K step.
__device__ __forceinline__ void umma_f8_chunk2(uint32_t d0, uint32_t d1, uint64_t a0, uint64_t a1, uint64_t b0,
                                               uint64_t b1, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 a0k, a1k, b0k, b1k;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %2, %4, %6, pf;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], %3, %5, %6, pf;\n\t"
        "add.u64 a0k, %2, 2;\n\tadd.u64 a1k, %3, 2;\n\tadd.u64 b0k, %4, 2;\n\tadd.u64 b1k, %5, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a0k, b0k, %6, pt;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], a1k, b1k, %6, pt;\n\t"
        "add.u64 a0k, %2, 4;\n\tadd.u64 a1k, %3, 4;\n\tadd.u64 b0k, %4, 4;\n\tadd.u64 b1k, %5, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a0k, b0k, %6, pt;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], a1k, b1k, %6, pt;\n\t"
        "add.u64 a0k, %2, 6;\n\tadd.u64 a1k, %3, 6;\n\tadd.u64 b0k, %4, 6;\n\tadd.u64 b1k, %5, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a0k, b0k, %6, pt;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%1], a1k, b1k, %6, pt;\n\t}"
        ::"r"(d0), "r"(d1), "l"(a0), "l"(a1), "l"(b0), "l"(b1), "r"(idesc)
        : "memory");
}
// Same for a single accumulator.
__device__ __forceinline__ void umma_f8_chunk1(uint32_t d0, uint64_t a0, uint64_t b, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred pf, pt;\n\t.reg .b64 a0k, bk;\n\t"
        "setp.ne.b32 pf, 0, 0;\n\tsetp.eq.b32 pt, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, pf;\n\t"
        "add.u64 a0k, %1, 2;\n\tadd.u64 bk, %2, 2;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a0k, bk, %3, pt;\n\t"
        "add.u64 a0k, %1, 4;\n\tadd.u64 bk, %2, 4;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a0k, bk, %3, pt;\n\t"
        "add.u64 a0k, %1, 6;\n\tadd.u64 bk, %2, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], a0k, bk, %3, pt;\n\t}"
        ::"r"(d0), "l"(a0), "l"(b), "r"(idesc)
        : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// mbarrier arrives once all UMMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread t of the warp gets lane (lane_base + t).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// --------------------------------------------------------------------------------------------- misc
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void red_add_bf16x2(__nv_bfloat16* addr, float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    // no "memory" clobber: nothing in a kernel reads `out` back, and the clobber would serialise the
    // shared-memory loads of neighbouring iterations behind each reduction
    asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(addr), "r"(*reinterpret_cast<uint32_t*>(&v)));
}
// Same, issued only where `row < nrows` (no branch: the bound check is a predicate on the instruction).
__device__ __forceinline__ void red_add_bf16x2_if(__nv_bfloat16* addr, float lo, float hi, int row, int nrows) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.lt.s32 p, %2, %3;\n\t"
        "@p red.global.add.noftz.bf16x2 [%0], %1;\n\t}"
        ::"l"(addr), "r"(*reinterpret_cast<uint32_t*>(&v)), "r"(row), "r"(nrows));
}
// Register re-balancing between warpgroups (all four warps of a warpgroup must execute it).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// Read-only global load that the compiler keeps where it is written (used to request small schedule words
// at kernel entry, ahead of the set-up work whose latency they then overlap).
__device__ __forceinline__ int ld_global_nc_s32(const int* p) {
    int v;
    asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation attribute may start while
// the kernel in front of it in the stream is still running; griddep_wait() returns once that kernel has completed and
// its writes are visible (at once if there is no such dependency), so nothing it produced may be read before.
// griddep_launch_dependents() tells the scheduler that the kernel behind this one may start now.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

}  // namespace amoe
