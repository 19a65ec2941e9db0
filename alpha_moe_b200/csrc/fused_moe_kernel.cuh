// Fused W8A8 MoE expert MLP for sm_100a: up-projection -> SwiGLU -> fp8 re-quantisation ->
// down-projection -> weighted accumulation into `out`, one launch per layer call.
//
// Replaces csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:654-1098 (the Hopper
// wgmma megakernel).  One CTA handles one block of block_m sorted assignments of one expert and
// SPC (1 or 2) 128-wide slices of the intermediate dimension - SPC = 1 is the reference's
// decomposition (:1125); SPC = 2 lets one CTA own two slices so that each (token, expert) pair adds
// into `out` once instead of twice.  The machine mapping is new:
//   * weights are the UMMA "M" operand (128 rows per instruction), the gathered tokens the "N"
//     operand, accumulators live in TMEM (tcgen05.mma kind::f8f6f4), not in registers;
//   * the gate and up halves of the 8-row-interleaved `w` are separated for free: one TMA box
//     brings 256 interleaved rows, and two UMMA descriptors with an 8-row-group stride of 2048 B
//     pick the 128 gate rows and the 128 up rows, so gate[i] and up[i] of one intermediate column
//     land in the same TMEM lane and SwiGLU is thread-local;
//   * each 128-deep K chunk is accumulated into its own TMEM buffer and promoted into fp32
//     registers with the (128x128 weight block) x (token, 128-group) scales (reference :915-933
//     promotes into bf16); there are 2 to 8 such buffers (acc_buffers) so that the MMAs of the
//     following chunks overlap chunk k's promotion;
//   * roles: 2 gather warps (token rows by cp.async with the 128-byte swizzle applied by hand; lane 0
//     of the first one also issues the weight TMA), 2 UMMA-issuing warps that take alternate chunks
//     (one thread cannot issue eight UMMAs plus its barrier traffic fast enough to keep the tensor
//     pipe busy), 1-2 epilogue warpgroups.
//
// Shared-memory ring slot: [256 weight rows x 128 B = 32 KB][token tile BMP x 128 B].
//   up phase   : rows = one slice's 256 interleaved w rows of K-chunk kc; token tile = x rows of the chunk
//   down phase : two 128-row x 128-byte tiles of w2 - SPC = 1: two consecutive hidden-row tiles of the
//                slice; SPC = 2: the same 128 hidden rows for each of the two slices
#pragma once

#include <type_traits>

#include "ptx_sm100.cuh"

namespace amoe {

constexpr int kMaxTpWorld = 8;       // ranks whose `out` buffers one launch can add into

struct MoeParams {
    const uint8_t* x;          // fp8 e4m3 [M, K]
    const float* x_scale;      // [M, K/128]
    const float* w_scale;      // [E, N/128, K/128], gate/up rows interleaved by 1
    const float* w2_scale;     // [E, K/128, I/128]
    __nv_bfloat16* out;        // [M, K]
    // Tensor parallelism with the exchange step fused into the epilogue (small batches): the other ranks' `out`
    // buffers, mapped into this GPU's address space.  Every partial result is added into all tp_world buffers with
    // plain reductions over NVLink (no multicast, no tensor map covers peer memory); 1 = no peers.
    __nv_bfloat16* out_more[kMaxTpWorld - 1];
    int tp_world;
    const int* sorted_token_ids;
    const int* expert_ids;
    const int* num_tokens_post_padded;
    const float* topk_weights;  // [M, top_k]
    int top_k, M, K, N, E, sorted_num, block_m;
    int stages;                 // ring depth actually used (fits in shared memory)
    int ksplit;                 // CTAs of a cluster that share one (block, slice): 1 (no cluster), 2, 4 or 8
    float scaling;
    KernelStatus* status;
};


constexpr int kTileBytes = 128 * 128;  // one 128-row x 128-byte operand tile

// bf16x2 reduction of (lo, hi) into element offset `off` of this rank's `out` if row < M; with PEERS also into
// every peer's.  (A template parameter, not a run-time test: the loop next to every 4-byte reduction cost the
// single-GPU kernels 10-80 % when it was one.)
template <bool PEERS>
__device__ __forceinline__ void red_out_all_ranks(const MoeParams& p, size_t off, float lo, float hi, int row) {
    red_add_bf16x2_if(p.out + off, lo, hi, row, p.M);
    if constexpr (PEERS)
        for (int pr = 0; pr + 1 < p.tp_world; ++pr) red_add_bf16x2_if(p.out_more[pr] + off, lo, hi, row, p.M);
}

// Accumulator buffers in tensor memory (each: two accumulators x BMP columns).  The chain of one K chunk - operands
// landed, UMMAs issued, completion seen by the epilogue, read-back, buffer handed back - takes well over a thousand
// cycles while its UMMAs need about a hundred at these widths, so a narrow tile keeps as many chunks in flight as
// fit 256 columns (two CTAs of that size can share an SM's 512).
__host__ __device__ constexpr int acc_buffers(int bmp, int ew = 1) { return bmp <= 16 ? 8 : bmp == 32 ? 4 : (bmp == 64 && ew == 2) ? 4 : 2; }

struct SmemPlan {
    uint32_t stage_bytes, hq, xs, swg, swu, sw2, tokrow, topkw, tokscale, amax, part, bars, misc, total;
};
// Offsets from a 1024-byte aligned base.  bmp = padded block_m, s = ring depth, kc = K/128,
// spc = slices per CTA, ksplit = CTAs per cluster sharing the K range (their partial sums are exchanged
// through a [2][bmp][128] fp32 buffer).
__host__ __device__ inline SmemPlan smem_plan(int bmp, int s, int kc, int spc, int ksplit = 1) {
    SmemPlan p;
    p.stage_bytes = 2 * kTileBytes + bmp * 128;
    uint32_t o = s * p.stage_bytes;
    p.hq = o;        o += spc * bmp * 128;
    p.xs = o;        o += kc * bmp * 4;
    p.swg = o;       o += spc * kc * 4;
    p.swu = o;       o += spc * kc * 4;
    p.sw2 = o;       o += spc * kc * 4;
    o = (o + 15u) & ~15u;
    p.tokrow = o;    o += bmp * 4;
    p.topkw = o;     o += bmp * 4;
    p.tokscale = o;  o += spc * bmp * 4;
    p.amax = o;      o += bmp * 8;
    p.part = o;      o += ksplit > 1 ? 2 * bmp * 128 * 4 : 0;
    p.bars = o;      o += (2 * s + 2 * acc_buffers(bmp, 2) + 6) * 8;      // (room for the wider of the two 64-token shapes)
    p.misc = o;      o += 16;
    p.total = o;
    return p;
}

// PEERS: the tensor-parallel form whose epilogue adds into every rank's `out` (MoeParams::out_more).
// EW = epilogue warpgroups.  BMP = 64 exists in two shapes: EW = 2 (one CTA per SM, deep ring) and EW = 1, whose
// 256 threads and two-slot ring let two CTAs share an SM, so that one CTA's waits (accumulator hand-offs, the
// switch between the two phases) are filled by the other CTA's work.
template <int BMP, int SPC, int EW = (BMP >= 64 ? 2 : 1), bool PEERS = false>
__global__ void __launch_bounds__(128 * EW + 128, (BMP <= 32 || (BMP == 64 && EW == 1)) ? 2 : 1)
fused_moe_w8a8_up_down_sm100_kernel(const __grid_constant__ CUtensorMap tm_w,
                                    const __grid_constant__ CUtensorMap tm_w2, const MoeParams p) {
    constexpr int NEPI_WG = EW;                  // epilogue warpgroups; each owns BMP/NEPI_WG token columns
    constexpr int NC = BMP / NEPI_WG;
    constexpr int EPI_THREADS = 128 * NEPI_WG;
    constexpr int W_G0 = 4 * NEPI_WG, W_MMA0 = W_G0 + 2;   // control warpgroup: gather, gather, UMMA, UMMA
    constexpr int NB = acc_buffers(BMP, EW);     // accumulator buffers (chunks in flight between UMMA and epilogue)
    constexpr uint32_t TMEM_COLS = NB * 2 * BMP; // buffers x two accumulators x BMP columns
    static_assert(BMP == 16 || BMP == 32 || BMP == 64 || BMP == 128, "padded block_m");
    static_assert(SPC == 1 || SPC == 2, "slices per CTA");

    // With ksplit > 1 the launch uses clusters of ksplit consecutive CTAs that share one (block, slice):
    // each takes a contiguous part of the K chunks of the up-projection, the partial sums are exchanged
    // through distributed shared memory, and each then takes a part of the hidden tiles of the
    // down-projection.  This is what lets a handful of active experts (small batches) use all SMs.
    const int ks = p.ksplit;
    const int crank = ks > 1 ? static_cast<int>(cluster_ctarank()) : 0;
    const int unit = blockIdx.x / ks;
    const int ngroups = (p.N >> 8) / SPC;
    const int mblock = unit / ngroups;
    const int slice0 = (unit - mblock * ngroups) * SPC;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Everything whose address is known at entry is requested here, before the early exit and the set-up work
    // (barriers, TMEM, cluster sync), whose time then overlaps the latency of these loads: the schedule's length,
    // this block's expert (in bounds: the launcher starts no more blocks than expert_ids has entries) and the
    // sorted ids this thread will need - a gather thread those of its rows, an epilogue thread that of one token
    // column.  What depends on them (token rows, token scales, routing weights, block scales) follows after set-up.
    constexpr int PRE = BMP / 8;
    int pid_pre[PRE];
    int expert;
    griddep_wait();      // the schedule, the activations and the cleared `out` may come from the kernel just before
    griddep_launch_dependents();   // an exchange kernel behind this launch may be scheduled; it waits for our completion
    {
        const int npad_raw = ld_global_nc_s32(p.num_tokens_post_padded);
        const int expert_raw = ld_global_nc_s32(p.expert_ids + mblock);
        const bool gather_role = warp >= 4 * EW && warp < 4 * EW + 2;
        const int first = gather_role ? ((threadIdx.x - 4 * EW * 32) >> 3) : (threadIdx.x % BMP);
#pragma unroll
        for (int i = 0; i < PRE; ++i) {
            const int row = first + 8 * i;
            const int idx = mblock * p.block_m + row;
            pid_pre[i] = -1;
            if ((gather_role || i == 0) && warp < 4 * EW + 2 && row < p.block_m && idx < p.sorted_num)
                pid_pre[i] = ld_global_nc_s32(p.sorted_token_ids + idx);
        }
        const int npad = min(npad_raw, p.sorted_num);
        if (mblock * p.block_m >= npad) return;          // block beyond the padded schedule (reference :678)
        if (expert_raw < 0 || expert_raw >= p.E) return; // (a whole cluster leaves together: same block)
        expert = expert_raw;
    }

    const int KC = p.K >> 7;                         // 128-deep K chunks of the up-projection
    const int kc_begin = crank * KC / ks, kc_end = (crank + 1) * KC / ks;       // this CTA's K chunks
    const int nd_all = SPC == 1 ? (KC + 1) >> 1 : KC;
    const int jt_begin = crank * nd_all / ks;                                   // this CTA's down iterations
    const int UPI = SPC * (kc_end - kc_begin);       // up-projection iterations (slice-major)
    const int ND = (crank + 1) * nd_all / ks - jt_begin;                        // down-projection iterations
    const int NIT = UPI + ND;
    const int S = p.stages;

    // The operand tiles need 1024-byte alignment (128-byte swizzle atoms).  The dynamic shared memory
    // window is declared with that alignment; should a toolchain ever place it differently, the CTA
    // reports it and returns instead of computing on mis-swizzled tiles.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (smem_u32(smem_raw) & 1023u) {
        if (threadIdx.x == 0) atomicCAS(&p.status->code, ST_OK, ST_SMEM_MISALIGNED);
        return;
    }
    const SmemPlan L = smem_plan(BMP, S, KC, SPC, ks);
    uint8_t* hq = smem + L.hq;                                        // fp8 intermediate [SPC][BMP][128], swizzled
    float* xs = reinterpret_cast<float*>(smem + L.xs);                // [KC][BMP] token scales
    float* swg = reinterpret_cast<float*>(smem + L.swg);              // [SPC][KC] gate block scales
    float* swu = reinterpret_cast<float*>(smem + L.swu);              // [SPC][KC] up block scales
    float* sw2 = reinterpret_cast<float*>(smem + L.sw2);              // [SPC][KC] w2 block scales per 128 hidden rows
    int* tokrow = reinterpret_cast<int*>(smem + L.tokrow);            // [BMP] row of x/out, or M if padding
    float* topkw = reinterpret_cast<float*>(smem + L.topkw);          // [BMP]
    float* tokscale = reinterpret_cast<float*>(smem + L.tokscale);    // [SPC][BMP] s_h * topk_weight * scaling
    uint16_t* amax_part = reinterpret_cast<uint16_t*>(smem + L.amax); // [BMP][4] per-warp |h| maxima: |h| is a bf16 value, so the upper half of its fp32 pattern is exact
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);      // slot filled: TMA bytes + 64 gather threads
    uint64_t* empty = full + S;                                       // slot free again
    uint64_t* acc_full = empty + S;
    uint64_t* acc_empty = acc_full + NB;
    uint64_t* h_ready = acc_empty + NB;
    uint64_t* xchg = h_ready + 1;                                     // [2] amax exchange inside an epilogue warpgroup
    uint64_t* peer_ready = xchg + 2;                                  // every CTA of the cluster has published its partial sums
    uint64_t* peer_done = peer_ready + 1;                             // every CTA of the cluster has finished reading ours
    uint64_t* xsync = peer_done + 1;                                  // all epilogue warps of this CTA (bounded stand-in for bar.sync)
    float* part = reinterpret_cast<float*>(smem + L.part);            // [2][BMP][128] this CTA's partial gate / up sums
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc + 4);
    volatile int* issue_turn = reinterpret_cast<volatile int*>(smem + L.misc + 8);   // chunks whose operands have been waited for

    if (threadIdx.x == W_G0 * 32) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1 + 64);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < NB; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4 * NEPI_WG);
        }
        mbar_init(h_ready, 1);
        mbar_init(&xchg[0], 4);
        mbar_init(&xchg[1], 4);
        mbar_init(peer_ready, ks);
        mbar_init(peer_done, ks);
        mbar_init(xsync, 4 * NEPI_WG);
        *abort_flag = 0;
        *issue_turn = 0;
        fence_mbar_init();
    }
    if (warp == W_MMA0) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (ks > 1) cluster_sync_all();      // no CTA may signal a peer's barriers before that peer has initialised them

    if (warp >= W_G0) {
    // ====================================================================== control warpgroup
    // The widest variant keeps 2 x 64 accumulators per epilogue thread: it moves registers from this
    // warpgroup to the two epilogue warpgroups.
    if constexpr (NC >= 64) setmaxnreg_dec<64>();
    if (warp >= W_MMA0) {
        // ------------------------------------------------------------------ UMMA issuers (even / odd chunks)
        if (lane == 0) {
            const int pw = warp - W_MMA0;                                   // chunk parity = TMEM buffer
            constexpr uint32_t idesc = umma_idesc_e4m3(128, BMP);
            const uint32_t st0 = smem_u32(smem);
            // Descriptors advance with the ring slot: only the 14-bit start-address field changes.
            const uint32_t dstep = L.stage_bytes >> 4;
            const uint64_t a0_up0 = umma_desc_sw128(st0, 2048u);            // 8 gate rows of every 16
            const uint64_t a1_up0 = umma_desc_sw128(st0 + 1024u, 2048u);    // 8 up rows of every 16
            const uint64_t x_up0 = umma_desc_sw128(st0 + 2 * kTileBytes);   // gathered token rows
            const uint64_t a0_dn0 = umma_desc_sw128(st0);                   // first w2 tile of the slot
            const uint64_t a1_dn0 = umma_desc_sw128(st0 + kTileBytes);      // second w2 tile of the slot
            const uint64_t h0 = umma_desc_sw128(smem_u32(hq));
            const uint64_t h1 = umma_desc_sw128(smem_u32(hq + (SPC - 1) * BMP * 128));
            // Two issuers take alternate chunks.  A parity wait can only tell "this phase" from "the one
            // before", so the second issuer may start on chunk 1 only when chunk 1 is the first fill of
            // its slot: with a one-slot ring the first issuer takes every chunk.
            const int step = S > 1 ? 2 : 1;
            int s = pw % S;
            uint32_t ph = 0;
            bool h_waited = false;
            for (int it = pw; it < NIT && pw < step; it += step) {
                const int b = it & (NB - 1);                                // TMEM buffer of this chunk
                const uint32_t aph = (it / NB) & 1;
                const uint32_t d0 = tmem_base + b * 2 * BMP;
                const bool up = it < UPI;
                if (!up && !h_waited) {
                    if (!mbar_wait(h_ready, 0, abort_flag, p.status, 20, it)) break;
                    h_waited = true;
                }
                if (!mbar_wait(&acc_empty[b], aph ^ 1, abort_flag, p.status, 21, it)) break;
                // The two issuers wait for their operands in chunk order.  A parity wait is only meaningful while
                // the waiter is at most one phase ahead of the barrier: waiting for fill n of a slot presumes that
                // fill n-1 has completed.  With an odd ring depth fill n-1 belongs to the other issuer's chunk
                // it - S, and with NB accumulator buffers this issuer may be NB chunks ahead of the epilogue, i.e.
                // further ahead of the other issuer than the ring is deep.
                if (step == 2) {
                    const long long t0 = clock64();
                    bool turn_ok = true;
                    while (*issue_turn < it) {
                        if (*abort_flag) { turn_ok = false; break; }
                        if (clock64() - t0 > kWaitLimitCycles) {
                            *abort_flag = 1;
                            if (atomicCAS(&p.status->code, ST_OK, ST_WAIT_TIMEOUT) == ST_OK) {
                                p.status->block = blockIdx.x;
                                p.status->where = 23;
                                p.status->iter = it;
                            }
                            turn_ok = false;
                            break;
                        }
                    }
                    if (!turn_ok) break;
                }
                if (!mbar_wait(&full[s], ph, abort_flag, p.status, 22, it)) break;
                *issue_turn = it + 1;
                fence_proxy_async_smem();      // token rows were written by cp.async, the UMMA reads them through the async proxy
                tc_fence_after();
                const uint64_t off = static_cast<uint64_t>(s * dstep);
                if (up) {
                    umma_f8_chunk2(d0, d0 + BMP, a0_up0 + off, a1_up0 + off, x_up0 + off, x_up0 + off, idesc);
                } else if (SPC == 2) {
                    umma_f8_chunk2(d0, d0 + BMP, a0_dn0 + off, a1_dn0 + off, h0, h1, idesc);
                } else if (2 * (jt_begin + it - UPI) + 1 < KC) {
                    umma_f8_chunk2(d0, d0 + BMP, a0_dn0 + off, a1_dn0 + off, h0, h0, idesc);
                } else {
                    umma_f8_chunk1(d0, a0_dn0 + off, h0, idesc);
                }
                // Two commits per chunk: the accumulators are complete (for the epilogue), and the MMAs have
                // finished reading the ring slot (for the producers, who need not wait for the epilogue).
                umma_commit(&acc_full[b]);
                umma_commit(&empty[s]);
                s += step;
                while (s >= S) { s -= S; ph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ token-row gather (2 warps) + weight TMA
        constexpr int PIECES = BMP / 8;             // 16-byte pieces per thread per chunk
        const int gtid = threadIdx.x - W_G0 * 32;   // 0..63
        const bool tma_thread = gtid == 0;
        const int row0 = gtid >> 3, ch = gtid & 7;
        uint32_t src16[PIECES];                     // (row * K) / 16, or 0xFFFFFFFF for a padding row
        static_assert(PIECES == PRE, "one preloaded id per gathered row");
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int pid = pid_pre[i];             // requested at kernel entry; -1 for rows past the block
            src16[i] = 0xFFFFFFFFu;
            if (pid >= 0 && pid < p.M * p.top_k)
                src16[i] = static_cast<uint32_t>((static_cast<size_t>(pid / p.top_k) * p.K) >> 4);
        }
        if (tma_thread) {
            prefetch_tmap(&tm_w);
            prefetch_tmap(&tm_w2);
        }
        const uint32_t dst0 = row0 * 128 + ((ch ^ (row0 & 7)) << 4);   // + i*1024 for piece i (row & 7 unchanged)
        bool ok = true;
        int s = 0;                                  // ring slot being filled
        uint32_t ph = 0;
        int kc = kc_begin, sl = 0;
        for (int it = 0; it < UPI; ++it) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 30, it)) { ok = false; break; }
            uint8_t* st = smem + s * L.stage_bytes;
            if (tma_thread) {
                mbar_arrive_expect_tx(&full[s], 2 * kTileBytes);
                // 256 interleaved rows (128 gate + 128 up) of slice (slice0 + sl) x 128 bytes of K chunk kc
                tma_load_3d(st, &tm_w, &full[s], kc * 128, (slice0 + sl) * 256, expert);
            }
            const uint32_t base = smem_u32(st + 2 * kTileBytes) + dst0;
            const uint8_t* col = p.x + kc * 128 + ch * 16;
#pragma unroll
            for (int i = 0; i < PIECES; ++i) {
                const bool v = src16[i] != 0xFFFFFFFFu;
                const uint8_t* src = v ? col + (static_cast<size_t>(src16[i]) << 4) : p.x;
                cp_async_16(base + i * 1024, src, v ? 16u : 0u);
            }
            cp_async_mbar_arrive_noinc(&full[s]);      // arrives when this thread's copies have landed
            if (++s == S) { s = 0; ph ^= 1; }
            if (++kc == kc_end) { kc = kc_begin; ++sl; }
        }
        cp_async_wait_all();                        // nothing of this thread may still be in flight at exit
        if (tma_thread && ok) {
            // down phase: this thread keeps feeding w2 tiles; there is no token gather any more, so it
            // also stands in for the 64 gather threads on the slot's barrier
            for (int jl = 0; jl < ND; ++jl) {
                const int it = UPI + jl;
                const int jt = jt_begin + jl;
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 10, it)) break;
                uint8_t* st = smem + s * L.stage_bytes;
                mbar_arrive_expect_tx(&full[s], 2 * kTileBytes);
                if (SPC == 1) {   // hidden rows [2jt*128, +256) of the slice's 128 columns; rows past K arrive as zeros
                    tma_load_3d(st, &tm_w2, &full[s], slice0 * 128, (2 * jt) * 128, expert);
                    tma_load_3d(st + kTileBytes, &tm_w2, &full[s], slice0 * 128, (2 * jt + 1) * 128, expert);
                } else {          // hidden rows [jt*128, +128) for each of the two slices
                    tma_load_3d(st, &tm_w2, &full[s], slice0 * 128, jt * 128, expert);
                    tma_load_3d(st + kTileBytes, &tm_w2, &full[s], (slice0 + 1) * 128, jt * 128, expert);
                }
                mbar_arrive_n(&full[s], 64);
                if (++s == S) { s = 0; ph ^= 1; }
            }
        }
    }
    } else {
        // ====================================================================== epilogue warpgroups
        if constexpr (NC >= 64) setmaxnreg_inc<(EW == 1 ? 192 : 216)>();
        const int q = warp & 3;              // TMEM lane quarter this warp may read
        const int hh = warp >> 2;            // which part of the token columns
        const int r = q * 32 + lane;         // weight row inside the tile = TMEM lane
        const int etid = threadIdx.x;
        const int mtk = p.M * p.top_k;
        // One token column per thread (column etid % BMP; its sorted id was requested at kernel entry): its row, its
        // routing weight, and its token scales for the K chunks etid / BMP, + EPI_THREADS / BMP, ...  No thread needs
        // another thread's result here, so one barrier publishes everything.
        {
            const int j = etid % BMP;
            const int pid = pid_pre[0];
            const bool live = pid >= 0 && pid < mtk;
            const int row = live ? pid / p.top_k : p.M;          // reference :757
            if (etid < BMP) {
                tokrow[j] = row;
                topkw[j] = live ? p.topk_weights[pid] : 0.f;     // reference :761
            }
            const float* xs_row = p.x_scale + static_cast<size_t>(live ? row : 0) * KC;
            for (int c = etid / BMP; c < KC; c += EPI_THREADS / BMP) xs[c * BMP + j] = live ? xs_row[c] : 0.f;
        }
        {
            const int nsr = p.N >> 7;                         // scale rows per expert in w_scale
            const int isl = p.N >> 8;                         // 128-column slices of the intermediate dim
            for (int i = etid; i < SPC * KC; i += EPI_THREADS) {
                const int sl = i / KC, c = i - sl * KC;
                const float* ws = p.w_scale + (static_cast<size_t>(expert) * nsr + 2 * (slice0 + sl)) * KC;
                swg[i] = ws[c];                               // interleave slot 0 = gate (reference :919-925)
                swu[i] = ws[KC + c];                          // slot 1 = up
                sw2[i] = p.w2_scale[(static_cast<size_t>(expert) * KC + c) * isl + slice0 + sl];
            }
        }
        named_bar_sync(1, EPI_THREADS);
        int nhi = 0;
        for (int j = 0; j < BMP; ++j)
            if (tokrow[j] < p.M) nhi = j + 1;
        const int my_ncols = min(max(nhi - hh * NC, 0), NC);
        const bool few = nhi <= 2 && NEPI_WG == 1;   // at most two live columns in the whole block (CTA-uniform)

        float accg[NC], accu[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j) accg[j] = accu[j] = 0.f;

        // Factor of column j for the output = s_h * topk weight * scaling (reference :997-1003) and its row
        // in `out` (M = padding): in registers for the narrow single-slice variants, else in shared memory.
        constexpr bool kFactorsInRegs = (NC <= 16) && (SPC == 1);
        constexpr int NF = kFactorsInRegs ? NC : 2;
        int rowj[NF];
        float facj[NF];

        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hh * NC;
        bool ok = true;
        int kc = kc_begin, sl = 0;
        uint32_t xph = 0;
        // ---- up-projection: promote each K chunk with its scales (reference :915-933)
        for (int it = 0; it < UPI && ok; ++it) {
            const int b = it & (NB - 1);
            const uint32_t aph = (it / NB) & 1;
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 40, it)) { ok = false; break; }
            tc_fence_after();
            const float sg = swg[sl * KC + kc], su = swu[sl * KC + kc];
            const uint32_t tb = tlane + b * 2 * BMP;
#pragma unroll
            for (int c0 = 0; c0 < NC; c0 += 16) {
                if (c0 < my_ncols) {
                    uint32_t vg[16], vu[16];
                    tmem_ld16(tb + c0, vg);
                    tmem_ld16(tb + BMP + c0, vu);
                    tmem_ld_wait();
                    const float4* sx4 = reinterpret_cast<const float4*>(xs + kc * BMP + hh * NC + c0);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        const float4 sx = sx4[jj];
                        const float f[4] = {sx.x, sx.y, sx.z, sx.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = c0 + 4 * jj + e;
                            accg[j] = fmaf(__uint_as_float(vg[4 * jj + e]), sg * f[e], accg[j]);
                            accu[j] = fmaf(__uint_as_float(vu[4 * jj + e]), su * f[e], accu[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);

            if (++kc == kc_end) {
                if (ks > 1) {
                    // ---- K-split: every CTA of the cluster holds partial sums over its own K chunks.  Publish
                    // ours in shared memory, tell every peer, wait (bounded) until all peers have published,
                    // then add up all partial sums straight out of the peers' shared memory.  All CTAs end up
                    // with the same totals and each re-quantises the intermediate for itself.
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        if (j < my_ncols) {
                            part[(hh * NC + j) * 128 + r] = accg[j];
                            part[(BMP + hh * NC + j) * 128 + r] = accu[j];
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xsync);
                    if (!mbar_wait(xsync, 0, abort_flag, p.status, 45, it)) ok = false;
                    if (etid < ks) mbar_arrive_cluster(mapa_shared(smem_u32(peer_ready), etid));
                    if (!mbar_wait_cluster(peer_ready, 0, abort_flag, p.status, 43, it)) ok = false;
                    // After a wait that ran out, a peer may have left already: no peer's shared memory is read from
                    // here on (this CTA is unwinding; its sums are not used any more).
                    // A load from a peer's shared memory takes several hundred cycles, and a thread that adds each value
                    // as it arrives waits that long per value: all loads of a column (2 x up to 8 peers) are issued
                    // before the first addition.
                    uint32_t peer_part[8];
#pragma unroll
                    for (int peer = 0; peer < 8; ++peer) peer_part[peer] = mapa_shared(smem_u32(part), peer < ks ? peer : 0);
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        if (j < my_ncols && ok) {
                            float vg[8], vu[8];
#pragma unroll
                            for (int peer = 0; peer < 8; ++peer) {
                                vg[peer] = 0.f;
                                vu[peer] = 0.f;
                                if (peer < ks) {
                                    vg[peer] = ld_dsmem_f32(peer_part[peer] + ((hh * NC + j) * 128 + r) * 4);
                                    vu[peer] = ld_dsmem_f32(peer_part[peer] + ((BMP + hh * NC + j) * 128 + r) * 4);
                                }
                            }
                            float g = 0.f, u = 0.f;
#pragma unroll
                            for (int peer = 0; peer < 8; ++peer) {      // in peer order: every CTA of the cluster gets the same sums
                                g += vg[peer];
                                u += vu[peer];
                            }
                            accg[j] = g;
                            accu[j] = u;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xsync);       // every thread of this CTA is done reading the peers
                    if (!mbar_wait(xsync, 1, abort_flag, p.status, 46, it)) ok = false;
                    if (etid < ks && ok) mbar_arrive_cluster(mapa_shared(smem_u32(peer_done), etid));
                }
                // ---- end of a slice: SwiGLU, per-token amax over the slice's 128 columns, fp8 re-quantisation
                //      (reference :936-1005; h stays in registers, only the fp8 tile goes to shared memory)
                // Blocks of one or two tokens are the rule at small batch: then only the first two columns are
                // worked on and the other rows of the intermediate tile are written as zeros.
                auto swiglu_quant = [&](auto live_cols) {
                    constexpr int NJ = decltype(live_cols)::value;
#pragma unroll
                    for (int j = 0; j < NJ; ++j) {
                        const float g = bf16_round(accg[j]);
                        const float u = bf16_round(accu[j]);
                        const float h = bf16_round(__fdividef(g, 1.0f + __expf(-g)) * u);
                        accg[j] = h;
                        const uint32_t a = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(h)));
                        if (lane == 0) amax_part[(hh * NC + j) * 4 + q] = static_cast<uint16_t>(a >> 16);
                    }
                    // exchange of the four warps' maxima through a (bounded) mbarrier rather than bar.sync, so
                    // that a warp that gave up on a wait can never leave the others parked at a hardware barrier
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&xchg[hh]);
                    if (!mbar_wait(&xchg[hh], xph, abort_flag, p.status, 42, it)) ok = false;
                    xph ^= 1;
                    uint8_t* hq_sl = hq + sl * BMP * 128;
#pragma unroll
                    for (int j = 0; j < NC; ++j) {
                        const int col = hh * NC + j;
                        const uint32_t hoff = col * 128 + ((((r >> 4) ^ (col & 7)) << 4) | (r & 15));
                        if (j < NJ) {
                            const uint2 pm = *reinterpret_cast<const uint2*>(amax_part + col * 4);
                            const float amax = __uint_as_float(
                                max(max(pm.x & 0xFFFFu, pm.x >> 16), max(pm.y & 0xFFFFu, pm.y >> 16)) << 16);
                            const float s_h = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
                            const float qv = fminf(fmaxf(__fdividef(accg[j], s_h), -448.0f), 448.0f);
                            hq_sl[hoff] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3));
                            const float fac = s_h * topkw[col] * p.scaling;
                            if constexpr (kFactorsInRegs) {
                                facj[j] = fac;
                                rowj[j] = tokrow[col];
                            } else {
                                if (r == 0) tokscale[sl * BMP + col] = fac;
                            }
                        } else {
                            hq_sl[hoff] = 0;
                            if constexpr (kFactorsInRegs) {
                                facj[j] = 0.f;
                                rowj[j] = p.M;
                            } else {
                                if (r == 0) tokscale[sl * BMP + col] = 0.f;
                            }
                        }
                        accg[j] = 0.f;
                        accu[j] = 0.f;
                    }
                };
                if (few) swiglu_quant(std::integral_constant<int, (NC < 2 ? NC : 2)>{});
                else swiglu_quant(std::integral_constant<int, NC>{});
                fence_proxy_async_smem();
                if constexpr (SPC == 2) {
                    // amax_part is rewritten at the end of the next slice, and with several accumulator buffers a warp
                    // may get there before another has read this slice's maxima: a second round of the same barrier
                    if (sl == 0) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&xchg[hh]);
                        if (!mbar_wait(&xchg[hh], xph, abort_flag, p.status, 47, it)) ok = false;
                        xph ^= 1;
                    }
                }
                kc = kc_begin;
                ++sl;
            }
        }
        named_bar_sync(1, EPI_THREADS);
        if (etid == 0) mbar_arrive(h_ready);

        // ---- down-projection epilogue: scale, pair adjacent hidden columns, bf16x2 reduce into out
        //      (reference :1052-1094 goes through stmatrix + per-row bulk reduce).
        // The accumulators are copied to registers and handed back to the MMA warps *before* any
        // reduction is issued: tcgen05.fence / mbarrier.arrive after a global reduction would wait for
        // L2 to acknowledge it, which would put an L2 round trip into every iteration.
        const bool odd = lane & 1;
        for (int jl = 0; jl < ND && ok; ++jl) {
            const int it = UPI + jl;
            const int jt = jt_begin + jl;            // hidden-tile pair (SPC = 1) / hidden tile (SPC = 2) of the whole layer
            const int b = it & (NB - 1);
            const uint32_t aph = (it / NB) & 1;
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 41, it)) { ok = false; break; }
            tc_fence_after();
            const bool two = SPC == 2 || (2 * jt + 1 < KC);
            const uint32_t tb = tlane + b * 2 * BMP;
            uint32_t v0[NC], v1[NC];
#pragma unroll
            for (int c0 = 0; c0 < NC; c0 += 16) {
                if (c0 < my_ncols) {
                    tmem_ld16(tb + c0, *reinterpret_cast<uint32_t(*)[16]>(&v0[c0]));
                    if (two) tmem_ld16(tb + BMP + c0, *reinterpret_cast<uint32_t(*)[16]>(&v1[c0]));
                }
            }
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_relaxed(&acc_empty[b]);

            if constexpr (SPC == 1) {
                // v0 / v1 = hidden tiles 2jt and 2jt+1 of the same slice
#pragma unroll
                for (int tt = 0; tt < 2; ++tt) {
                    if (tt == 0 || two) {
                        const int tile = 2 * jt + tt;
                        const float s2 = sw2[tile];
                        const size_t obase = static_cast<size_t>(tile) * 128 + (r & ~1);
                        // Straight-line over each live 16-column group (padding columns carry row == M and are
                        // masked at the reduction): per-pair branches would serialise this single warp.
#pragma unroll
                        for (int c0 = 0; c0 < NC; c0 += 16) {
                            if (c0 < my_ncols) {
#pragma unroll
                                for (int j = c0; j < c0 + 16; j += 2) {
                                    if (j >= 2 && few) break;      // one or two live columns: the first pair is all there is
                                    float f0, f1;
                                    int r0, r1;
                                    if constexpr (kFactorsInRegs) {
                                        f0 = facj[j]; f1 = facj[j + 1]; r0 = rowj[j]; r1 = rowj[j + 1];
                                    } else {
                                        const float2 ff = *reinterpret_cast<const float2*>(tokscale + hh * NC + j);
                                        const int2 rr = *reinterpret_cast<const int2*>(tokrow + hh * NC + j);
                                        f0 = ff.x; f1 = ff.y; r0 = rr.x; r1 = rr.y;
                                    }
                                    const float a = __uint_as_float(tt ? v1[j] : v0[j]) * (s2 * f0);
                                    const float bb = __uint_as_float(tt ? v1[j + 1] : v0[j + 1]) * (s2 * f1);
                                    const float recv = __shfl_xor_sync(0xFFFFFFFFu, odd ? a : bb, 1);
                                    const float lo = odd ? recv : a;
                                    const float hi = odd ? bb : recv;
                                    const int row = odd ? r1 : r0;
                                    red_out_all_ranks<PEERS>(p, obase + static_cast<size_t>(row) * p.K, lo, hi, row);
                                }
                            }
                        }
                    }
                }
            } else {
                // v0 / v1 = partial sums of hidden tile jt over slice 0 / slice 1: each has its own block scale
                // and its own per-token quantisation scale, so they are combined here, then reduced once
                const float s2a = sw2[jt], s2b = sw2[KC + jt];
                const size_t obase = static_cast<size_t>(jt) * 128 + (r & ~1);
#pragma unroll
                for (int c0 = 0; c0 < NC; c0 += 16) {
                    if (c0 < my_ncols) {
#pragma unroll
                        for (int j = c0; j < c0 + 16; j += 2) {
                            if (j >= 2 && few) break;
                            const float2 fa = *reinterpret_cast<const float2*>(tokscale + hh * NC + j);
                            const float2 fb = *reinterpret_cast<const float2*>(tokscale + BMP + hh * NC + j);
                            const int2 rr = *reinterpret_cast<const int2*>(tokrow + hh * NC + j);
                            const float a = fmaf(__uint_as_float(v0[j]), s2a * fa.x,
                                                 __uint_as_float(v1[j]) * (s2b * fb.x));
                            const float bb = fmaf(__uint_as_float(v0[j + 1]), s2a * fa.y,
                                                  __uint_as_float(v1[j + 1]) * (s2b * fb.y));
                            const float recv = __shfl_xor_sync(0xFFFFFFFFu, odd ? a : bb, 1);
                            const float lo = odd ? recv : a;
                            const float hi = odd ? bb : recv;
                            const int row = odd ? rr.y : rr.x;
                            red_out_all_ranks<PEERS>(p, obase + static_cast<size_t>(row) * p.K, lo, hi, row);
                        }
                    }
                }
            }
        }
        // our partial sums must stay readable until every peer of the cluster has read them
        if (ks > 1 && etid == 0) mbar_wait_cluster(peer_done, 0, abort_flag, p.status, 44, NIT);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace amoe
