// Token-major variant of the fused W8A8 MoE kernel for large blocks (64 < block_m <= 128).
//
// Same operator and same work decomposition as fused_moe_kernel.cuh (which replaces
// csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:654-1098), but with the operands the other
// way round: the block's tokens are the UMMA "M" operand (one token per TMEM lane, padded to 128) and
// the weight rows are the "N" operand (256 per instruction).  With a full block this runs the tensor
// pipe at its rated speed (an M=128, N=256, K=32 fp8 UMMA is compute-bound; the weight-major
// orientation is operand-fetch-bound at N <= 64), and everything the epilogue does becomes local to
// one thread = one token:
//   * scale promotion needs two scalars per chunk (token scale x gate / up block scale) instead of a
//     multiplication per column (reference :915-933);
//   * the interleaved gate/up rows arrive as interleaved accumulator columns (columns 16j..16j+7 gate,
//     16j+8..16j+15 up of the same intermediate columns), so SwiGLU needs no data movement
//     (reference :919-931, :945-946 obtains the same pairing inside a wgmma fragment);
//   * the fp8 intermediate is written as 16-byte vectors into the swizzled operand tile;
//   * each thread owns consecutive hidden columns of its token in the down-projection, so the
//     accumulation into `out` is done with 16-byte vector reductions (red.global.add.noftz.v4.bf16x2)
//     instead of one 4-byte reduction per pair of columns (reference :1085-1091 uses a 512-byte bulk
//     reduce per row).
//
// Ring slot: [256 weight rows x 128 B = 32 KB][128 token rows x 128 B = 16 KB]; slot contents as in
// fused_moe_kernel.cuh.  TMEM: up phase two buffers of 256 columns (one per K chunk in flight); down
// phase two buffers of 256 columns (SPC = 1: two hidden tiles; SPC = 2: the two slices' partial sums
// of one hidden tile, combined by the epilogue because each carries its own scales).
#pragma once

#include "fused_moe_kernel.cuh"

namespace amoe {

constexpr int kTmRows = 128;   // token rows of a block (TMEM lanes)
constexpr int kStgPitch = 144;                     // staging row pitch: 128 B + 16 B so that rows spread over the banks
constexpr int kStgWarpBytes = 32 * kStgPitch;      // one warp's staging tile
constexpr uint32_t kStgAliased = 0xFFFFFFFFu;      // SmemPlanTm::stage_out when the staging tiles alias the ring

struct SmemPlanTm {
    uint32_t stage_bytes, hq, stage_out, swg, swu, sw2, amaxx, xs, bars, misc, total;
};
__host__ __device__ inline SmemPlanTm smem_plan_tm(int s, int kc, int spc) {
    SmemPlanTm p;
    p.stage_bytes = 2 * kTileBytes + kTmRows * 128;
    uint32_t o = s * p.stage_bytes;
    p.hq = o;     o += spc * kTmRows * 128;
    // per epilogue warp a staging tile of 32 rows x 128 B (+16 B pitch padding) for the down phase; with three
    // or more ring slots these live in the slots' token-row tiles, which that phase does not use
    if (s >= 3) { p.stage_out = kStgAliased; } else { p.stage_out = o;  o += 8 * kStgWarpBytes; }
    p.swg = o;    o += spc * kc * 4;
    p.swu = o;    o += spc * kc * 4;
    p.sw2 = o;    o += spc * kc * 4;
    o = (o + 15u) & ~15u;
    p.amaxx = o;  o += 2 * kTmRows * 4;
    p.xs = o;     o += kc * kTmRows * 4;      // token scales [K chunk][token]
    p.bars = o;   o += (2 * s + 7) * 8;
    p.misc = o;   o += 16;
    p.total = o;
    return p;
}

__device__ __forceinline__ void red_add_v4_bf16x2_raw_if(__nv_bfloat16* addr, const uint4& w, bool pred) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %5, 0;\n\t"
        "@p red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};\n\t}"
        ::"l"(addr), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w), "r"(static_cast<uint32_t>(pred)));
}

constexpr int kTmThreads = 512;     // 2 epilogue warpgroups + control warpgroup + gather warpgroup
constexpr int kTmGatherWarps = 5;   // one warp of the control warpgroup + the gather warpgroup

template <int SPC>
__global__ void __launch_bounds__(kTmThreads, 1)
fused_moe_w8a8_up_down_sm100_tokmajor_kernel(const __grid_constant__ CUtensorMap tm_w,
                                             const __grid_constant__ CUtensorMap tm_w2, const MoeParams p) {
    constexpr int EPI_THREADS = 256;
    // control warpgroup: weight TMA, gather, UMMA (even chunks), UMMA (odd chunks); then four more gather warps.
    // One warp issues a 16-byte cp.async of 32 lanes only about every 100 cycles, whatever the addresses, and a
    // 128-row x 128-byte token tile takes 32 of them: five warps bring a tile in about as long as its UMMAs run.
    constexpr int W_TMA = 8, W_G0 = 9, W_MMA0 = 10, W_G1 = 12;
    constexpr int GATHER_THREADS = kTmGatherWarps * 32;
    constexpr uint32_t TMEM_COLS = 512;
    static_assert(SPC == 1 || SPC == 2, "slices per CTA");

    const int ngroups = (p.N >> 8) / SPC;
    const int mblock = blockIdx.x / ngroups;
    const int slice0 = (blockIdx.x - mblock * ngroups) * SPC;
    griddep_wait();      // the schedule, the activations and the cleared `out` may come from the kernel just before
    griddep_launch_dependents();   // a kernel behind this launch may be scheduled; it waits for our completion
    const int npad = min(p.num_tokens_post_padded[0], p.sorted_num);
    if (mblock * p.block_m >= npad) return;
    const int expert = p.expert_ids[mblock];
    if (expert < 0 || expert >= p.E) return;

    const int KC = p.K >> 7;
    const int UPI = SPC * KC;
    const int ND = SPC == 1 ? (KC + 1) >> 1 : KC;
    const int NIT = UPI + ND;
    const int S = p.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // The operand tiles need 1024-byte alignment (128-byte swizzle atoms).  The dynamic shared memory
    // window is declared with that alignment; should a toolchain ever place it differently, the CTA
    // reports it and returns instead of computing on mis-swizzled tiles.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (smem_u32(smem_raw) & 1023u) {
        if (threadIdx.x == 0) atomicCAS(&p.status->code, ST_OK, ST_SMEM_MISALIGNED);
        return;
    }
    const SmemPlanTm L = smem_plan_tm(S, KC, SPC);
    uint8_t* hq = smem + L.hq;                                        // fp8 intermediate [SPC][128][128], swizzled
    float* swg = reinterpret_cast<float*>(smem + L.swg);
    float* swu = reinterpret_cast<float*>(smem + L.swu);
    float* sw2 = reinterpret_cast<float*>(smem + L.sw2);
    uint32_t* amaxx = reinterpret_cast<uint32_t*>(smem + L.amaxx);    // [2][128] per-thread |h| maxima of each column half
    float* xs = reinterpret_cast<float*>(smem + L.xs);                // [KC][128] token scales (0 for padding rows)
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
    uint64_t* empty = full + S;
    uint64_t* acc_full = empty + S;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* h_ready = acc_empty + 2;
    uint64_t* xchg = h_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc + 4);
    volatile int* issue_turn = reinterpret_cast<volatile int*>(smem + L.misc + 8);   // iterations whose operands have been waited for

    if (threadIdx.x == W_TMA * 32) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 1 + GATHER_THREADS);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 8);
        }
        mbar_init(h_ready, 1);
        mbar_init(&xchg[0], 8);
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

    if (warp >= W_TMA) {
    // ====================================================================== control + gather warpgroups
    setmaxnreg_dec<40>();
    if (warp == W_MMA0 || warp == W_MMA0 + 1) {
        // ------------------------------------------------------------------ UMMA issuers (even / odd chunks)
        if (lane == 0) {
            const int pw = warp - W_MMA0;
            constexpr uint32_t idesc256 = umma_idesc_e4m3(128, 256);
            constexpr uint32_t idesc128 = umma_idesc_e4m3(128, 128);
            const uint32_t st0 = smem_u32(smem);
            const uint32_t dstep = L.stage_bytes >> 4;
            const uint64_t w_0 = umma_desc_sw128(st0);                      // 256 weight rows of the slot (N operand)
            const uint64_t w_1 = umma_desc_sw128(st0 + kTileBytes);         // its second 128 rows
            const uint64_t x_0 = umma_desc_sw128(st0 + 2 * kTileBytes);     // gathered token rows (M operand)
            const uint64_t h0 = umma_desc_sw128(smem_u32(hq));
            const uint64_t h1 = umma_desc_sw128(smem_u32(hq + (SPC - 1) * kTmRows * 128));
            const int step = S > 1 ? 2 : 1;      // see fused_moe_kernel.cuh: one issuer when the ring has one slot
            int s = pw % S;
            uint32_t ph = 0;
            bool h_waited = false;
            for (int it = pw; it < NIT && pw < step; it += step) {
                const int b = it & 1;
                const uint32_t aph = (it >> 1) & 1;
                const uint32_t d = tmem_base + b * 256;
                const bool up = it < UPI;
                if (!up && !h_waited) {
                    if (!mbar_wait(h_ready, 0, abort_flag, p.status, 20, it)) break;
                    h_waited = true;
                }
                if (!mbar_wait(&acc_empty[b], aph ^ 1, abort_flag, p.status, 21, it)) break;
                // The two issuers take their turns in iteration order.  A parity wait is only meaningful while
                // the waiter is at most one phase ahead of the barrier: waiting for fill n of a slot presumes
                // that fill n-1 has completed.  Fill n-1 belongs to iteration it-S, which with an odd ring depth
                // is the other issuer's; in the down phase the two warpgroups of the epilogue release the
                // accumulator buffers independently, so without the turn one issuer could get that far ahead.
                {
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
                    umma_f8_chunk1(d, x_0 + off, w_0 + off, idesc256);           // D[token, 256 interleaved w rows]
                } else if (SPC == 1) {
                    umma_f8_chunk1(d, h0, w_0 + off, idesc256);                  // D[token, 2 x 128 hidden rows]
                } else {
                    umma_f8_chunk2(d, d + 128, h0, h1, w_0 + off, w_1 + off, idesc128);   // per-slice partial sums
                }
                umma_commit(&acc_full[b]);
                umma_commit(&empty[s]);        // the ring slot is free once these MMAs have read it
                s += step;
                while (s >= S) { s -= S; ph ^= 1; }
            }
        }
    } else if (warp == W_TMA) {
        // ------------------------------------------------------------------ weight TMA (one thread)
        if (lane == 0) {
            prefetch_tmap(&tm_w);
            prefetch_tmap(&tm_w2);
            int s = 0;
            uint32_t ph = 0;
            int kc = 0, sl = 0;
            for (int it = 0; it < NIT; ++it) {
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 30, it)) break;
                uint8_t* st = smem + s * L.stage_bytes;
                mbar_arrive_expect_tx(&full[s], 2 * kTileBytes);
                if (it < UPI) {
                    tma_load_3d(st, &tm_w, &full[s], kc * 128, (slice0 + sl) * 256, expert);
                    if (++kc == KC) { kc = 0; ++sl; }
                } else {
                    // down phase: no token rows any more, so this thread also stands in for the gather threads
                    const int jt = it - UPI;
                    if (SPC == 1) {
                        tma_load_3d(st, &tm_w2, &full[s], slice0 * 128, (2 * jt) * 128, expert);
                        tma_load_3d(st + kTileBytes, &tm_w2, &full[s], slice0 * 128, (2 * jt + 1) * 128, expert);
                    } else {
                        tma_load_3d(st, &tm_w2, &full[s], slice0 * 128, jt * 128, expert);
                        tma_load_3d(st + kTileBytes, &tm_w2, &full[s], (slice0 + 1) * 128, jt * 128, expert);
                    }
                    mbar_arrive_n(&full[s], GATHER_THREADS);
                }
                if (++s == S) { s = 0; ph ^= 1; }
            }
        }
    } else {
        // ------------------------------------------------------------------ token-row gather (5 warps)
        // Row group j (4 token rows x 128 B, one cp.async of the warp) belongs to gather warp j % 5: 7 groups for
        // the first two warps, 6 for the others.  Lane l copies 16-byte piece l & 7 of row 4j + (l >> 3).
        constexpr int GROUPS = kTmRows / 4;
        constexpr int MAXG = (GROUPS + kTmGatherWarps - 1) / kTmGatherWarps;
        const int gw = warp == W_G0 ? 0 : warp - W_G1 + 1;
        const int ch = lane & 7;
        uint32_t src16[MAXG];
        uint32_t dst[MAXG];
#pragma unroll
        for (int i = 0; i < MAXG; ++i) {
            const int grp = gw + kTmGatherWarps * i;
            const int row = 4 * grp + (lane >> 3);
            const int idx = mblock * p.block_m + row;
            src16[i] = 0xFFFFFFFFu;
            dst[i] = 0xFFFFFFFFu;                  // no such group for this warp
            if (grp < GROUPS) {
                dst[i] = row * 128 + ((ch ^ (row & 7)) << 4);
                if (row < p.block_m && idx < p.sorted_num) {
                    const int pid = p.sorted_token_ids[idx];
                    if (pid >= 0 && pid < p.M * p.top_k)
                        src16[i] = static_cast<uint32_t>((static_cast<size_t>(pid / p.top_k) * p.K) >> 4);
                }
            }
        }
        int s = 0;
        uint32_t ph = 0;
        int kc = 0;
        for (int it = 0; it < UPI; ++it) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 31, it)) break;
            const uint32_t base = smem_u32(smem + s * L.stage_bytes + 2 * kTileBytes);
            const uint8_t* col = p.x + kc * 128 + ch * 16;
#pragma unroll
            for (int i = 0; i < MAXG; ++i) {
                if (dst[i] != 0xFFFFFFFFu) {
                    const bool v = src16[i] != 0xFFFFFFFFu;
                    const uint8_t* src = v ? col + (static_cast<size_t>(src16[i]) << 4) : p.x;
                    cp_async_16(base + dst[i], src, v ? 16u : 0u);
                }
            }
            cp_async_mbar_arrive_noinc(&full[s]);      // arrives when this thread's copies have landed
            if (++s == S) { s = 0; ph ^= 1; }
            if (++kc == KC) kc = 0;
        }
        cp_async_wait_all();                        // nothing of this thread may still be in flight at exit
    }
    } else {
        // ====================================================================== epilogue: thread = token
        setmaxnreg_inc<216>();
        const int q = warp & 3;              // TMEM lane quarter
        const int hh = warp >> 2;            // column half handled by this warpgroup
        const int t = q * 32 + lane;         // token slot of the block = TMEM lane
        const int etid = threadIdx.x;
        int row = p.M;
        float tw = 0.f;
        {
            const int idx = mblock * p.block_m + t;
            if (t < p.block_m && idx < p.sorted_num) {
                const int pid = p.sorted_token_ids[idx];
                if (pid >= 0 && pid < p.M * p.top_k) {
                    row = pid / p.top_k;             // reference :757
                    tw = p.topk_weights[pid];        // reference :761
                }
            }
        }
        const bool valid = row < p.M;
        const bool warp_valid = __any_sync(0xFFFFFFFFu, valid);
        {
            const int nsr = p.N >> 7;
            const int isl = p.N >> 8;
            for (int i = etid; i < SPC * KC; i += EPI_THREADS) {
                const int sl = i / KC, c = i - sl * KC;
                const float* ws = p.w_scale + (static_cast<size_t>(expert) * nsr + 2 * (slice0 + sl)) * KC;
                swg[i] = ws[c];
                swu[i] = ws[KC + c];
                sw2[i] = p.w2_scale[(static_cast<size_t>(expert) * KC + c) * isl + slice0 + sl];
            }
        }
        named_bar_sync(1, EPI_THREADS);

        // Token scales go to shared memory once (each warpgroup fetches one half of the K chunks of its tokens): the
        // chunk loop then holds no global load, whose latency a releasing hand-off would have to wait out.
        {
            const float* xs_row = p.x_scale + static_cast<size_t>(valid ? row : 0) * KC;
            const int c_begin = hh * (KC >> 1), c_end = hh == 0 ? (KC >> 1) : KC;
            for (int c = c_begin; c < c_end; ++c) xs[c * kTmRows + t] = valid ? xs_row[c] : 0.f;
        }
        named_bar_sync(1, EPI_THREADS);

        // accumulators of this token: 8 groups of (8 gate, 8 up) columns = 64 intermediate columns
        float acc[128];
#pragma unroll
        for (int j = 0; j < 128; ++j) acc[j] = 0.f;
        float fac[SPC];                      // s_h * topk weight * scaling per slice (reference :997-1003)

        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
        bool ok = true;
        uint32_t xph = 0;
        // ---- up-projection: promote each K chunk with its scales (reference :915-933).  The chunk loop is kept
        // small and contiguous (the slice-end code follows it instead of sitting inside it).
        for (int sl = 0, it = 0; sl < SPC && ok; ++sl) {
        for (int kc = 0; kc < KC; ++kc, ++it) {
            const int b = it & 1;
            const uint32_t aph = (it >> 1) & 1;
            const float sx = xs[kc * kTmRows + t];
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 40, it)) { ok = false; break; }
            tc_fence_after();
            if (warp_valid) {
                const float fg = sx * swg[sl * KC + kc], fu = sx * swu[sl * KC + kc];
                const uint32_t tb = tlane + b * 256 + hh * 128;
#pragma unroll
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t va[16], vb[16];
                    tmem_ld16(tb + c0, va);
                    tmem_ld16(tb + c0 + 16, vb);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        acc[c0 + e] = fmaf(__uint_as_float(va[e]), fg, acc[c0 + e]);
                        acc[c0 + 8 + e] = fmaf(__uint_as_float(va[8 + e]), fu, acc[c0 + 8 + e]);
                        acc[c0 + 16 + e] = fmaf(__uint_as_float(vb[e]), fg, acc[c0 + 16 + e]);
                        acc[c0 + 24 + e] = fmaf(__uint_as_float(vb[8 + e]), fu, acc[c0 + 24 + e]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_relaxed(&acc_empty[b]);
        }
            if (ok) {
                // ---- end of a slice: SwiGLU, amax over the slice's 128 columns (64 here + 64 in the partner
                //      warpgroup's thread of the same token), fp8 re-quantisation (reference :936-1005)
                float amax = 0.f;
#pragma unroll
                for (int g8 = 0; g8 < 8; ++g8) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float g = bf16_round(acc[16 * g8 + e]);
                        const float u = bf16_round(acc[16 * g8 + 8 + e]);
                        const float h = bf16_round(__fdividef(g, 1.0f + __expf(-g)) * u);
                        acc[16 * g8 + e] = h;
                        amax = fmaxf(amax, fabsf(h));
                    }
                }
                amaxx[hh * kTmRows + t] = __float_as_uint(amax);
                __syncwarp();
                if (lane == 0) mbar_arrive(&xchg[0]);
                if (!mbar_wait(&xchg[0], xph, abort_flag, p.status, 42, sl)) ok = false;
                xph ^= 1;
                amax = fmaxf(amax, __uint_as_float(amaxx[(hh ^ 1) * kTmRows + t]));
                const float s_h = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
                uint8_t* hrow = hq + sl * kTmRows * 128 + t * 128;
#pragma unroll
                for (int i = 0; i < 4; ++i) {             // 16 intermediate columns = 16 bytes per store
                    uint32_t w4[4];
#pragma unroll
                    for (int k2 = 0; k2 < 4; ++k2) {
                        const int base = 16 * (2 * i + (k2 >> 1)) + 4 * (k2 & 1);
                        float qv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            qv[e] = fminf(fmaxf(__fdividef(acc[base + e], s_h), -448.0f), 448.0f);
                        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(qv[0], qv[1]), __NV_SATFINITE, __NV_E4M3);
                        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(qv[2], qv[3]), __NV_SATFINITE, __NV_E4M3);
                        w4[k2] = lo | (hi << 16);
                    }
                    const int chunk = (hh * 4 + i) ^ (t & 7);
                    *reinterpret_cast<uint4*>(hrow + chunk * 16) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                }
                fac[sl] = s_h * tw * p.scaling;
#pragma unroll
                for (int j = 0; j < 128; ++j) acc[j] = 0.f;
                fence_proxy_async_smem();
            }
        }
        named_bar_sync(1, EPI_THREADS);
        if (etid == 0) mbar_arrive(h_ready);

        // ---- down-projection epilogue (reference :1052-1094).  A thread holds 64 consecutive hidden columns
        // of its own token, but 32 lanes reducing into 32 different rows would make every reduction
        // instruction 32 separate half-sector requests.  So each warp turns its 32 x 128-byte block around in
        // a private staging tile: afterwards one instruction covers four token rows x 128 contiguous bytes
        // (whole lines), which is what the reduction path of the memory system handles best.  (Handing each
        // row to the bulk-copy engine instead - cp.reduce.async.bulk, 128 B per lane - measured 14 % slower.)
        // staging tiles: the token-row part of the ring slots is idle in this phase (three tiles per slot);
        // a ring of fewer than three slots has room for a dedicated area
        uint8_t* stg = L.stage_out != kStgAliased ? smem + L.stage_out + warp * kStgWarpBytes
                                                  : smem + (warp / 3) * L.stage_bytes + 2 * kTileBytes + (warp % 3) * kStgWarpBytes;
        const int my_row = valid ? row : p.M;
        auto reduce_64 = [&](const float (&y)[64], int col0) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(y[8 * g + 2 * i], y[8 * g + 2 * i + 1]);
                    w[i] = *reinterpret_cast<uint32_t*>(&h2);
                }
                *reinterpret_cast<uint4*>(stg + lane * kStgPitch + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int r = 4 * i + (lane >> 3), c = lane & 7;
                const uint4 v = *reinterpret_cast<const uint4*>(stg + r * kStgPitch + c * 16);
                const int row_r = __shfl_sync(0xFFFFFFFFu, my_row, r);
                __nv_bfloat16* dst = p.out + static_cast<size_t>(row_r < p.M ? row_r : 0) * p.K + col0 + c * 8;
                red_add_v4_bf16x2_raw_if(dst, v, row_r < p.M);
            }
            __syncwarp();
        };
        // The two warpgroups take alternate iterations: while one is held up issuing its reductions (an SM
        // passes only about 22 bytes of them per cycle) the other reads its accumulator and converts, so the
        // reduction path stays busy.  A warpgroup therefore handles all columns of its iteration, in parts of
        // 64 hidden columns: SPC = 2 -> 2 parts of hidden tile jt (columns [0,128) of the buffer are slice 0's
        // partial sums, [128,256) slice 1's); SPC = 1 -> 4 parts covering hidden tiles 2jt and 2jt+1.
        constexpr int PARTS = SPC == 1 ? 4 : 2;
        for (int jt = 0; jt < ND && ok; ++jt) {
            const int it = UPI + jt;
            const int b = it & 1;
            const uint32_t aph = (it >> 1) & 1;
            if ((jt & 1) != hh) continue;
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 41, it)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int part = 0; part < PARTS; ++part) {
                const int tile = SPC == 1 ? 2 * jt + (part >> 1) : jt;
                const bool live = warp_valid && tile < KC;
                float y[64];
                if (live) {
                    const uint32_t tb = tlane + b * 256 + part * 64;
                    if constexpr (SPC == 1) {
                        uint32_t v[64];
#pragma unroll
                        for (int c0 = 0; c0 < 64; c0 += 16)
                            tmem_ld16(tb + c0, *reinterpret_cast<uint32_t(*)[16]>(&v[c0]));
                        tmem_ld_wait();
                        const float f = sw2[tile] * fac[0];
#pragma unroll
                        for (int e = 0; e < 64; ++e) y[e] = __uint_as_float(v[e]) * f;
                    } else {
                        uint32_t va[64], vb[64];
#pragma unroll
                        for (int c0 = 0; c0 < 64; c0 += 16) {
                            tmem_ld16(tb + c0, *reinterpret_cast<uint32_t(*)[16]>(&va[c0]));
                            tmem_ld16(tb + 128 + c0, *reinterpret_cast<uint32_t(*)[16]>(&vb[c0]));
                        }
                        tmem_ld_wait();
                        const float fa = sw2[jt] * fac[0], fb = sw2[KC + jt] * fac[SPC - 1];
#pragma unroll
                        for (int e = 0; e < 64; ++e)
                            y[e] = fmaf(__uint_as_float(va[e]), fa, __uint_as_float(vb[e]) * fb);
                    }
                }
                if (part == PARTS - 1) {
                    // the buffer has been read completely: hand it back before the last reductions are issued
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_relaxed_n(&acc_empty[b], 2);   // 4 warps stand in for the barrier's 8
                }
                if (live) reduce_64(y, (SPC == 1 ? tile * 128 + (part & 1) * 64 : jt * 128 + part * 64));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace amoe
