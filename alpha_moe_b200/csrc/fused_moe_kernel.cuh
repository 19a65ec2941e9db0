// Fused W8A8 MoE expert MLP for sm_100a: up-projection -> SwiGLU -> fp8 re-quantisation ->
// down-projection -> weighted accumulation into `out`, one launch per layer call.
//
// Replaces csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:654-1098 (the Hopper
// wgmma megakernel).  Same decomposition of the problem - one CTA per (block of block_m sorted
// assignments of one expert, 128-wide slice of the intermediate dimension) - but a different
// machine mapping:
//   * weights are the UMMA "M" operand (128 rows per instruction), the gathered tokens the "N"
//     operand, accumulators live in TMEM (tcgen05.mma kind::f8f6f4), not in registers;
//   * the gate and up halves of the 8-row-interleaved `w` are separated for free: one TMA box
//     brings 256 interleaved rows, and two UMMA descriptors with an 8-row-group stride of 2048 B
//     pick the 128 gate rows and the 128 up rows, so gate[i] and up[i] of one intermediate column
//     land in the same TMEM lane and SwiGLU is thread-local;
//   * each 128-deep K chunk is accumulated into its own TMEM buffer and promoted into fp32
//     registers with the (128x128 weight block) x (token, 128-group) scales (reference :915-933
//     promotes into bf16); TMEM buffers are double-buffered so chunk k+1's MMAs overlap chunk k's
//     promotion;
//   * roles: 1 TMA thread (weights), 1 UMMA thread, 2 gather warps (token rows, cp.async with the
//     128-byte swizzle applied by hand), 1-2 epilogue warpgroups.
//
// Shared-memory ring slot: [256 weight rows x 128 B = 32 KB][token tile BMP x 128 B].
//   up phase   : rows = the slice's 256 interleaved w rows of K-chunk `it`; token tile = x rows of the chunk
//   down phase : rows = 256 consecutive hidden rows of w2 (the slice's 128 columns), i.e. two 128-row tiles
#pragma once

#include "ptx_sm100.cuh"

namespace amoe {

struct MoeParams {
    const uint8_t* x;          // fp8 e4m3 [M, K]
    const float* x_scale;      // [M, K/128]
    const float* w_scale;      // [E, N/128, K/128], gate/up rows interleaved by 1
    const float* w2_scale;     // [E, K/128, I/128]
    __nv_bfloat16* out;        // [M, K]
    const int* sorted_token_ids;
    const int* expert_ids;
    const int* num_tokens_post_padded;
    const float* topk_weights;  // [M, top_k]
    int top_k, M, K, N, E, sorted_num, block_m;
    int stages;                 // ring depth actually used (fits in shared memory)
    int lag;                    // gather completion is signalled `lag` chunks late (< stages)
    float scaling;
    KernelStatus* status;
#ifdef AMOE_TRACE
    long long* trace;           // [12][KC+ND] clock64 stamps of one CTA (debug builds only)
    int trace_block;
#endif
};

#ifdef AMOE_TRACE
#define AMOE_STAMP(ev, it)                                                                   \
    do {                                                                                     \
        if (p.trace && static_cast<int>(blockIdx.x) == p.trace_block)                        \
            p.trace[(ev) * (KC + ND) + (it)] = clock64();                                    \
    } while (0)
#else
#define AMOE_STAMP(ev, it) do { } while (0)
#endif

constexpr int kTileBytes = 128 * 128;  // one 128-row x 128-byte operand tile

struct SmemPlan {
    uint32_t stage_bytes, hq, xs, swg, swu, sw2, tokrow, topkw, tokscale, amax, bars, misc, total;
};
// Offsets from a 1024-byte aligned base.  bmp = padded block_m, s = ring depth, kc = K/128.
__host__ __device__ inline SmemPlan smem_plan(int bmp, int s, int kc) {
    SmemPlan p;
    p.stage_bytes = 2 * kTileBytes + bmp * 128;
    uint32_t o = s * p.stage_bytes;
    p.hq = o;        o += bmp * 128;
    p.xs = o;        o += kc * bmp * 4;
    p.swg = o;       o += kc * 4;
    p.swu = o;       o += kc * 4;
    p.sw2 = o;       o += kc * 4;
    o = (o + 15u) & ~15u;
    p.tokrow = o;    o += bmp * 4;
    p.topkw = o;     o += bmp * 4;
    p.tokscale = o;  o += bmp * 4;
    p.amax = o;      o += bmp * 16;
    p.bars = o;      o += (2 * s + 5) * 8;
    p.misc = o;      o += 16;
    p.total = o;
    return p;
}

template <int LAGMAX>
__device__ __forceinline__ void cp_async_wait_dyn(int n) {
    if (n <= 0) cp_async_wait<0>();
    else if (n == 1) cp_async_wait<1>();
    else cp_async_wait<2>();
}

template <int BMP>
__global__ void __launch_bounds__(128 * (BMP >= 64 ? 2 : 1) + 128, 1)
fused_moe_w8a8_up_down_sm100_kernel(const __grid_constant__ CUtensorMap tm_w,
                                    const __grid_constant__ CUtensorMap tm_w2, const MoeParams p) {
    constexpr int NEPI_WG = BMP >= 64 ? 2 : 1;   // epilogue warpgroups; each owns BMP/NEPI_WG token columns
    constexpr int NC = BMP / NEPI_WG;
    constexpr int EPI_THREADS = 128 * NEPI_WG;
    constexpr int W_TMA = 4 * NEPI_WG, W_MMA = W_TMA + 1, W_G0 = W_TMA + 2;
    constexpr uint32_t TMEM_COLS = 4 * BMP;      // two buffers x (gate|up) x BMP columns
    static_assert(BMP == 16 || BMP == 32 || BMP == 64 || BMP == 128, "padded block_m");

    const int nslices = p.N >> 8;
    const int mblock = blockIdx.x / nslices;
    const int slice = blockIdx.x - mblock * nslices;
    const int npad = min(p.num_tokens_post_padded[0], p.sorted_num);
    if (mblock * p.block_m >= npad) return;          // block beyond the padded schedule (reference :678)
    const int expert = p.expert_ids[mblock];
    if (expert < 0 || expert >= p.E) return;

    const int KC = p.K >> 7;           // 128-deep K chunks of the up-projection
    const int ND = (KC + 1) >> 1;      // ring slots of the down-projection (two 128-row w2 tiles each)
    const int S = p.stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const SmemPlan L = smem_plan(BMP, S, KC);
    uint8_t* hq = smem + L.hq;                                        // fp8 intermediate [BMP][128], swizzled
    float* xs = reinterpret_cast<float*>(smem + L.xs);                // [KC][BMP] token scales
    float* swg = reinterpret_cast<float*>(smem + L.swg);              // [KC] gate block scales
    float* swu = reinterpret_cast<float*>(smem + L.swu);              // [KC] up block scales
    float* sw2 = reinterpret_cast<float*>(smem + L.sw2);              // [KC] w2 block scales (per 128 hidden rows)
    int* tokrow = reinterpret_cast<int*>(smem + L.tokrow);            // [BMP] row of x/out, or M if padding
    float* topkw = reinterpret_cast<float*>(smem + L.topkw);          // [BMP]
    float* tokscale = reinterpret_cast<float*>(smem + L.tokscale);    // [BMP] s_h * topk_weight * scaling
    uint32_t* amax_part = reinterpret_cast<uint32_t*>(smem + L.amax); // [BMP][4] per-warp |h| maxima
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);   // slot filled: TMA bytes + 2 gather warps
    uint64_t* empty = full + S;                                    // slot free again
    uint64_t* acc_full = empty + S;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* h_ready = acc_empty + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L.misc);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L.misc + 4);

    if (threadIdx.x == W_TMA * 32) {
        for (int i = 0; i < S; ++i) {
            mbar_init(&full[i], 3);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 4 * NEPI_WG);
        }
        mbar_init(h_ready, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == W_MMA) {
        tmem_alloc(tmem_slot, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp >= W_TMA) {
    // ====================================================================== control warpgroup
    // The widest variant keeps 2 x 64 accumulators per epilogue thread: it moves registers from this
    // warpgroup (TMA / UMMA / gather warps) to the two epilogue warpgroups.
    if constexpr (BMP == 128) setmaxnreg_dec<64>();
    if (warp == W_TMA) {
        // ------------------------------------------------------------------ weight producer
        if (lane == 0) {
            prefetch_tmap(&tm_w);
            prefetch_tmap(&tm_w2);
            int s = 0;
            uint32_t ph = 0;
            uint8_t* st = smem;
            for (int it = 0; it < KC + ND; ++it) {
                AMOE_STAMP(7, it);
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 10, it)) break;
                AMOE_STAMP(0, it);
                mbar_arrive_expect_tx(&full[s], 2 * kTileBytes);
                if (it < KC) {  // 256 interleaved rows (128 gate + 128 up) x 128 bytes of K chunk `it`
                    tma_load_3d(st, &tm_w, &full[s], it * 128, slice * 256, expert);
                } else {        // 256 hidden rows x the slice's 128 columns of w2; rows past K arrive as zeros
                    tma_load_3d(st, &tm_w2, &full[s], slice * 128, (it - KC) * 256, expert);
                    mbar_arrive(&full[s]);   // no token gather in this phase: stand in for the two
                    mbar_arrive(&full[s]);   // gather warps so that the barrier's count stays 3
                }
                AMOE_STAMP(6, it);
                st += L.stage_bytes;
                if (++s == S) { s = 0; ph ^= 1; st = smem; }
            }
        }
    } else if (warp == W_MMA) {
        // ------------------------------------------------------------------ UMMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_e4m3(128, BMP);
            const uint64_t hdesc = umma_desc_sw128(smem_u32(hq));
            const uint32_t st0 = smem_u32(smem);
            // Descriptors advance with the ring slot: only the 14-bit start-address field changes.
            const uint64_t dstep = L.stage_bytes >> 4;
            const uint64_t a0_up0 = umma_desc_sw128(st0, 2048u);            // 8 gate rows of every 16
            const uint64_t a1_up0 = umma_desc_sw128(st0 + 1024u, 2048u);    // 8 up rows of every 16
            const uint64_t x_up0 = umma_desc_sw128(st0 + 2 * kTileBytes);   // gathered token rows
            const uint64_t a0_dn0 = umma_desc_sw128(st0);                   // first 128 hidden rows of the slot
            const uint64_t a1_dn0 = umma_desc_sw128(st0 + kTileBytes);      // second 128 hidden rows
            int s = 0;
            uint32_t ph = 0;
            uint64_t off = 0;
            for (int it = 0; it < KC + ND; ++it) {
                const int b = it & 1;
                const uint32_t aph = (it >> 1) & 1;
                const bool up = it < KC;
                AMOE_STAMP(8, it);
                if (it == KC && !mbar_wait(h_ready, 0, abort_flag, p.status, 20, it)) break;
                if (!mbar_wait(&acc_empty[b], aph ^ 1, abort_flag, p.status, 21, it)) break;
                AMOE_STAMP(9, it);
                if (!mbar_wait(&full[s], ph, abort_flag, p.status, 22, it)) break;
                tc_fence_after();
                AMOE_STAMP(1, it);
                const uint32_t d0 = tmem_base + b * 2 * BMP;
                if (up)
                    umma_f8_chunk2(d0, d0 + BMP, a0_up0 + off, a1_up0 + off, x_up0 + off, idesc);
                else if (2 * (it - KC) + 1 < KC)
                    umma_f8_chunk2(d0, d0 + BMP, a0_dn0 + off, a1_dn0 + off, hdesc, idesc);
                else
                    umma_f8_chunk1(d0, a0_dn0 + off, hdesc, idesc);
                AMOE_STAMP(11, it);
                // One commit per chunk: the epilogue, once it sees the accumulators complete, also hands
                // the ring slot back to the producers (the MMAs have finished reading it by then).
                umma_commit(&acc_full[b]);
                AMOE_STAMP(2, it);
                off += dstep;
                if (++s == S) { s = 0; ph ^= 1; off = 0; }
            }
        }
    } else {
        // ------------------------------------------------------------------ token-row gather (2 warps)
        constexpr int PIECES = BMP / 8;             // 16-byte pieces per thread per chunk
        const int gtid = threadIdx.x - W_G0 * 32;   // 0..63
        const int row0 = gtid >> 3, ch = gtid & 7;
        uint32_t src16[PIECES];                     // (row * K) / 16, or 0xFFFFFFFF for a padding row
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
            const int row = row0 + 8 * i;
            const int idx = mblock * p.block_m + row;
            src16[i] = 0xFFFFFFFFu;
            if (row < p.block_m && idx < p.sorted_num) {
                const int pid = p.sorted_token_ids[idx];
                if (pid >= 0 && pid < p.M * p.top_k)
                    src16[i] = static_cast<uint32_t>((static_cast<size_t>(pid / p.top_k) * p.K) >> 4);
            }
        }
        const uint32_t dst0 = row0 * 128 + ((ch ^ (row0 & 7)) << 4);   // + i*1024 for piece i (row & 7 unchanged)
        const int lag = p.lag;
        bool ok = true;
        int s = 0, sl = 0;                          // slot being filled / slot whose completion is signalled next
        uint32_t ph = 0;
        for (int it = 0; it < KC; ++it) {
            if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 30, it)) { ok = false; break; }
            const uint32_t base = smem_u32(smem + s * L.stage_bytes + 2 * kTileBytes) + dst0;
            const uint8_t* col = p.x + it * 128 + ch * 16;
#pragma unroll
            for (int i = 0; i < PIECES; ++i) {
                const bool v = src16[i] != 0xFFFFFFFFu;
                const uint8_t* src = v ? col + (static_cast<size_t>(src16[i]) << 4) : p.x;
                cp_async_16(base + i * 1024, src, v ? 16u : 0u);
            }
            cp_async_commit();
            if (gtid == 0) AMOE_STAMP(5, it);
            if (it >= lag) {
                cp_async_wait_dyn<2>(lag);
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[sl]);
                if (++sl == S) sl = 0;
            }
            if (++s == S) { s = 0; ph ^= 1; }
        }
        cp_async_wait<0>();
        if (ok) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
                for (int it = max(KC - lag, 0); it < KC; ++it) {
                    mbar_arrive(&full[sl]);
                    if (++sl == S) sl = 0;
                }
        }
    }
    } else {
        // ====================================================================== epilogue warpgroups
        if constexpr (BMP == 128) setmaxnreg_inc<216>();
        const int q = warp & 3;              // TMEM lane quarter this warp may read
        const int hh = warp >> 2;            // which half of the token columns
        const int r = q * 32 + lane;         // weight row inside the tile = TMEM lane
        const int etid = threadIdx.x;
        const int mtk = p.M * p.top_k;
        for (int j = etid; j < BMP; j += EPI_THREADS) {
            int row = p.M;
            float tw = 0.f;
            const int idx = mblock * p.block_m + j;
            if (j < p.block_m && idx < p.sorted_num) {
                const int pid = p.sorted_token_ids[idx];
                if (pid >= 0 && pid < mtk) {
                    row = pid / p.top_k;             // reference :757
                    tw = p.topk_weights[pid];        // reference :761
                }
            }
            tokrow[j] = row;
            topkw[j] = tw;
        }
        {
            const int nsr = p.N >> 7;                         // scale rows per expert in w_scale
            const int isl = p.N >> 8;                         // 128-column slices of the intermediate dim
            const float* ws = p.w_scale + (static_cast<size_t>(expert) * nsr + 2 * slice) * KC;
            const float* w2s = p.w2_scale + static_cast<size_t>(expert) * KC * isl + slice;
            for (int i = etid; i < KC; i += EPI_THREADS) {
                swg[i] = ws[i];                               // interleave slot 0 = gate (reference :919-925)
                swu[i] = ws[KC + i];                          // slot 1 = up
                sw2[i] = w2s[static_cast<size_t>(i) * isl];
            }
        }
        named_bar_sync(1, EPI_THREADS);
        for (int i = etid; i < BMP * KC; i += EPI_THREADS) {
            const int j = i / KC, kc = i - j * KC;
            const int row = tokrow[j];
            xs[kc * BMP + j] = row < p.M ? p.x_scale[static_cast<size_t>(row) * KC + kc] : 0.f;
        }
        int nhi = 0;
        for (int j = 0; j < BMP; ++j)
            if (tokrow[j] < p.M) nhi = j + 1;
        const int my_ncols = min(max(nhi - hh * NC, 0), NC);
        named_bar_sync(1, EPI_THREADS);

        float accg[NC], accu[NC];
#pragma unroll
        for (int j = 0; j < NC; ++j) accg[j] = accu[j] = 0.f;

        const uint32_t tlane = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + hh * NC;
        bool ok = true;
        int es = 0;                          // ring slot of the chunk being retired (for handing it back)
        // ---- up-projection: promote each K chunk with its scales (reference :915-933)
        for (int it = 0; it < KC; ++it) {
            const int b = it & 1;
            const uint32_t aph = (it >> 1) & 1;
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 40, it)) { ok = false; break; }
            if (etid == 0) mbar_arrive(&empty[es]);      // the MMAs of this chunk have consumed the slot
            if (++es == S) es = 0;
            tc_fence_after();
            if (etid == 0) AMOE_STAMP(3, it);
            const float sg = swg[it], su = swu[it];
            const uint32_t tb = tlane + b * 2 * BMP;
#pragma unroll
            for (int c0 = 0; c0 < NC; c0 += 16) {
                if (c0 < my_ncols) {
                    uint32_t vg[16], vu[16];
                    tmem_ld16(tb + c0, vg);
                    tmem_ld16(tb + BMP + c0, vu);
                    tmem_ld_wait();
                    const float4* sx4 = reinterpret_cast<const float4*>(xs + it * BMP + hh * NC + c0);
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
            if (etid == 0) AMOE_STAMP(4, it);
        }

        // ---- SwiGLU, per-token amax over the 128 columns of the slice, fp8 re-quantisation
        //      (reference :936-1005; here h stays in registers, only the fp8 tile goes to shared memory)
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const float g = bf16_round(accg[j]);
            const float u = bf16_round(accu[j]);
            const float h = bf16_round(__fdividef(g, 1.0f + __expf(-g)) * u);
            accg[j] = h;
            const uint32_t a = __reduce_max_sync(0xFFFFFFFFu, __float_as_uint(fabsf(h)));
            if (lane == 0) amax_part[(hh * NC + j) * 4 + q] = a;
        }
        named_bar_sync(2 + hh, 128);
        // Factor of column j for the output = s_h * topk weight * scaling (reference :997-1003), and its
        // row in `out` (M = padding): kept in registers, except in the widest variant where the registers
        // are needed for the accumulators and the pair comes from shared memory instead.
        constexpr bool kFactorsInRegs = NC <= 32;
        constexpr int NF = kFactorsInRegs ? NC : 2;
        int rowj[NF];
        float facj[NF];
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int col = hh * NC + j;
            const uint4 pm = *reinterpret_cast<const uint4*>(amax_part + col * 4);
            const float amax = __uint_as_float(max(max(pm.x, pm.y), max(pm.z, pm.w)));
            const float s_h = fmaxf(amax, 1e-10f) * (1.0f / 448.0f);
            const float qv = fminf(fmaxf(__fdividef(accg[j], s_h), -448.0f), 448.0f);
            const uint8_t qb = static_cast<uint8_t>(__nv_cvt_float_to_fp8(qv, __NV_SATFINITE, __NV_E4M3));
            hq[col * 128 + ((((r >> 4) ^ (col & 7)) << 4) | (r & 15))] = qb;
            const float fac = s_h * topkw[col] * p.scaling;
            if constexpr (kFactorsInRegs) {
                facj[j] = fac;
                rowj[j] = tokrow[col];
            } else {
                if (r == 0) tokscale[col] = fac;
            }
        }
        fence_proxy_async_smem();
        named_bar_sync(1, EPI_THREADS);
        if (etid == 0) mbar_arrive(h_ready);

        // ---- down-projection epilogue: scale, pair adjacent hidden columns, bf16x2 reduce into out
        //      (reference :1052-1094 goes through stmatrix + per-row bulk reduce).
        // The accumulators are copied to registers and handed back to the MMA thread *before* any
        // reduction is issued: tcgen05.fence / mbarrier.arrive after a global reduction would wait for
        // L2 to acknowledge it, which would put an L2 round trip into every iteration.
        const bool odd = lane & 1;
        for (int jt = 0; jt < ND && ok; ++jt) {
            const int it = KC + jt;
            const int b = it & 1;
            const uint32_t aph = (it >> 1) & 1;
            if (etid == 0) AMOE_STAMP(6, it);
            if (!mbar_wait(&acc_full[b], aph, abort_flag, p.status, 41, it)) { ok = false; break; }
            if (etid == 0) AMOE_STAMP(10, it);
            if (etid == 0) mbar_arrive_relaxed(&empty[es]);
            if (++es == S) es = 0;
            tc_fence_after();
            if (etid == 0) AMOE_STAMP(3, it);
            const bool two = 2 * jt + 1 < KC;
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
            if (etid == 0) AMOE_STAMP(4, it);
#pragma unroll
            for (int tt = 0; tt < 2; ++tt) {
                if (tt == 0 || two) {
                    const int tile = 2 * jt + tt;
                    const float s2 = sw2[tile];
                    __nv_bfloat16* obase = p.out + tile * 128 + (r & ~1);
                    // Straight-line over each live 16-column group (padding columns carry row == M and
                    // are masked at the reduction): per-pair branches would serialise this single warp.
#pragma unroll
                    for (int c0 = 0; c0 < NC; c0 += 16) {
                        if (c0 < my_ncols) {
#pragma unroll
                            for (int j = c0; j < c0 + 16; j += 2) {
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
                                red_add_bf16x2_if(obase + static_cast<size_t>(row) * p.K, lo, hi, row, p.M);
                            }
                        }
                    }
                }
            }
            if (etid == 0) AMOE_STAMP(5, it);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace amoe
