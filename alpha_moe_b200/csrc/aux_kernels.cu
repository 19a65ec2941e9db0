// The two kernels a serving engine runs immediately before the fused MoE operator, which the
// reference imports from SGLang (jit_moe.py:142,158; extra/sglang.patch:30-35):
//   * moe_align_block_size  - block schedule (sorted_token_ids, expert_ids, num_tokens_post_padded)
//   * per-token-group fp8 quantisation of the activations (group = 128), optionally zeroing the
//     bf16 source afterwards, which is what the call site does next (extra/sglang.patch:31).
// Both are integer / byte work bound by memory traffic; no tensor cores involved.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/alpha_moe_b200.h"
#include "capi_internal.h"

namespace amoe_aux {

using amoe_capi::fail;

#define AUX_TRY(expr)                                                                              \
    do {                                                                                           \
        cudaError_t err__ = (expr);                                                                \
        if (err__ != cudaSuccess)                                                                  \
            return fail(ALPHA_MOE_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));      \
    } while (0)

// ------------------------------------------------------------------------------------------------
// moe_align_block_size.  Flat assignment index p = token * top_k + j, expert topk_ids[p].
// Each expert's indices are written in ascending order (a stable counting sort), starting at a
// multiple of `block`, the rest of the expert's last block holding the sentinel `numel`.
//
// Work is cut into chunks of kChunk consecutive assignments, one CTA each:
//   phase A  fill outputs with their defaults; per-chunk histogram -> hist[chunk][expert]
//   phase B  every CTA derives, from the whole histogram table, the padded expert sizes, their exclusive scan and
//            the first output slot of its own chunk's assignments of every expert; CTA 0 also writes expert_ids per
//            block and num_tokens_post_padded
//   phase C  stable scatter: warps walk their 128 assignments in order, ranking equal experts inside a warp round
//            with match.any
// One launch runs all three phases with a grid-wide barrier after phase A (a cooperative launch, used whenever all
// chunks fit on the GPU at once); otherwise phase A and phases B + C are two launches of the same kernel.  When
// everything fits one chunk the phases run inside one CTA of an ordinary launch.
// Programmatic dependent launch: the kernel behind this one in the stream (the fused operator, which is launched with
// the matching attribute and waits for this kernel's completion before it reads anything) may be scheduled from here on.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

constexpr int kChunk = 1024;          // assignments per CTA (8 warps x 4 rounds x 32 lanes)
constexpr int kAlignThreads = 256;
constexpr int kMaxExperts = 1024;     // per-warp counters live in shared memory: 8 x E ints

// Per-warp counts of each expert over the warp's 128 consecutive assignments of the chunk.
__device__ __forceinline__ void count_chunk(const int32_t* ids, int numel, int chunk_start, int E, int* cnt /*[8][E]*/) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 8 * E; i += kAlignThreads) cnt[i] = 0;
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int p = chunk_start + warp * 128 + r * 32 + lane;
        const bool in = p < numel;
        int e = in ? ids[p] : -1;
        if (e < 0 || e >= E) e = -1;                       // ids outside [0,E) are ignored
        const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
        if (e >= 0 && (same & ((1u << lane) - 1)) == 0) cnt[warp * E + e] += __popc(same);   // leader lane
        __syncwarp();
    }
    __syncthreads();
}

// Stable scatter of one chunk.  base[w][e] = first output slot for warp w's assignments of expert e.
__device__ __forceinline__ void scatter_chunk(const int32_t* ids, int numel, int chunk_start, int E, int* base,
                                              int32_t* sorted) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int p = chunk_start + warp * 128 + r * 32 + lane;
        const bool in = p < numel;
        int e = in ? ids[p] : -1;
        if (e < 0 || e >= E) e = -1;
        const unsigned same = __match_any_sync(0xFFFFFFFFu, e);
        const int leader = __ffs(same) - 1;
        int pos0 = 0;
        if (e >= 0 && lane == leader) {
            pos0 = base[warp * E + e];
            base[warp * E + e] = pos0 + __popc(same);
        }
        pos0 = __shfl_sync(0xFFFFFFFFu, pos0, leader);
        if (e >= 0) sorted[pos0 + __popc(same & ((1u << lane) - 1))] = p;
        __syncwarp();
    }
}

constexpr int kPhaseA = 1, kPhaseBC = 2;

// `phases` = kPhaseA, kPhaseBC or both; both only in a cooperative launch (grid-wide barrier in between).
__global__ void __launch_bounds__(kAlignThreads)
moe_align_chunks_kernel(const int32_t* ids, int numel, int E, int block, int32_t* sorted, int sorted_len,
                        int32_t* expert_ids, int n_blocks_max, int* hist /*[chunks][E]*/, int32_t* num_post_pad,
                        int phases) {
    __shared__ int cnt[8 * kMaxExperts];
    __shared__ int warp_tot[kAlignThreads / 32];
    const int chunks = gridDim.x, chunk = blockIdx.x;
    launch_dependents();
    if (phases & kPhaseA) {
        const int gtid = chunk * kAlignThreads + threadIdx.x, gsz = chunks * kAlignThreads;
        for (int i = gtid; i < sorted_len; i += gsz) sorted[i] = numel;
        for (int i = gtid; i < n_blocks_max; i += gsz) expert_ids[i] = 0;
    }
    count_chunk(ids, numel, chunk * kChunk, E, cnt);       // (needed by both phases: recounted in a second launch)
    if (phases & kPhaseA) {
        for (int e = threadIdx.x; e < E; e += kAlignThreads) {
            int s = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += cnt[w * E + e];
            hist[chunk * E + e] = s;
        }
    }
    if (!(phases & kPhaseBC)) return;
    if (phases & kPhaseA) cooperative_groups::this_grid().sync();

    // Phase B.  Thread t owns the experts [t * per, (t + 1) * per): their totals over all chunks, the part of it that
    // precedes this chunk, and (after a scan over the padded totals) their first output slots.
    const int per = (E + kAlignThreads - 1) / kAlignThreads;           // <= 4
    int before[4], padded[4], mine = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x * per + i;
        before[i] = 0;
        padded[i] = 0;
        if (i < per && e < E) {
            int tot = 0, bef = 0;
#pragma unroll 8
            for (int c = 0; c < chunks; ++c) {
                const int v = hist[c * E + e];
                tot += v;
                bef += c < chunk ? v : 0;
            }
            before[i] = bef;
            padded[i] = (tot + block - 1) / block * block;
            mine += padded[i];
        }
    }
    // exclusive scan of `mine` over the threads (warp shuffles, then the eight warp totals)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int run = incl - mine;
    for (int w = 0; w < warp; ++w) run += warp_tot[w];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x * per + i;
        if (i < per && e < E) {
            if (chunk == 0)
                for (int b = run / block; b < (run + padded[i]) / block; ++b) expert_ids[b] = e;
            int slot = run + before[i];
#pragma unroll
            for (int w = 0; w < 8; ++w) {          // counts -> first slot of each warp's assignments of expert e
                const int n = cnt[w * E + e];
                cnt[w * E + e] = slot;
                slot += n;
            }
            run += padded[i];
        }
    }
    if (chunk == 0 && threadIdx.x == kAlignThreads - 1) num_post_pad[0] = run;     // the last thread's running end = total
    __syncthreads();
    scatter_chunk(ids, numel, chunk * kChunk, E, cnt, sorted);
}

// Everything in one CTA when there is a single chunk (numel <= kChunk: e.g. up to 113 tokens at top_k = 9).
// cnt: 8 * kMaxExperts ints, warp_tot: 8 ints of shared memory.  Thread t owns the experts [t * per, (t + 1) * per):
// their padded sizes, then (after a scan over the threads: warp shuffles and the eight warp totals) their first output
// slots - a single thread walking over all experts took longer than everything else in this kernel together.
__device__ __forceinline__ void align_single_body(const int32_t* ids, int numel, int E, int block, int32_t* sorted,
                                                  int sorted_len, int32_t* expert_ids, int n_blocks_max,
                                                  int32_t* num_post_pad, int* cnt, int* warp_tot) {
    for (int i = threadIdx.x; i < sorted_len; i += kAlignThreads) sorted[i] = numel;
    for (int i = threadIdx.x; i < n_blocks_max; i += kAlignThreads) expert_ids[i] = 0;
    count_chunk(ids, numel, 0, E, cnt);                   // (its barriers also order the default fills before the writes below)
    const int per = (E + kAlignThreads - 1) / kAlignThreads;           // <= 4
    int padded[4], mine = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x * per + i;
        padded[i] = 0;
        if (i < per && e < E) {
            int tot = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) tot += cnt[w * E + e];
            padded[i] = (tot + block - 1) / block * block;
            mine += padded[i];
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int run = incl - mine;
    for (int w = 0; w < warp; ++w) run += warp_tot[w];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x * per + i;
        if (i < per && e < E) {
            for (int b = run / block; b < (run + padded[i]) / block; ++b) expert_ids[b] = e;
            int slot = run;
#pragma unroll
            for (int w = 0; w < 8; ++w) {          // counts -> first slot of each warp's assignments of expert e
                const int n = cnt[w * E + e];
                cnt[w * E + e] = slot;
                slot += n;
            }
            run += padded[i];
        }
    }
    if (threadIdx.x == kAlignThreads - 1) num_post_pad[0] = run;       // the last thread's running end = total
    __syncthreads();
    scatter_chunk(ids, numel, 0, E, cnt, sorted);
}

__global__ void __launch_bounds__(kAlignThreads)
moe_align_single_kernel(const int32_t* ids, int numel, int E, int block, int32_t* sorted, int sorted_len,
                        int32_t* expert_ids, int n_blocks_max, int32_t* num_post_pad) {
    __shared__ int cnt[8 * kMaxExperts];
    __shared__ int warp_tot[kAlignThreads / 32];
    launch_dependents();
    align_single_body(ids, numel, E, block, sorted, sorted_len, expert_ids, n_blocks_max, num_post_pad, cnt, warp_tot);
}

// ------------------------------------------------------------------------------------------------
// Per-(token, 128-group) fp8 quantisation: scale = max(amax, 1e-10) / 448, q = e4m3_rn(clamp(x / scale)).
// Eight lanes per group, 16 elements per lane: two 16-byte loads in, one 16-byte store out (algorithmic traffic
// 3 bytes per element, + 2 when the source is zeroed); a warp takes four consecutive groups per step and the grid
// strides over the tensor.  The quotients are the correctly rounded IEEE ones, so the result is bit-identical to the
// CPU restatement.
__device__ __forceinline__ void group_quant_body(__nv_bfloat16* x, uint8_t* q, float* scale, long long n_groups,
                                                 int zero_src, int block, int nblocks) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 7;                   // 16-element piece of the group
    const long long warp0 = static_cast<long long>(block) * 8 + (threadIdx.x >> 5);
    const long long nwarps = static_cast<long long>(nblocks) * 8;
    // the loads of the next step are issued before the arithmetic of the current one (one step = 32 bytes per lane)
    uint4 n0 = make_uint4(0u, 0u, 0u, 0u), n1 = n0;
    {
        const long long g = warp0 * 4 + (lane >> 3);
        if (g < n_groups) {
            const uint4* first = reinterpret_cast<const uint4*>(x + g * 128 + sub * 16);
            n0 = first[0];
            n1 = first[1];
        }
    }
    for (long long g0 = warp0 * 4; g0 < n_groups; g0 += nwarps * 4) {
        const long long g = g0 + (lane >> 3);
        const bool live = g < n_groups;
        uint4* src = reinterpret_cast<uint4*>(x + (live ? g : 0) * 128 + sub * 16);
        const uint4 r0 = n0, r1 = n1;
        {
            const long long gn = g + nwarps * 4;
            if (gn < n_groups) {
                const uint4* nxt = reinterpret_cast<const uint4*>(x + gn * 128 + sub * 16);
                n0 = nxt[0];
                n1 = nxt[1];
            }
        }
        const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
        float v[16];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            v[2 * i] = __low2float(a);
            v[2 * i + 1] = __high2float(a);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        const float s = __fdiv_rn(fmaxf(amax, 1e-10f), 448.0f);
        // x / s, correctly rounded, for sixteen x and one s: with rcp = RN(1 / s), q0 = RN(x * rcp), the exact
        // remainder r = x - q0 * s (one FMA) and q = RN(q0 + r * rcp) give the IEEE quotient (Markstein's theorem)
        // for every s whose mantissa is not all ones - three instructions per element instead of a division's ten.
        // The exception takes the division.  Every output byte still equals the CPU restatement's.
        const float rcp = __frcp_rn(s);
        const bool plain_division = (__float_as_uint(s) & 0x7FFFFFu) == 0x7FFFFFu;
        uint32_t out[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float y[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float xv = v[4 * i + j];
                float qv;
                if (plain_division) {
                    qv = __fdiv_rn(xv, s);
                } else {
                    const float q0 = __fmul_rn(xv, rcp);
                    qv = __fmaf_rn(__fmaf_rn(-q0, s, xv), rcp, q0);
                }
                y[j] = fminf(fmaxf(qv, -448.0f), 448.0f);
            }
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(y[0], y[1]), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(y[2], y[3]), __NV_SATFINITE, __NV_E4M3);
            out[i] = lo | (hi << 16);
        }
        if (live) {
            *reinterpret_cast<uint4*>(q + g * 128 + sub * 16) = make_uint4(out[0], out[1], out[2], out[3]);
            if (sub == 0) scale[g] = s;
            if (zero_src) {
                src[0] = make_uint4(0u, 0u, 0u, 0u);
                src[1] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    }
}

__global__ void __launch_bounds__(256)
group_quant_fp8_kernel(__nv_bfloat16* x, uint8_t* q, float* scale, long long n_groups, int zero_src) {
    launch_dependents();
    group_quant_body(x, q, scale, n_groups, zero_src, blockIdx.x, gridDim.x);
}

// The two steps in front of the operator at a serving call site - quantise the activations (and clear their buffer,
// which the layer then accumulates into) and build the block schedule - are independent of each other.  For decode-
// size batches, whose schedule fits one CTA, they run as one launch: the last CTA builds the schedule, the others
// quantise.  Same code, same bits as the two separate kernels.
__global__ void __launch_bounds__(256)
quant_and_align_small_kernel(__nv_bfloat16* x, uint8_t* q, float* scale, long long n_groups, int zero_src,
                             const int32_t* ids, int numel, int E, int block, int32_t* sorted, int sorted_len,
                             int32_t* expert_ids, int n_blocks_max, int32_t* num_post_pad) {
    __shared__ int cnt[8 * kMaxExperts];
    __shared__ int warp_tot[kAlignThreads / 32];
    static_assert(kAlignThreads == 256, "one block shape for both halves");
    launch_dependents();      // the operator behind this launch may be scheduled; it waits for our completion
    if (blockIdx.x == gridDim.x - 1) {
        align_single_body(ids, numel, E, block, sorted, sorted_len, expert_ids, n_blocks_max, num_post_pad, cnt, warp_tot);
        return;
    }
    group_quant_body(x, q, scale, n_groups, zero_src, blockIdx.x, gridDim.x - 1);
}

// Scratch of the entry point that allocates nothing: the per-chunk histogram table lives here instead of
// in a caller-provided workspace.  Every GPU that loads the library holds these 256 KB until exit.
constexpr int kNoAllocScratchInts = 64 * 1024;
static __device__ __align__(256) int g_align_scratch[kNoAllocScratchInts];

}  // namespace amoe_aux

// A second stream and two events per (host thread, device) for entry points that run two independent kernels side by
// side: fork from the caller's stream, join back into it.  Created at the first use (make that first call outside
// any stream capture) and kept for the life of the thread.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    bool ready = false;
};
static SideStream* side_stream(int dev) {
    thread_local SideStream per_device[64];
    if (dev < 0 || dev >= 64) return nullptr;
    SideStream& s = per_device[dev];
    if (!s.ready) {
        if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;              // the caller falls back to one stream
        }
        s.ready = true;
    }
    return &s;
}

extern "C" {

int64_t alpha_moe_b200_align_workspace_bytes(int numel, int num_experts) {
    if (numel <= 0 || num_experts <= 0) return 0;
    const int64_t chunks = (static_cast<int64_t>(numel) + amoe_aux::kChunk - 1) / amoe_aux::kChunk;
    return chunks <= 1 ? 0 : chunks * num_experts * static_cast<int64_t>(sizeof(int));
}

int alpha_moe_b200_moe_align_block_size(const int32_t* topk_ids, int numel, int num_experts, int block_m,
                                        int32_t* sorted_token_ids, int32_t* expert_ids,
                                        int32_t* num_tokens_post_padded, void* workspace, void* stream) {
    using namespace amoe_aux;
    if (!topk_ids || !sorted_token_ids || !expert_ids || !num_tokens_post_padded)
        return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (numel <= 0) return fail(ALPHA_MOE_E_ARG, "numel must be positive (got %d)", numel);
    if (num_experts <= 0 || num_experts > kMaxExperts)
        return fail(ALPHA_MOE_E_ARG, "num_experts must be in 1..%d (got %d)", kMaxExperts, num_experts);
    if (block_m <= 0) return fail(ALPHA_MOE_E_ARG, "block_m must be positive (got %d)", block_m);
    const long long sorted_len = static_cast<long long>(numel) + static_cast<long long>(num_experts) * (block_m - 1);
    if (sorted_len > 0x7FFFFFFFLL) return fail(ALPHA_MOE_E_ARG, "schedule too long for int32 indices");
    const int n_blocks_max = static_cast<int>((sorted_len + block_m - 1) / block_m);
    const int chunks = (numel + kChunk - 1) / kChunk;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (chunks == 1) {
        moe_align_single_kernel<<<1, kAlignThreads, 0, st>>>(topk_ids, numel, num_experts, block_m, sorted_token_ids,
                                                            static_cast<int>(sorted_len), expert_ids, n_blocks_max,
                                                            num_tokens_post_padded);
        AUX_TRY(cudaGetLastError());
        return ALPHA_MOE_OK;
    }
    if (!workspace) return fail(ALPHA_MOE_E_ARG, "workspace is required for more than %d assignments", kChunk);
    int* hist = static_cast<int*>(workspace);
    int sorted_len_i = static_cast<int>(sorted_len);
    int n_blocks_max_v = n_blocks_max, numel_v = numel, e_v = num_experts, block_v = block_m;
    // One cooperative launch when every chunk's CTA can be resident at once (the grid-wide barrier needs that);
    // the capacity of a device is looked up once.
    static std::atomic<int> capacity[64];
    int dev = 0;
    AUX_TRY(cudaGetDevice(&dev));
    int cap = dev >= 0 && dev < 64 ? capacity[dev].load(std::memory_order_acquire) : 0;
    if (cap == 0) {
        int per_sm = 0, sms = 0, coop = 0;
        AUX_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_align_chunks_kernel, kAlignThreads, 0));
        AUX_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        AUX_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
        cap = coop ? per_sm * sms : -1;
        if (cap == 0) cap = -1;
        if (dev >= 0 && dev < 64) capacity[dev].store(cap, std::memory_order_release);
    }
    if (chunks <= cap) {
        int phases = kPhaseA | kPhaseBC;
        void* args[] = {&topk_ids, &numel_v, &e_v, &block_v, &sorted_token_ids, &sorted_len_i, &expert_ids,
                        &n_blocks_max_v, &hist, &num_tokens_post_padded, &phases};
        AUX_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(moe_align_chunks_kernel), dim3(chunks),
                                            dim3(kAlignThreads), args, 0, st));
        return ALPHA_MOE_OK;
    }
    moe_align_chunks_kernel<<<chunks, kAlignThreads, 0, st>>>(topk_ids, numel, num_experts, block_m, sorted_token_ids,
                                                             sorted_len_i, expert_ids, n_blocks_max, hist,
                                                             num_tokens_post_padded, kPhaseA);
    AUX_TRY(cudaGetLastError());
    moe_align_chunks_kernel<<<chunks, kAlignThreads, 0, st>>>(topk_ids, numel, num_experts, block_m, sorted_token_ids,
                                                             sorted_len_i, expert_ids, n_blocks_max, hist,
                                                             num_tokens_post_padded, kPhaseBC);
    AUX_TRY(cudaGetLastError());
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_moe_align_block_size_noalloc(const int32_t* topk_ids, int numel, int num_experts, int block_m,
                                                int32_t* sorted_token_ids, int32_t* expert_ids,
                                                int32_t* num_tokens_post_padded, void* stream) {
    using namespace amoe_aux;
    if (numel <= 0 || num_experts <= 0) return fail(ALPHA_MOE_E_ARG, "numel and num_experts must be positive");
    const long long chunks = (static_cast<long long>(numel) + kChunk - 1) / kChunk;
    if (chunks > 1 && chunks * num_experts > kNoAllocScratchInts)
        return fail(ALPHA_MOE_E_ARG,
                    "problem too large for the built-in scratch: ceil(numel/%d) * num_experts = %lld exceeds %d; "
                    "use alpha_moe_b200_moe_align_block_size with a caller-provided workspace",
                    kChunk, chunks * num_experts, kNoAllocScratchInts);
    // In host code the array's name is only a handle; the device address has to be asked for, once per
    // device, with that device current.  This first call on a device should come before any stream capture.
    static int* scratch_of_device[64] = {nullptr};
    int dev = 0;
    AUX_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(ALPHA_MOE_E_ARG, "device ordinal %d not supported", dev);
    if (!scratch_of_device[dev]) {
        int* ptr = nullptr;
        AUX_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_align_scratch));
        scratch_of_device[dev] = ptr;
    }
    // Nothing in the scratch has to start at zero: phase A overwrites every [chunk][expert] entry this call reads.
    return alpha_moe_b200_moe_align_block_size(topk_ids, numel, num_experts, block_m, sorted_token_ids, expert_ids,
                                               num_tokens_post_padded, scratch_of_device[dev], stream);
}

int alpha_moe_b200_per_token_group_quant_fp8(void* x_bf16, void* x_fp8, float* x_scale, int M, int K, int zero_src,
                                             void* stream) {
    using namespace amoe_aux;
    if (!x_bf16 || !x_fp8 || !x_scale) return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (M <= 0 || K <= 0 || K % 128 != 0) return fail(ALPHA_MOE_E_ARG, "need M > 0 and K a positive multiple of 128");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(x_fp8) & 15))
        return fail(ALPHA_MOE_E_ARG, "x_bf16 and x_fp8 must be 16-byte aligned");
    const long long n_groups = static_cast<long long>(M) * (K / 128);
    // 32 groups per block and step; enough blocks for eight per SM at most, the rest is covered by the stride
    int dev = 0, sms = 0;
    AUX_TRY(cudaGetDevice(&dev));
    AUX_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long blocks = (n_groups + 31) / 32;
    if (blocks > static_cast<long long>(sms) * 8) blocks = static_cast<long long>(sms) * 8;
    group_quant_fp8_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(x_fp8), x_scale, n_groups, zero_src);
    AUX_TRY(cudaGetLastError());
    return ALPHA_MOE_OK;
}

int alpha_moe_b200_quant_and_align(void* x_bf16, void* x_fp8, float* x_scale, int M, int K, int zero_src,
                                   const int32_t* topk_ids, int top_k, int num_experts, int block_m,
                                   int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_padded,
                                   void* workspace, void* stream) {
    using namespace amoe_aux;
    if (M <= 0 || top_k <= 0) return fail(ALPHA_MOE_E_ARG, "M and top_k must be positive");
    const long long numel = static_cast<long long>(M) * top_k;
    if (numel > 0x7FFFFFFFLL) return fail(ALPHA_MOE_E_ARG, "M*top_k overflows int32");
    // every argument is checked before anything touches a device or a stream
    if (!x_bf16 || !x_fp8 || !x_scale || !topk_ids || !sorted_token_ids || !expert_ids || !num_tokens_post_padded)
        return fail(ALPHA_MOE_E_ARG, "null pointer argument");
    if (K <= 0 || K % 128 != 0) return fail(ALPHA_MOE_E_ARG, "need M > 0 and K a positive multiple of 128");
    if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) || (reinterpret_cast<uintptr_t>(x_fp8) & 15))
        return fail(ALPHA_MOE_E_ARG, "x_bf16 and x_fp8 must be 16-byte aligned");
    if (num_experts <= 0 || num_experts > kMaxExperts)
        return fail(ALPHA_MOE_E_ARG, "num_experts must be in 1..%d (got %d)", kMaxExperts, num_experts);
    if (block_m <= 0) return fail(ALPHA_MOE_E_ARG, "block_m must be positive (got %d)", block_m);
    if (numel > kChunk) {
        // Two launches (the schedule needs several CTAs and a grid-wide barrier) that do not depend on each other: the
        // schedule runs on a side stream forked from the caller's and joined back into it, beside the quantiser.  It
        // is launched first so that its few CTAs have their places before the quantiser's grid fills every SM.
        cudaStream_t user = static_cast<cudaStream_t>(stream);
        int dev = 0;
        AUX_TRY(cudaGetDevice(&dev));
        SideStream* side = side_stream(dev);
        const bool forked = side && cudaEventRecord(side->fork, user) == cudaSuccess &&
                            cudaStreamWaitEvent(side->stream, side->fork, 0) == cudaSuccess;
        const int rc_align = alpha_moe_b200_moe_align_block_size(topk_ids, static_cast<int>(numel), num_experts, block_m,
                                                                 sorted_token_ids, expert_ids, num_tokens_post_padded,
                                                                 workspace, forked ? side->stream : user);
        const int rc_quant = rc_align ? rc_align
                                      : alpha_moe_b200_per_token_group_quant_fp8(x_bf16, x_fp8, x_scale, M, K, zero_src, stream);
        if (forked) {            // joined whatever happened above: the side stream never stays attached to a capture
            AUX_TRY(cudaEventRecord(side->join, side->stream));
            AUX_TRY(cudaStreamWaitEvent(user, side->join, 0));
        }
        return rc_quant;
    }
    const long long sorted_len = numel + static_cast<long long>(num_experts) * (block_m - 1);
    if (sorted_len > 0x7FFFFFFFLL) return fail(ALPHA_MOE_E_ARG, "schedule too long for int32 indices");
    const int n_blocks_max = static_cast<int>((sorted_len + block_m - 1) / block_m);
    const long long n_groups = static_cast<long long>(M) * (K / 128);
    const long long qblocks = (n_groups + 31) / 32;      // at most 1024 * K / 4096 blocks: no cap needed
    quant_and_align_small_kernel<<<static_cast<unsigned>(qblocks + 1), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(x_fp8), x_scale, n_groups, zero_src, topk_ids,
        static_cast<int>(numel), num_experts, block_m, sorted_token_ids, static_cast<int>(sorted_len), expert_ids,
        n_blocks_max, num_tokens_post_padded);
    AUX_TRY(cudaGetLastError());
    return ALPHA_MOE_OK;
}

}  // extern "C"
