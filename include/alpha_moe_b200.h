/* C ABI of the B200 (sm_100a) fused W8A8 MoE library, libalpha_moe_b200.so.
 *
 * Every entry point takes plain device pointers and sizes - no torch types - and returns 0 on
 * success or a negative ALPHA_MOE_E_* code; alpha_moe_b200_last_error() then gives the message
 * of the failing call on the calling thread.  Nothing here allocates device memory unless the
 * comment of the entry point says so.  All work is enqueued on `stream` (a cudaStream_t passed
 * as void*, NULL = default stream) and is asynchronous with respect to the host.
 *
 * Citations are into the reference project (Aleph-Alpha/Alpha-MoE).
 */
#ifndef ALPHA_MOE_B200_H_
#define ALPHA_MOE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ALPHA_MOE_OK 0
#define ALPHA_MOE_E_ARG (-1)     /* argument rejected (shape, knob, alignment, null pointer) */
#define ALPHA_MOE_E_CUDA (-2)    /* a CUDA runtime / driver call failed */
#define ALPHA_MOE_E_DEVICE (-3)  /* the kernel reported a run-out wait through its status word */

/* Replaces: void fused_moe_w8a8_wgmma_up_down_acc(...) declared at csrc/torch_interface.cpp:12-34 and
 * defined at csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:1258-1303 (the launcher the
 * torch operator calls).  Same arguments in the same order and meaning:
 *   x [M,K] fp8 e4m3, x_scale [M,K/128] f32, w [E,N,K] fp8 (gate/up rows interleaved by 8),
 *   w_scale [E,N/128,K/128] f32 (interleaved by 1), w2 [E,K,N/2] fp8, w2_scale [E,K/128,N/256] f32,
 *   out [M,K] bf16 - must be zero on entry, results are accumulated in place,
 *   sorted_token_ids [sorted_num] i32, expert_ids [ceil(sorted_num/block_m)] i32,
 *   num_tokens_post_padded [1] i32, topk_weights [M,top_k] f32.
 * block_m is semantic (the block size given to moe_align_block_size); block_n/warp_n/stages are the
 * reference's tuning knobs and are validated like csrc/torch_interface.cpp:62-64:
 * (block_n,warp_n) in {(64,4),(32,8)}, 1 <= stages <= 5, block_m in {8,16,...,128}.
 * Here stages = depth of the shared-memory ring (lowered if it would not fit), and block_n = 64
 * selects the variant in which one CTA owns two 128-column slices of the intermediate dimension.
 * Requires K % 128 == 0, N % 256 == 0, 16-byte aligned w / w2 / x; `out` 4-byte aligned for block_m <= 64 and
 * 16-byte aligned for block_m > 64 (those kernels accumulate with 16-byte vector reductions). */
int alpha_moe_b200_fused_moe_w8a8_up_down(
    const void* x, const float* x_scale, const void* w, const float* w_scale, const void* w2,
    const float* w2_scale, void* out, const int32_t* sorted_token_ids, const int32_t* expert_ids,
    const int32_t* num_tokens_post_padded, const float* topk_weights, int top_k, int M, int K, int N,
    int num_experts, int sorted_num, int block_m, int block_n, int warp_n, int stages,
    float scaling_factor, void* stream);

/* Tensor-parallel form of the operator with the exchange step fused into the kernel's epilogue, for small batches
 * (block_m <= 64); no counterpart in the reference, whose caller all-reduces the partial outputs afterwards
 * (extra/sglang.patch:38-41, README.md:1).  Arguments as above, except that `out` becomes `outs`: a HOST array of
 * tp_world device pointers, outs[r] = rank r's [M,K] bf16 output buffer mapped into this GPU's address space
 * (CUDA IPC / virtual-memory export, e.g. torch.distributed._symmetric_memory); outs[tp_rank] is this GPU's own.
 * Every rank runs the call on its shard of the intermediate dimension with the same x / routing / schedule, and each
 * partial result is added into all tp_world buffers with plain reductions over NVLink, so that after a cross-GPU
 * barrier (alpha_moe_b200_tp_barrier) every rank holds the full layer output and no collective call is needed.
 * All tp_world buffers must be zero before ANY rank starts: clear a buffer before the barrier of the previous step
 * (use two buffers alternately).  tp_world <= 8.  The kernel itself waits for no other GPU. */
int alpha_moe_b200_fused_moe_w8a8_up_down_tp(
    const void* x, const float* x_scale, const void* w, const float* w_scale, const void* w2,
    const float* w2_scale, void* const* outs, int tp_world, int tp_rank, const int32_t* sorted_token_ids,
    const int32_t* expert_ids, const int32_t* num_tokens_post_padded, const float* topk_weights, int top_k, int M,
    int K, int N, int num_experts, int sorted_num, int block_m, int block_n, int warp_n, int stages,
    float scaling_factor, void* stream);

/* Barrier over the tp_world GPUs of the fused tensor-parallel path, enqueued on `stream` (no counterpart in the
 * reference).  flags: HOST array of tp_world device pointers, flags[r] = rank r's flag array of 10 uint32 in memory
 * that every rank can write (symmetric memory), all zero before the first barrier.  Work enqueued on this stream
 * before the barrier on every rank (the reductions of alpha_moe_b200_fused_moe_w8a8_up_down_tp, the clearing of the
 * next buffer) is complete and visible on every rank once the barrier has passed there.  The wait is bounded: after
 * timeout_ms (1..2000) the kernel records {code 1, this rank, 90 + the rank that did not arrive, epoch} in the status
 * word and returns; read it with alpha_moe_b200_read_status.  Nothing traps. */
int alpha_moe_b200_tp_barrier(void* const* flags, int tp_world, int tp_rank, int timeout_ms, void* stream);

/* Exchange step of tensor parallelism for small batches as ONE kernel of this library instead of a collective call
 * (no counterpart in the reference; its caller all-reduces, extra/sglang.patch:38-41): barrier over the ranks, then
 * this rank sums the partial outputs of all ranks - partials[r] = rank r's bf16 buffer of `count` elements, mapped
 * into this GPU's address space, read with plain 16-byte loads over NVLink, summed in fp32 in rank order (every rank
 * obtains the same bits) - into `result` (this GPU's memory, bf16, `count` elements), and clears `clear_count` bf16
 * elements at `clear_next` (this rank's partial buffer of the NEXT step; may be NULL with clear_count 0).
 * Use two partial buffers alternately: a rank may overwrite a partial buffer only after the exchange of the following
 * step has passed its barrier, which the fused clear guarantees.  flags as for alpha_moe_b200_tp_barrier, 10 words per
 * rank.  count, clear_count: multiples of 8; all buffers 16-byte aligned.  Bounded wait as in alpha_moe_b200_tp_barrier;
 * after a run-out wait `result` is not written. */
int alpha_moe_b200_tp_exchange_sum(void* const* partials, void* result, void* clear_next, long long count,
                                   long long clear_count, void* const* flags, int tp_world, int tp_rank, int timeout_ms,
                                   void* stream);

/* In-place all-reduce (sum, bf16) of the ranks' partial outputs as ONE kernel of this library, for batches whose
 * payload is too large for alpha_moe_b200_tp_exchange_sum's every-rank-reads-everything (no counterpart in the
 * reference).  bufs[r] = rank r's buffer of `count` bf16 elements, mapped into this GPU's address space; on return
 * (stream order) bufs[tp_rank] holds the sum over all ranks, the same bits on every rank.  Two phases with a bounded
 * flag barrier before each: every rank sums its 1/tp_world slice over all ranks and writes it back into its own
 * buffer, then copies the other slices from their owners; each rank reads 2 (tp_world-1)/tp_world of the payload over
 * NVLink with plain 16-byte loads.  flags as for alpha_moe_b200_tp_barrier (10 zeroed uint32 per rank, shared with
 * the other tensor-parallel entry points).  Use two buffers alternately: a rank may clear and refill a buffer only
 * after the all-reduce of the following step has started everywhere, which stream order gives when the next step uses
 * the other buffer.  count: multiple of 8; buffers 16-byte aligned. */
int alpha_moe_b200_tp_allreduce(void* const* bufs, long long count, void* const* flags, int tp_world, int tp_rank,
                                int timeout_ms, void* stream);

/* The first half of the all-reduce above for callers whose next operator takes row shards (sequence-parallel layers):
 * same arguments, same flag protocol and barriers, but the kernel stops after every rank has summed ITS slice, so each
 * rank reads (tp_world-1)/tp_world of the payload over NVLink instead of twice that.  On return bufs[tp_rank] holds
 * the sum over all ranks in elements [tp_rank * per, min(count, (tp_rank + 1) * per)), per = 8 * ceil(count / 8 /
 * tp_world) (whole rows when the token count is a multiple of tp_world and the row length of 8); the rest of the
 * buffer holds this rank's partial values.  No rank reads a peer's buffer after the kernel's closing barrier, so a
 * buffer may be cleared and reused as soon as the call has completed in stream order. */
int alpha_moe_b200_tp_reduce_scatter(void* const* bufs, long long count, void* const* flags, int tp_world, int tp_rank,
                                     int timeout_ms, void* stream);

/* Replaces the external moe_align_block_size the reference calls before the operator
 * (jit_moe.py:158, extra/sglang.patch:33-35).  topk_ids [numel] i32 (the flattened [M,top_k] expert
 * ids; ids outside [0,num_experts) are ignored).  Outputs: sorted_token_ids
 * [numel + num_experts*(block_m-1)] - each expert's flat indices in ascending order, starting at a
 * multiple of block_m, unused slots = numel; expert_ids [ceil(that length / block_m)] - expert of each
 * used block, 0 for unused ones; num_tokens_post_padded [1].  num_experts <= 1024.
 * workspace: device scratch of alpha_moe_b200_align_workspace_bytes(numel, num_experts) bytes
 * (0 - and workspace may be NULL - when numel <= 1024). */
int alpha_moe_b200_moe_align_block_size(const int32_t* topk_ids, int numel, int num_experts, int block_m,
                                        int32_t* sorted_token_ids, int32_t* expert_ids,
                                        int32_t* num_tokens_post_padded, void* workspace, void* stream);
int64_t alpha_moe_b200_align_workspace_bytes(int numel, int num_experts);

/* No counterpart in the reference.  Same result as alpha_moe_b200_moe_align_block_size, for callers
 * that must not allocate device memory around the call: code running inside a CUDA-graph capture or a
 * serving loop with a frozen memory pool, plugins that are handed buffers but no allocator, and embedders
 * whose device-memory budget is fixed at start-up.  The per-chunk histogram table lives in a 256 KB array
 * compiled into the library (held by every GPU that loads it, until exit) instead of a workspace.
 * Limit: ceil(numel/1024) * num_experts <= 65536 (e.g. 8192 tokens x top_k 9 with 257 experts uses 18504);
 * larger problems are rejected with ALPHA_MOE_E_ARG.  The call itself performs no cudaMalloc / cudaFree and
 * calls no allocating library routine.  The first call on each device looks up the array's device address;
 * make that first call outside any stream capture.  All calls share the one array and nothing in it is
 * assumed zero on entry, but two calls whose kernels overlap on the GPU (different streams, several host
 * threads) race on it: serialise them. */
int alpha_moe_b200_moe_align_block_size_noalloc(const int32_t* topk_ids, int numel, int num_experts, int block_m,
                                                int32_t* sorted_token_ids, int32_t* expert_ids,
                                                int32_t* num_tokens_post_padded, void* stream);

/* Replaces the external sglang_per_token_group_quant_fp8(x, 128) the reference calls before the
 * operator (jit_moe.py:142, extra/sglang.patch:30): bf16 [M,K] -> fp8 e4m3 [M,K] + f32 scale [M,K/128],
 * scale = max(amax,1e-10)/448.  If zero_src != 0 the bf16 source is zeroed after it has been read,
 * which is what the call site does next (extra/sglang.patch:31) because `out` aliases it.
 * x_bf16 and x_fp8 must be 16-byte aligned. */
int alpha_moe_b200_per_token_group_quant_fp8(void* x_bf16, void* x_fp8, float* x_scale, int M, int K,
                                             int zero_src, void* stream);

/* The two steps in front of the operator at the reference's call sites - the quantisation above (jit_moe.py:142,
 * extra/sglang.patch:30-31) and the block schedule (jit_moe.py:158, extra/sglang.patch:33-35) - are independent of
 * each other.  This entry runs both: as ONE launch when the schedule fits one CTA (M * top_k <= 1024: decode-size
 * batches, where a launch costs about as much as either step), otherwise as the two launches above side by side - the
 * schedule on a stream of the library's own that is forked from `stream` and joined back into it before the call
 * returns (capturable; one such stream and two events per host thread and device, created at the first use: make that
 * first call outside any stream capture).  Outputs are
 * bit-identical to alpha_moe_b200_per_token_group_quant_fp8 + alpha_moe_b200_moe_align_block_size with the same
 * arguments (numel = M * top_k; workspace as for that entry, unused for M * top_k <= 1024). */
int alpha_moe_b200_quant_and_align(void* x_bf16, void* x_fp8, float* x_scale, int M, int K, int zero_src,
                                   const int32_t* topk_ids, int top_k, int num_experts, int block_m,
                                   int32_t* sorted_token_ids, int32_t* expert_ids, int32_t* num_tokens_post_padded,
                                   void* workspace, void* stream);

/* The whole call-site sequence of the reference's serving patch as one call (extra/sglang.patch:25-40, the body
 * it gives fused_experts_impl): quantise the bf16 activations per token and 128-group, clear them (the layer's
 * output accumulates into the same buffer), build the block schedule for `block_m`, run the fused operator.
 * hidden_states: bf16 [M,K], activations on entry, layer output on return.  Scratch, all caller-owned device
 * memory: x_fp8 [M,K] bytes, x_scale [M,K/128] f32, sorted_token_ids [M*top_k + num_experts*(block_m-1)] i32,
 * expert_ids [ceil(that / block_m)] i32, num_tokens_post_padded [1] i32, align_workspace of
 * alpha_moe_b200_align_workspace_bytes(M*top_k, num_experts) bytes (may be NULL when that is 0).
 * Everything is enqueued on `stream`; nothing is allocated.  Error codes as for the single steps. */
int alpha_moe_b200_fused_experts(void* hidden_states, void* x_fp8, float* x_scale, const void* w,
                                 const float* w_scale, const void* w2, const float* w2_scale,
                                 const int32_t* topk_ids, const float* topk_weights, int top_k, int M, int K, int N,
                                 int num_experts, int32_t* sorted_token_ids, int32_t* expert_ids,
                                 int32_t* num_tokens_post_padded, void* align_workspace, int block_m, int block_n,
                                 int warp_n, int stages, float scaling_factor, void* stream);

/* Reads (and optionally clears) the status word of the current device: out4 = {code, block, where, iter};
 * code 0 means no kernel wait has ever run out.  Synchronises the device. */
int alpha_moe_b200_read_status(int32_t* out4, int reset);

/* Self-test of the bounded device waits (no counterpart in the reference, whose wait at
 * csrc/kernels/fused_moe_w8a8/fused_moe_w8a8_up_down_acc.cu:563-575 spins without limit).  Launches one small CTA
 * in which one warp waits, with a limit of `limit_cycles` SM clocks, on an mbarrier that nothing ever arrives on,
 * and a second warp waits on another such barrier with the product kernels' own limit.  The first wait runs out,
 * records {code = 1 (wait ran out), block = 0, where, iter} in the device status word and raises the CTA's abort flag,
 * which releases the second waiter; the kernel then returns normally (nothing traps or faults, the context stays
 * usable).  result2 (device, 2 x int32) receives what the two waits returned: 0 = gave up.  Read the status word
 * with alpha_moe_b200_read_status afterwards (and clear it).  limit_cycles in 1000..200000000. */
int alpha_moe_b200_selftest_wait_timeout(int limit_cycles, int where, int iter, int32_t* result2, void* stream);

/* What the launcher uses for a problem and a knob tuple; for tuners and tests.  It runs the launcher's own
 * planning code.  num_blocks = live upper bound of schedule blocks, min(ceil(sorted_num / block_m), M * top_k);
 * num_sms = SM count of a device (148 on B200): the cluster capacity that decides ksplit is then modelled (GPCs of
 * about 18 SMs; one CTA per SM, two when the ring is shallow enough for two to share an SM) and nothing touches a
 * device; num_sms = 0 = the current device, whose driver is asked as a launch would (launches nothing).  out6 = {ring_depth, padded_block_m, dynamic_smem_bytes,
 * slices_per_cta (2 when block_n = 64 and N/256 is even), ksplit (CTAs per cluster along K, small batches: the
 * largest of 2..8 for which all (block, slice) units get their cluster at the same time, else 1),
 * kernel (0 weight-major, 1 token-major)}. */
int alpha_moe_b200_plan(int K, int N, int block_m, int block_n, int stages, int num_blocks, int num_sms,
                        int32_t* out6);

/* Tuning hook (tuners, tests): forces the number of CTAs per cluster along K for small batches; 0 = automatic
 * choice (the default), otherwise 1..8.  Process-wide.  No counterpart in the reference. */
int alpha_moe_b200_set_ksplit(int ksplit);

const char* alpha_moe_b200_last_error(void);
const char* alpha_moe_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ALPHA_MOE_B200_H_ */
