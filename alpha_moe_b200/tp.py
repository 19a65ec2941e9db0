"""Tensor parallelism over the intermediate dimension for the fused MoE operator.

The reference has no collective code: the serving engine hands the operator a weight shard of
N = 2*I/tp rows ("tailored for TP servings", reference README.md:1) and all-reduces the partial
outputs in its own model code after extra/sglang.patch:38-41.  These helpers make that contract
explicit: how to cut the operator-layout tensors, and the one exchange step (sum of bf16 partials).

Slicing is exact because SwiGLU is element-wise in the intermediate dimension, the re-quantisation
group (128) divides I/tp, and the 8-row gate/up interleave is local to 16-row groups.
"""
from __future__ import annotations

import torch


def shard_weights(w, w_scale, w2, w2_scale, rank: int, tp: int):
    """Rank `rank`'s shard of operator-layout weights.

    w [E, 2I, K] (interleaved by 8) -> rows [rank*2I/tp, (rank+1)*2I/tp)
    w_scale [E, 2I/128, K/128] (interleaved by 1) -> the matching scale rows
    w2 [E, K, I] -> columns [rank*I/tp, (rank+1)*I/tp) (made contiguous)
    w2_scale [E, K/128, I/128] -> the matching scale columns
    """
    e, n, k = w.shape
    inter = n // 2
    if inter % tp != 0 or (inter // tp) % 128 != 0:
        raise ValueError(f"I={inter} must split into tp={tp} shards that are multiples of 128")
    ish = inter // tp
    rows = slice(rank * 2 * ish, (rank + 1) * 2 * ish)
    srows = slice(rank * 2 * ish // 128, (rank + 1) * 2 * ish // 128)
    cols = slice(rank * ish, (rank + 1) * ish)
    scols = slice(rank * ish // 128, (rank + 1) * ish // 128)
    return (w[:, rows, :].contiguous(), w_scale[:, srows, :].contiguous(),
            w2[:, :, cols].contiguous(), w2_scale[:, :, scols].contiguous())


def tp_layer(compute, out: torch.Tensor, group=None) -> torch.Tensor:
    """One tensor-parallel layer call: zero `out`, run `compute(out)` (this rank's fused operator
    call, accumulating into `out`), then sum the partial outputs over the group in place."""
    import torch.distributed as dist
    out.zero_()
    compute(out)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
    return out


class PeerReducedLayer:
    """Small-batch tensor parallelism without a collective call.  Two forms of the exchange step, both over
    peer-mapped symmetric memory and both closed by a bounded cross-GPU barrier of this library:

      mode="exchange" (default)  every rank's fused kernel accumulates into its own partial buffer; ONE further kernel
                                 then waits for all ranks, sums all ranks' partials with 16-byte loads over NVLink
                                 (fp32, in rank order: every rank gets the same bits) and clears this rank's partial
                                 buffer of the next step (alpha_moe_b200_tp_exchange_sum);
      mode="epilogue"            the fused kernel's epilogue adds every partial result straight into the output buffers
                                 of all ranks (alpha_moe_b200_fused_moe_w8a8_up_down_tp), then a barrier kernel.  This
                                 sends every (token, expert) row to every peer as 4-byte reductions and measured
                                 slower than an all-reduce at every batch size; it is kept as the reference point.

    Two buffers are used alternately, so that a step needs one barrier only.  Buffers come from
    torch.distributed._symmetric_memory (one process per GPU, NCCL process group up); `max_tokens` x `hidden` bf16 each.
    Meant for blocks of at most 64 assignments (decode-size batches); larger batches run the plain operator followed
    by an all-reduce (`tp_layer`)."""

    def __init__(self, max_tokens: int, hidden: int, group=None, timeout_ms: int = 1000, mode: str = "exchange"):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if mode not in ("exchange", "epilogue"):
            raise ValueError("mode must be 'exchange' or 'epilogue'")
        if hidden % 8 != 0:
            raise ValueError("hidden must be a multiple of 8")
        group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.max_tokens, self.hidden, self.timeout_ms, self.mode = max_tokens, hidden, timeout_ms, mode
        self.out = symm_mem.empty(2, max_tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.flags = symm_mem.empty(16, dtype=torch.int32, device=dev)
        self.out.zero_()
        self.flags.zero_()
        self.result = torch.zeros(2, max_tokens, hidden, dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        h_out = symm_mem.rendezvous(self.out, group.group_name)
        h_flags = symm_mem.rendezvous(self.flags, group.group_name)
        self._out_ptrs = [int(p) for p in h_out.buffer_ptrs]
        self._flag_ptrs = [int(p) for p in h_flags.buffer_ptrs]
        self._handles = (h_out, h_flags)
        self._step = 0
        nbytes = max_tokens * hidden * 2
        self._outs = [[p + j * nbytes for p in self._out_ptrs] for j in (0, 1)]     # per buffer: every rank's address
        self._result_ptr = [self.result[j].data_ptr() for j in (0, 1)]
        dist.barrier(group)             # every rank's buffers are zero before anyone's first step

    def run(self, x, x_scale, w, w_scale, w2, w2_scale, sorted_token_ids, expert_ids, num_tokens_post_padded,
            topk_weights, top_k, block_m, block_n, warp_n, stages, scaling_factor) -> torch.Tensor:
        """One layer call on this rank's weight shard; returns the full (summed over ranks) bf16 [M, K] output, a
        view of a buffer that stays valid until the call after next."""
        from . import capi
        m, k = x.shape
        if m > self.max_tokens or k != self.hidden:
            raise ValueError(f"x is [{m}, {k}], the buffers hold [{self.max_tokens}, {self.hidden}]")
        j = self._step & 1
        self._step += 1
        outs = self._outs[j]
        stream = torch.cuda.current_stream().cuda_stream
        e, n, _ = w.shape
        common = (sorted_token_ids.data_ptr(), expert_ids.data_ptr(), num_tokens_post_padded.data_ptr(),
                  topk_weights.data_ptr(), top_k, m, k, n, e, sorted_token_ids.numel(), block_m, block_n, warp_n, stages,
                  float(scaling_factor), stream)
        tensors = (x.data_ptr(), x_scale.data_ptr(), w.data_ptr(), w_scale.data_ptr(), w2.data_ptr(), w2_scale.data_ptr())
        if self.mode == "epilogue":
            capi.fused_moe_w8a8_up_down_tp(*tensors, outs, self.rank, *common)
            self.out[j ^ 1].zero_()         # the next step's buffer (all of it), cleared before this step's barrier
            capi.tp_barrier(self._flag_ptrs, self.rank, self.timeout_ms, stream)
            return self.out[j, :m]
        capi.fused_moe_w8a8_up_down(*tensors, outs[self.rank], *common)
        capi.tp_exchange_sum(outs, self._result_ptr[j], self._outs[j ^ 1][self.rank], m * k, self.max_tokens * self.hidden,
                             self._flag_ptrs, self.rank, self.timeout_ms, stream)
        return self.result[j, :m]


class PeerAllReduce:
    """Two peer-mapped bf16 `out` buffers of [max_tokens, hidden] per rank and this library's own in-place all-reduce
    over them (alpha_moe_b200_tp_allreduce: two flag barriers, every rank sums its slice of the rows and fetches the
    others'), for batches too large for PeerReducedLayer.  A step is: `buf = ar.next_buffer(m)` (a zeroed [m, hidden]
    view), run the operator into it, `ar.all_reduce()`; `buf` then holds the layer output on every rank and stays
    valid until the call after next."""

    def __init__(self, max_tokens: int, hidden: int, group=None, timeout_ms: int = 1000):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        if hidden % 8 != 0:
            raise ValueError("hidden must be a multiple of 8")
        group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        dev = torch.device("cuda", torch.cuda.current_device())
        self.max_tokens, self.hidden, self.timeout_ms = max_tokens, hidden, timeout_ms
        self.out = symm_mem.empty(2, max_tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.flags = symm_mem.empty(16, dtype=torch.int32, device=dev)
        self.out.zero_()
        self.flags.zero_()
        torch.cuda.synchronize()
        h_out = symm_mem.rendezvous(self.out, group.group_name)
        h_flags = symm_mem.rendezvous(self.flags, group.group_name)
        nbytes = max_tokens * hidden * 2
        self._bufs = [[int(p) + j * nbytes for p in h_out.buffer_ptrs] for j in (0, 1)]
        self._flag_ptrs = [int(p) for p in h_flags.buffer_ptrs]
        self._handles = (h_out, h_flags)
        self._step = 0
        self._cur = None
        dist.barrier(group)

    def next_buffer(self, m: int) -> torch.Tensor:
        if m > self.max_tokens:
            raise ValueError(f"{m} tokens, the buffers hold {self.max_tokens}")
        j = self._step & 1
        self._step += 1
        buf = self.out[j, :m]
        buf.zero_()
        self._cur = (j, m)
        return buf

    def all_reduce(self) -> None:
        from . import capi
        j, m = self._cur
        capi.tp_allreduce(self._bufs[j], m * self.hidden, self._flag_ptrs, self.rank, self.timeout_ms,
                          torch.cuda.current_stream().cuda_stream)

    def reduce_scatter(self) -> torch.Tensor:
        """Sum over all ranks of this rank's share of the rows only (alpha_moe_b200_tp_reduce_scatter): returns the
        [rows of this rank, hidden] view of the current buffer that holds it.  The token count of the step must be a
        multiple of the number of ranks."""
        from . import capi
        j, m = self._cur
        if m % self.world != 0:
            raise ValueError(f"{m} tokens do not split evenly over {self.world} ranks")
        capi.tp_reduce_scatter(self._bufs[j], m * self.hidden, self._flag_ptrs, self.rank, self.timeout_ms,
                               torch.cuda.current_stream().cuda_stream)
        per = m // self.world
        return self.out[j, self.rank * per:(self.rank + 1) * per]
