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
