"""Weight-layout and tuning-table helpers with the reference's names and semantics
(alpha_moe_python/utils.py:5-29)."""
from __future__ import annotations

import functools
import json

import torch


def interleave_tensor(tensor: torch.Tensor, rep: int = 8) -> torch.Tensor:
    """[E, N, K] with rows [gate; up] -> groups of `rep` gate rows followed by `rep` up rows.

    Weights use rep=8, block scales rep=1 (reference README.md:96-102).  New row
    c*2*rep + h*rep + r is old row h*N/2 + c*rep + r.
    """
    e, n, k = tensor.shape
    if n % (2 * rep) != 0:
        raise ValueError(f"N={n} must be a multiple of 2*rep={2 * rep}")
    halves = tensor.reshape(e, 2, n // (2 * rep), rep, k)
    return halves.transpose(1, 2).reshape(e, n, k).contiguous()


@functools.lru_cache()
def get_best_config(path: str, n_tokens: int):
    """Knobs {block_m, block_n, warp_n, stages} of the M bucket nearest to n_tokens; on a tie the
    bucket that appears first in the file wins (reference utils.py:19-29)."""
    with open(path, "r") as f:
        table = json.load(f)
    best, best_dist = None, float("inf")
    for bucket, knobs in table.items():
        dist = abs(int(bucket) - n_tokens)
        if dist < best_dist:
            best, best_dist = knobs, dist
    return best
