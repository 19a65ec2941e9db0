"""Python wrapper and fake (meta) implementation of the operator, mirroring alpha_moe_ops.py:5-88."""
from __future__ import annotations

import torch

from . import load_torch_op

load_torch_op()


@torch.library.register_fake("alpha_moe::fused_moe_w8a8_up_down")
def _fused_moe_w8a8_up_down_fake(x, x_scale, w, w_scale, w2, w2_scale, sorted_token_ids, expert_ids,
                                 num_tokens_post_padded, topk_weights, out, top_k, block_m, block_n,
                                 warp_n, stages, scaling_factor):
    # The operator's schema returns nothing: it mutates `out` in place.
    return None


def fused_moe_w8a8_up_down(x, x_scale, w, w_scale, w2, w2_scale, sorted_token_ids, expert_ids,
                           num_tokens_post_padded, topk_weights, out, top_k, block_m, block_n, warp_n,
                           stages, scaling_factor) -> torch.Tensor:
    """Fused W8A8 MoE expert MLP; accumulates into `out` (bf16 [M,K], zero on entry) and returns it.

    x [M,K] fp8, x_scale [M,K/128]; w [E,N,K] fp8 gate/up interleaved by 8, w_scale [E,N/128,K/128]
    interleaved by 1; w2 [E,K,N/2] fp8, w2_scale [E,K/128,N/256]; sorted_token_ids / expert_ids /
    num_tokens_post_padded from moe_align_block_size(topk_ids, block_m, E); topk_weights [M,top_k] f32.
    block_m must be the block size of that schedule; block_n, warp_n, stages are tuning knobs.
    """
    torch.ops.alpha_moe.fused_moe_w8a8_up_down(
        x, x_scale, w, w_scale, w2, w2_scale, sorted_token_ids, expert_ids, num_tokens_post_padded,
        topk_weights, out, top_k, block_m, block_n, warp_n, stages, scaling_factor)
    return out


__all__ = ["fused_moe_w8a8_up_down"]
