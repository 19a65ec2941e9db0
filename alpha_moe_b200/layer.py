"""The body the reference's serving patch gives `fused_experts_impl` (extra/sglang.patch:25-40), on this
library's own kernels: knob look-up for the batch size, activation quantisation, clearing of the buffer the
layer accumulates into, block schedule, fused operator.  `hidden_states` holds the layer output on return,
as in the patch.  Buffers come from torch; the work is one C-ABI call."""
from __future__ import annotations

import os

import torch

from . import capi
from .utils import get_best_config


def fused_experts_impl(hidden_states: torch.Tensor, w1: torch.Tensor, w1_scale: torch.Tensor, w2: torch.Tensor,
                       w2_scale: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                       routed_scaling_factor: float | None = None, block_shape=(128, 128),
                       config: dict | str | None = None) -> torch.Tensor:
    """hidden_states bf16 [M,K] (overwritten with the result); w1 fp8 [E,2I,K] gate/up interleaved by 8 with
    w1_scale [E,2I/128,K/128] interleaved by 1; w2 fp8 [E,K,I], w2_scale [E,K/128,I/128]; topk_ids int32 [M,top_k],
    topk_weights f32 [M,top_k].  `config`: a knob dict, a table path, or None for $ALPHA_MOE_CONFIG."""
    if tuple(block_shape) != (128, 128):
        raise ValueError("only 128 x 128 block scales are supported (the operator's scale layout)")
    if not hidden_states.is_cuda or hidden_states.dtype != torch.bfloat16 or hidden_states.dim() != 2 \
            or not hidden_states.is_contiguous():
        raise RuntimeError("hidden_states must be a contiguous 2-D bfloat16 CUDA tensor")
    m, k = hidden_states.shape
    e, n, _ = w1.shape
    top_k = topk_ids.shape[1]
    if isinstance(config, dict):
        conf = config
    else:
        path = config or os.getenv("ALPHA_MOE_CONFIG")
        if not path:
            raise RuntimeError("no knob table: pass config= or set ALPHA_MOE_CONFIG")
        conf = get_best_config(path, m)
    block_m, bn, wn, stages = conf["block_m"], conf["block_n"], conf["warp_n"], conf["stages"]
    dev = hidden_states.device
    ids = topk_ids.to(torch.int32).contiguous()
    wts = topk_weights.to(torch.float32).contiguous()
    numel = m * top_k
    total = numel + e * (block_m - 1)
    x_q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=dev)
    x_s = torch.empty(m, k // 128, dtype=torch.float32, device=dev)
    sorted_ids = torch.empty(total, dtype=torch.int32, device=dev)
    expert_ids = torch.empty((total + block_m - 1) // block_m, dtype=torch.int32, device=dev)
    num_post_pad = torch.empty(1, dtype=torch.int32, device=dev)
    ws_bytes = capi.align_workspace_bytes(numel, e)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        capi.fused_experts(hidden_states.data_ptr(), x_q.data_ptr(), x_s.data_ptr(), w1.data_ptr(), w1_scale.data_ptr(),
                           w2.data_ptr(), w2_scale.data_ptr(), ids.data_ptr(), wts.data_ptr(), top_k, m, k, n, e,
                           sorted_ids.data_ptr(), expert_ids.data_ptr(), num_post_pad.data_ptr(),
                           ws.data_ptr() if ws_bytes else 0, block_m, bn, wn, stages,
                           float(routed_scaling_factor or 1.0), torch.cuda.current_stream(dev).cuda_stream)
    return hidden_states
