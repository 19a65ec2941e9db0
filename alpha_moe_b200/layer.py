"""The body the reference's serving patch gives `fused_experts_impl` (extra/sglang.patch:25-40), on this
library's own kernels: knob look-up for the batch size, activation quantisation, clearing of the buffer the
layer accumulates into, block schedule, fused operator.  `hidden_states` holds the layer output on return,
as in the patch.  Buffers come from torch; the work is one C-ABI call."""
from __future__ import annotations

import os

import torch

from . import capi
from .utils import get_best_config


def _check_layer_arguments(hidden_states, w1, w1_scale, w2, w2_scale, topk_weights, topk_ids) -> None:
    """The checks the torch operator makes on its tensors (csrc/torch_interface.cpp:58-76 of the reference, plus
    the dtype / device / shape checks this library's operator adds), made here before any raw pointer is taken:
    this path goes straight to the C ABI, which sees only addresses."""
    def need(cond, msg):
        if not cond:
            raise RuntimeError(msg)
    need(hidden_states.dtype == torch.bfloat16 and hidden_states.dim() == 2 and hidden_states.is_contiguous(),
         "hidden_states must be a contiguous 2-D bfloat16 tensor")
    dev = hidden_states.device
    m, k = hidden_states.shape
    need(m > 0, "hidden_states must have at least one row")
    need(k % 128 == 0, "K dimension must be a multiple of 128")
    need(w1.dim() == 3 and w2.dim() == 3, "w1 must be [E, 2I, K] and w2 [E, K, I]")
    e, n, kw = w1.shape
    need(kw == k, "w1.size(2) must equal hidden_states.size(1)")
    need(n % 256 == 0, "N (2 x intermediate size) must be a multiple of 256")
    need(tuple(w2.shape) == (e, k, n // 2), "w2 must be [E, K, N/2]")
    need(w1.dtype == torch.float8_e4m3fn and w2.dtype == torch.float8_e4m3fn, "w1 and w2 must be float8_e4m3fn")
    need(tuple(w1_scale.shape) == (e, n // 128, k // 128), "w1_scale must be [E, N/128, K/128]")
    need(tuple(w2_scale.shape) == (e, k // 128, n // 256), "w2_scale must be [E, K/128, N/256]")
    need(w1_scale.dtype == torch.float32 and w2_scale.dtype == torch.float32, "weight scales must be float32")
    need(topk_ids.dim() == 2 and topk_ids.shape[0] == m, "topk_ids must be [M, top_k]")
    need(tuple(topk_weights.shape) == tuple(topk_ids.shape), "topk_weights must have the shape of topk_ids")
    for name, t in (("w1", w1), ("w1_scale", w1_scale), ("w2", w2), ("w2_scale", w2_scale)):
        need(t.is_contiguous(), f"{name} must be contiguous")
    for name, t in (("w1", w1), ("w1_scale", w1_scale), ("w2", w2), ("w2_scale", w2_scale),
                    ("topk_weights", topk_weights), ("topk_ids", topk_ids)):
        need(t.device == dev, f"{name} must be on {dev}")


def fused_experts_impl(hidden_states: torch.Tensor, w1: torch.Tensor, w1_scale: torch.Tensor, w2: torch.Tensor,
                       w2_scale: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                       routed_scaling_factor: float | None = None, block_shape=(128, 128),
                       config: dict | str | None = None) -> torch.Tensor:
    """hidden_states bf16 [M,K] (overwritten with the result); w1 fp8 [E,2I,K] gate/up interleaved by 8 with
    w1_scale [E,2I/128,K/128] interleaved by 1; w2 fp8 [E,K,I], w2_scale [E,K/128,I/128]; topk_ids int32 [M,top_k],
    topk_weights f32 [M,top_k].  `config`: a knob dict, a table path, or None for $ALPHA_MOE_CONFIG."""
    if tuple(block_shape) != (128, 128):
        raise ValueError("only 128 x 128 block scales are supported (the operator's scale layout)")
    _check_layer_arguments(hidden_states, w1, w1_scale, w2, w2_scale, topk_weights, topk_ids)
    if not hidden_states.is_cuda:
        raise RuntimeError("hidden_states must be a CUDA tensor (there is no CPU implementation)")
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
