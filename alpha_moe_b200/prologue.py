"""The two steps a serving engine runs right before the fused operator, with the names and the
return conventions of the functions the reference imports from SGLang for them
(jit_moe.py:4-9,142,158; extra/sglang.patch:11-13,30-35).  Both run CUDA kernels of this library;
torch is used only to allocate the outputs and to pick the stream."""
from __future__ import annotations

import torch

from . import capi


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """(sorted_token_ids, expert_ids, num_tokens_post_padded) for topk_ids [M, top_k] (int32, CUDA)."""
    if not topk_ids.is_cuda:
        raise RuntimeError("moe_align_block_size needs a CUDA tensor (there is no CPU implementation)")
    ids = topk_ids.to(torch.int32).contiguous()
    numel = ids.numel()
    total = numel + num_experts * (block_size - 1)
    dev = ids.device
    sorted_ids = torch.empty(total, dtype=torch.int32, device=dev)
    expert_ids = torch.empty((total + block_size - 1) // block_size, dtype=torch.int32, device=dev)
    num_post_pad = torch.empty(1, dtype=torch.int32, device=dev)
    ws_bytes = capi.align_workspace_bytes(numel, num_experts)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        capi.moe_align_block_size(ids.data_ptr(), numel, num_experts, block_size, sorted_ids.data_ptr(),
                                  expert_ids.data_ptr(), num_post_pad.data_ptr(), ws.data_ptr() if ws_bytes else 0,
                                  torch.cuda.current_stream(dev).cuda_stream)
    return sorted_ids, expert_ids, num_post_pad


def per_token_group_quant_fp8(x: torch.Tensor, group_size: int = 128, zero_input: bool = False):
    """(x_q fp8 e4m3 [M,K], x_scale f32 [M,K/128]) for bf16 x [M,K]; zero_input=True also clears x,
    which the call site does next because the operator accumulates into that buffer."""
    if group_size != 128:
        raise ValueError("only group_size=128 is supported (the operator's scale layout)")
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2:
        raise RuntimeError("x must be a contiguous 2-D bfloat16 CUDA tensor")
    m, k = x.shape
    x_q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=x.device)
    x_s = torch.empty(m, k // 128, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        capi.per_token_group_quant_fp8(x.data_ptr(), x_q.data_ptr(), x_s.data_ptr(), m, k, zero_input,
                                       torch.cuda.current_stream(x.device).cuda_stream)
    return x_q, x_s


sglang_per_token_group_quant_fp8 = per_token_group_quant_fp8   # the name used at the reference's call sites


def quant_and_align(x: torch.Tensor, topk_ids: torch.Tensor, block_size: int, num_experts: int,
                    zero_input: bool = False):
    """Both steps above in one call: (x_q, x_scale, sorted_token_ids, expert_ids, num_tokens_post_padded), the same
    bits as per_token_group_quant_fp8 + moe_align_block_size.  One kernel launch when M * top_k <= 1024."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2:
        raise RuntimeError("x must be a contiguous 2-D bfloat16 CUDA tensor")
    if not topk_ids.is_cuda or topk_ids.dim() != 2 or topk_ids.shape[0] != x.shape[0]:
        raise RuntimeError("topk_ids must be a CUDA tensor of shape [M, top_k]")
    m, k = x.shape
    ids = topk_ids.to(torch.int32).contiguous()
    numel = ids.numel()
    total = numel + num_experts * (block_size - 1)
    dev = x.device
    x_q = torch.empty(m, k, dtype=torch.float8_e4m3fn, device=dev)
    x_s = torch.empty(m, k // 128, dtype=torch.float32, device=dev)
    sorted_ids = torch.empty(total, dtype=torch.int32, device=dev)
    expert_ids = torch.empty((total + block_size - 1) // block_size, dtype=torch.int32, device=dev)
    num_post_pad = torch.empty(1, dtype=torch.int32, device=dev)
    ws_bytes = capi.align_workspace_bytes(numel, num_experts)
    ws = torch.empty(max(ws_bytes, 4), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        capi.quant_and_align(x.data_ptr(), x_q.data_ptr(), x_s.data_ptr(), m, k, zero_input, ids.data_ptr(),
                             ids.shape[1], num_experts, block_size, sorted_ids.data_ptr(), expert_ids.data_ptr(),
                             num_post_pad.data_ptr(), ws.data_ptr() if ws_bytes else 0,
                             torch.cuda.current_stream(dev).cuda_stream)
    return x_q, x_s, sorted_ids, expert_ids, num_post_pad
