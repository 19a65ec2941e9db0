"""An independent comparator for the parity tests: vLLM's Triton block-fp8 fused-MoE pipeline.

The reference's correctness script treats SGLang's Triton pipeline as the truth
(test/test_moe_correctness.py:77-89: invoke_fused_moe_kernel, silu_and_mul, invoke_fused_moe_kernel,
moe_sum_reduce); SGLang took that pipeline from vLLM, whose copy is what this module drives
(vllm.model_executor.layers.fused_moe.fused_moe.fused_experts_impl: per-token-group fp8 quantisation of
the activations, moe_align_block_size, Triton grouped GEMM with 128x128 block scales, silu_and_mul in
bf16, re-quantisation, second grouped GEMM weighted by topk_weights, sum over top_k).  It consumes the
plain [gate; up] weight layout, so the operator-layout weights of a case are de-interleaved first.

TEST INFRASTRUCTURE ONLY: nothing in the product package may import this file or vLLM.
"""
from __future__ import annotations

import os

# On Blackwell vLLM rounds the activation scales of its group quantiser up to powers of two (UE8M0, for
# DeepGEMM) unless told otherwise; the reference's comparator (SGLang on Hopper) and the operator's contract
# use plain fp32 scales = amax/448, so the comparator is run that way.  Read by vLLM at first use.
os.environ["VLLM_USE_DEEP_GEMM_E8M0"] = "0"

import torch  # noqa: E402

from oracle import moe_oracle as orc  # noqa: E402


def plain_weights(case: orc.MoeCase):
    """(w13 [E,2I,K] fp8 in [gate; up] layout, its block scales) from the operator-layout tensors."""
    w13 = orc.deinterleave_rows(case.w.view(torch.uint8), 8).view(orc.FP8)
    s13 = orc.deinterleave_rows(case.w_scale.float(), 1)
    return w13.contiguous(), s13.contiguous()


def vllm_fused_moe(case: orc.MoeCase, dev="cuda:0") -> torch.Tensor:
    """bf16(scaling * vLLM's fused MoE) for `case` on CPU; needs case.x_bf16 (vLLM quantises the activations itself)."""
    from vllm.model_executor.layers.fused_moe.fused_moe import fused_experts_impl
    assert case.x_bf16 is not None, "the comparator quantises the bf16 activations itself"
    w13, s13 = plain_weights(case)
    out = fused_experts_impl(
        case.x_bf16.to(dev).contiguous(), w13.to(dev), case.w2.to(dev).contiguous(),
        case.topk_weights.to(dev).float().contiguous(), case.topk_ids.to(dev).contiguous(), inplace=False,
        activation="silu", use_fp8_w8a8=True, per_channel_quant=False, global_num_experts=case.num_experts,
        w1_scale=s13.to(dev), w2_scale=case.w2_scale.to(dev).float().contiguous(), block_shape=[128, 128])
    torch.cuda.synchronize()
    return (out.float() * float(case.scaling_factor)).to(torch.bfloat16).cpu()


def vllm_group_quant(x_bf16: torch.Tensor, dev="cuda:0"):
    """(fp8, f32 scales) of vLLM's per-token-group-128 quantiser, on CPU."""
    from vllm.model_executor.layers.quantization.utils.fp8_utils import per_token_group_quant_fp8
    q, s = per_token_group_quant_fp8(x_bf16.to(dev).contiguous(), 128)
    torch.cuda.synchronize()
    return q.cpu(), s.float().cpu().contiguous()


def vllm_align(topk_ids: torch.Tensor, block: int, num_experts: int, dev="cuda:0"):
    """(sorted_token_ids, expert_ids, num_tokens_post_padded) of vLLM's moe_align_block_size, on CPU."""
    from vllm.model_executor.layers.fused_moe.moe_align_block_size import moe_align_block_size
    sid, eid, npp = moe_align_block_size(topk_ids.to(dev).to(torch.int32).contiguous(), block, num_experts)
    torch.cuda.synchronize()
    return sid.cpu(), eid.cpu(), npp.cpu()
