"""ctypes bindings of the C ABI declared in include/alpha_moe_b200.h.

The functions here take raw device addresses (ints) so that they can be driven from torch
tensors (`t.data_ptr()`), cuda-python buffers or anything else; they are what the GPU parity
tests call.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libalpha_moe_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m alpha_moe_b200.build` "
        "(the CUDA library is the only implementation; there is no fallback)")

lib = ctypes.CDLL(LIB_PATH)

_vp, _i, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

lib.alpha_moe_b200_fused_moe_w8a8_up_down.restype = _i
lib.alpha_moe_b200_fused_moe_w8a8_up_down.argtypes = [_vp] * 11 + [_i] * 10 + [_f, _vp]
lib.alpha_moe_b200_fused_moe_w8a8_up_down_tp.restype = _i
lib.alpha_moe_b200_fused_moe_w8a8_up_down_tp.argtypes = [_vp] * 6 + [ctypes.POINTER(_vp), _i, _i] + [_vp] * 4 + [_i] * 10 + [_f, _vp]
lib.alpha_moe_b200_tp_exchange_sum.restype = _i
lib.alpha_moe_b200_tp_exchange_sum.argtypes = [ctypes.POINTER(_vp), _vp, _vp, ctypes.c_longlong, ctypes.c_longlong,
                                               ctypes.POINTER(_vp), _i, _i, _i, _vp]
lib.alpha_moe_b200_tp_allreduce.restype = _i
lib.alpha_moe_b200_tp_allreduce.argtypes = [ctypes.POINTER(_vp), ctypes.c_longlong, ctypes.POINTER(_vp), _i, _i, _i, _vp]
lib.alpha_moe_b200_tp_reduce_scatter.restype = _i
lib.alpha_moe_b200_tp_reduce_scatter.argtypes = [ctypes.POINTER(_vp), ctypes.c_longlong, ctypes.POINTER(_vp), _i, _i, _i, _vp]
lib.alpha_moe_b200_tp_barrier.restype = _i
lib.alpha_moe_b200_tp_barrier.argtypes = [ctypes.POINTER(_vp), _i, _i, _i, _vp]
lib.alpha_moe_b200_read_status.restype = _i
lib.alpha_moe_b200_read_status.argtypes = [ctypes.POINTER(ctypes.c_int32), _i]
lib.alpha_moe_b200_plan.restype = _i
lib.alpha_moe_b200_plan.argtypes = [_i] * 7 + [ctypes.POINTER(ctypes.c_int32)]
lib.alpha_moe_b200_set_ksplit.restype = _i
lib.alpha_moe_b200_set_ksplit.argtypes = [_i]
lib.alpha_moe_b200_moe_align_block_size.restype = _i
lib.alpha_moe_b200_moe_align_block_size.argtypes = [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]
lib.alpha_moe_b200_moe_align_block_size_noalloc.restype = _i
lib.alpha_moe_b200_moe_align_block_size_noalloc.argtypes = [_vp, _i, _i, _i, _vp, _vp, _vp, _vp]
lib.alpha_moe_b200_align_workspace_bytes.restype = ctypes.c_int64
lib.alpha_moe_b200_align_workspace_bytes.argtypes = [_i, _i]
lib.alpha_moe_b200_per_token_group_quant_fp8.restype = _i
lib.alpha_moe_b200_per_token_group_quant_fp8.argtypes = [_vp, _vp, _vp, _i, _i, _i, _vp]
lib.alpha_moe_b200_quant_and_align.restype = _i
lib.alpha_moe_b200_quant_and_align.argtypes = [_vp, _vp, _vp, _i, _i, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]
lib.alpha_moe_b200_fused_experts.argtypes = [_vp] * 9 + [_i] * 5 + [_vp] * 4 + [_i] * 4 + [_f, _vp]
lib.alpha_moe_b200_fused_experts.restype = _i
lib.alpha_moe_b200_selftest_wait_timeout.restype = _i
lib.alpha_moe_b200_selftest_wait_timeout.argtypes = [_i, _i, _i, _vp, _vp]
lib.alpha_moe_b200_last_error.restype = ctypes.c_char_p
lib.alpha_moe_b200_version.restype = ctypes.c_char_p


class AlphaMoeError(RuntimeError):
    pass


def last_error() -> str:
    return lib.alpha_moe_b200_last_error().decode()


def _check(rc: int) -> None:
    if rc != 0:
        raise AlphaMoeError(f"alpha_moe_b200 error {rc}: {last_error()}")


def fused_moe_w8a8_up_down(x, x_scale, w, w_scale, w2, w2_scale, out, sorted_token_ids, expert_ids,
                           num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num,
                           block_m, block_n, warp_n, stages, scaling_factor, stream=0) -> None:
    """Raw call: every tensor argument is a device address (int)."""
    _check(lib.alpha_moe_b200_fused_moe_w8a8_up_down(
        x, x_scale, w, w_scale, w2, w2_scale, out, sorted_token_ids, expert_ids,
        num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num,
        block_m, block_n, warp_n, stages, scaling_factor, stream))


def fused_moe_w8a8_up_down_tp(x, x_scale, w, w_scale, w2, w2_scale, outs, tp_rank, sorted_token_ids, expert_ids,
                              num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num,
                              block_m, block_n, warp_n, stages, scaling_factor, stream=0) -> None:
    """Raw call of the tensor-parallel form: `outs` = device addresses of every rank's output buffer as seen from this
    GPU (outs[tp_rank] is this rank's own); the other tensor arguments are device addresses (ints)."""
    arr = (_vp * len(outs))(*outs)
    _check(lib.alpha_moe_b200_fused_moe_w8a8_up_down_tp(
        x, x_scale, w, w_scale, w2, w2_scale, arr, len(outs), tp_rank, sorted_token_ids, expert_ids,
        num_tokens_post_padded, topk_weights, top_k, M, K, N, num_experts, sorted_num,
        block_m, block_n, warp_n, stages, scaling_factor, stream))


def tp_barrier(flags, tp_rank, timeout_ms=1000, stream=0) -> None:
    """Enqueues the cross-GPU barrier; `flags` = device addresses of every rank's flag array (9 uint32 each)."""
    arr = (_vp * len(flags))(*flags)
    _check(lib.alpha_moe_b200_tp_barrier(arr, len(flags), tp_rank, timeout_ms, stream))


def tp_exchange_sum(partials, result, clear_next, count, clear_count, flags, tp_rank, timeout_ms=1000, stream=0) -> None:
    """Enqueues barrier + sum of all ranks' partial outputs + clearing of the next partial buffer (device addresses)."""
    pa = (_vp * len(partials))(*partials)
    fa = (_vp * len(flags))(*flags)
    _check(lib.alpha_moe_b200_tp_exchange_sum(pa, result, clear_next or None, count, clear_count, fa, len(partials), tp_rank,
                                              timeout_ms, stream))


def tp_allreduce(bufs, count, flags, tp_rank, timeout_ms=1000, stream=0) -> None:
    """Enqueues the in-place all-reduce over the ranks' peer-mapped buffers (device addresses; count in bf16 elements)."""
    ba = (_vp * len(bufs))(*bufs)
    fa = (_vp * len(flags))(*flags)
    _check(lib.alpha_moe_b200_tp_allreduce(ba, count, fa, len(bufs), tp_rank, timeout_ms, stream))


def tp_reduce_scatter(bufs, count, flags, tp_rank, timeout_ms=1000, stream=0) -> None:
    """Enqueues the reduce-scatter over the ranks' peer-mapped buffers: this rank's slice of its own buffer receives
    the sum over all ranks (device addresses; count in bf16 elements)."""
    ba = (_vp * len(bufs))(*bufs)
    fa = (_vp * len(flags))(*flags)
    _check(lib.alpha_moe_b200_tp_reduce_scatter(ba, count, fa, len(bufs), tp_rank, timeout_ms, stream))


def moe_align_block_size(topk_ids, numel, num_experts, block_m, sorted_token_ids, expert_ids,
                         num_tokens_post_padded, workspace=0, stream=0) -> None:
    """Raw call: device addresses (ints); workspace of align_workspace_bytes(numel, num_experts) bytes."""
    _check(lib.alpha_moe_b200_moe_align_block_size(topk_ids, numel, num_experts, block_m, sorted_token_ids,
                                                   expert_ids, num_tokens_post_padded, workspace or None, stream))


def moe_align_block_size_noalloc(topk_ids, numel, num_experts, block_m, sorted_token_ids, expert_ids,
                                 num_tokens_post_padded, stream=0) -> None:
    """Raw call of the variant that uses the library's built-in scratch array (no workspace argument)."""
    _check(lib.alpha_moe_b200_moe_align_block_size_noalloc(topk_ids, numel, num_experts, block_m, sorted_token_ids,
                                                           expert_ids, num_tokens_post_padded, stream))


def align_workspace_bytes(numel: int, num_experts: int) -> int:
    return int(lib.alpha_moe_b200_align_workspace_bytes(numel, num_experts))


def quant_and_align(x_bf16, x_fp8, x_scale, M, K, zero_src, topk_ids, top_k, num_experts, block_m, sorted_token_ids,
                    expert_ids, num_tokens_post_padded, workspace=None, stream=0) -> None:
    """Quantisation of the activations and the block schedule, as one launch when M * top_k <= 1024."""
    _check(lib.alpha_moe_b200_quant_and_align(x_bf16, x_fp8, x_scale, M, K, int(zero_src), topk_ids, top_k, num_experts,
                                              block_m, sorted_token_ids, expert_ids, num_tokens_post_padded, workspace,
                                              stream))


def per_token_group_quant_fp8(x_bf16, x_fp8, x_scale, M, K, zero_src=False, stream=0) -> None:
    """Raw call: device addresses (ints)."""
    _check(lib.alpha_moe_b200_per_token_group_quant_fp8(x_bf16, x_fp8, x_scale, M, K, int(zero_src), stream))


def fused_experts(hidden_states, x_fp8, x_scale, w, w_scale, w2, w2_scale, topk_ids, topk_weights, top_k, M, K, N,
                  num_experts, sorted_token_ids, expert_ids, num_tokens_post_padded, align_workspace, block_m, block_n,
                  warp_n, stages, scaling_factor, stream=0) -> None:
    """Quantise + clear + schedule + fused operator in one call (device addresses as integers)."""
    _check(lib.alpha_moe_b200_fused_experts(hidden_states, x_fp8, x_scale, w, w_scale, w2, w2_scale, topk_ids,
                                            topk_weights, top_k, M, K, N, num_experts, sorted_token_ids, expert_ids,
                                            num_tokens_post_padded, align_workspace, block_m, block_n, warp_n, stages,
                                            scaling_factor, stream))


def selftest_wait_timeout(limit_cycles: int, where: int, iter_: int, result2, stream=0) -> None:
    """Launches the bounded-wait self-test; result2 = device address of two int32 (what the two waits returned)."""
    _check(lib.alpha_moe_b200_selftest_wait_timeout(limit_cycles, where, iter_, result2, stream))


def read_status(reset: bool = False):
    """(code, block, where, iter) of the current device; code 0 = healthy.  Synchronises."""
    buf = (ctypes.c_int32 * 4)()
    _check(lib.alpha_moe_b200_read_status(buf, int(reset)))
    return tuple(buf)


def plan(K: int, block_m: int, stages: int, block_n: int = 32, N: int = 512, num_blocks: int = 1 << 20,
         num_sms: int = 148):
    """(ring_depth, padded_block_m, dynamic_smem_bytes, slices_per_cta, ksplit, kernel) the launcher uses;
    kernel: 0 weight-major, 1 token-major.  num_sms = 0 asks the current device for its cluster capacity (as a
    launch does); a positive count models it and touches no device."""
    buf = (ctypes.c_int32 * 6)()
    _check(lib.alpha_moe_b200_plan(K, N, block_m, block_n, stages, num_blocks, num_sms, buf))
    return tuple(buf)


def set_ksplit(ksplit: int = 0) -> None:
    """Tuning hook: CTAs per cluster along K for small batches (0 = automatic)."""
    _check(lib.alpha_moe_b200_set_ksplit(ksplit))


def version() -> str:
    return lib.alpha_moe_b200_version().decode()
