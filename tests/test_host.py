"""CPU tests of the host side: layout / table helpers against reference goldens, the C ABI
library (loads, exports every declared symbol, argument validation without touching a GPU)."""
import ctypes
import json
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_interleave_tensor_matches_reference_goldens():
    from alpha_moe_python.utils import interleave_tensor
    g = np.load(os.path.join(GOLD, "ref_interleave.npz"))
    for src, rep, key in (("a", 8, "a_rep8"), ("a", 2, "a_rep2"), ("b", 8, "b_rep8"), ("s", 1, "s_rep1")):
        got = interleave_tensor(torch.from_numpy(g[src]), rep)
        assert got.is_contiguous()
        assert torch.equal(got, torch.from_numpy(g[key]))
    with pytest.raises(ValueError):
        interleave_tensor(torch.zeros(1, 24, 2), 8)


def test_get_best_config_matches_reference_goldens():
    from alpha_moe_python.utils import get_best_config
    with open(os.path.join(GOLD, "ref_best_config.json")) as f:
        want = json.load(f)
    table = os.path.join(GOLD, "best_config_table.json")
    for q, knobs in want.items():
        assert get_best_config(table, int(q)) == knobs


def test_shipped_config_tables_are_valid():
    cfg_dir = os.path.join(ROOT, "configs")
    if not os.path.isdir(cfg_dir):
        pytest.skip("no tuned tables shipped")
    for name in os.listdir(cfg_dir):
        if not name.endswith(".json"):
            continue
        with open(os.path.join(cfg_dir, name)) as f:
            table = json.load(f)
        assert table
        for bucket, knobs in table.items():
            assert int(bucket) > 0
            assert knobs["block_m"] % 8 == 0 and 8 <= knobs["block_m"] <= 128
            assert (knobs["block_n"], knobs["warp_n"]) in ((64, 4), (32, 8))
            assert 1 <= knobs["stages"] <= 5


def _declared_symbols():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names += re.findall(r"\b(alpha_moe_b200_\w+)\s*\(", text)
    return sorted(set(names))


def test_capi_library_exports_every_declared_symbol():
    from alpha_moe_b200 import capi
    names = _declared_symbols()
    assert "alpha_moe_b200_fused_moe_w8a8_up_down" in names
    for n in names:
        assert hasattr(capi.lib, n), f"{n} declared in include/ but not exported"
    assert "sm_100a" in capi.version()


def test_capi_rejects_bad_arguments_without_a_gpu():
    from alpha_moe_b200 import capi
    p = 0x1000   # never dereferenced: validation fails first
    base = dict(x=p, x_scale=p, w=p, w_scale=p, w2=p, w2_scale=p, out=p, sorted_token_ids=p, expert_ids=p,
                num_tokens_post_padded=p, topk_weights=p, top_k=2, M=4, K=512, N=256, num_experts=8,
                sorted_num=128, block_m=16, block_n=32, warp_n=8, stages=3, scaling_factor=1.0)

    def call(**kw):
        a = dict(base, **kw)
        return capi.fused_moe_w8a8_up_down(*a.values())

    for bad, msg in ((dict(K=500), "multiple of 128"), (dict(block_n=64, warp_n=8), "block_n"),
                     (dict(stages=0), "stages"), (dict(stages=6), "stages"), (dict(block_m=12), "block_m"),
                     (dict(block_m=136), "block_m"), (dict(N=384), "multiple of 256"), (dict(M=0), "at least one row"),
                     (dict(x=0), "null"), (dict(w=p + 8), "aligned")):
        with pytest.raises(capi.AlphaMoeError, match=msg):
            call(**bad)


def test_fused_experts_entry_rejects_bad_arguments_without_a_gpu():
    """The single-call layer entry validates before it enqueues anything."""
    from alpha_moe_b200 import capi
    p = 0x1000
    base = dict(hidden_states=p, x_fp8=p, x_scale=p, w=p, w_scale=p, w2=p, w2_scale=p, topk_ids=p, topk_weights=p,
                top_k=2, M=4, K=512, N=256, num_experts=8, sorted_token_ids=p, expert_ids=p,
                num_tokens_post_padded=p, align_workspace=0, block_m=16, block_n=32, warp_n=8, stages=3,
                scaling_factor=1.0)
    for bad, msg in ((dict(hidden_states=0), "null"), (dict(topk_ids=0), "null"), (dict(M=0), "positive"),
                     (dict(block_m=12), "block_m"), (dict(block_m=200), "block_m"), (dict(K=500), "multiple of 128")):
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.fused_experts(*dict(base, **bad).values())


def test_plan_fits_shared_memory_for_every_knob():
    """alpha_moe_b200_plan runs the launcher's own planning code: ring depth, tile, shared memory, slices per CTA,
    K-split and kernel for every knob tuple, slice count and batch regime."""
    from alpha_moe_b200 import capi
    for k in (128, 2048, 4096, 7168):
        for n in (256, 512, 768, 4096):
            for bm in range(8, 129, 8):
                for st in range(1, 6):
                    for bn in (32, 64):
                        for nblocks in (9, 600):
                            depth, bmp, smem, spc, ks, kern = capi.plan(k, bm, st, bn, N=n, num_blocks=nblocks)
                            assert 1 <= depth <= st and bmp >= bm and bmp in (16, 32, 64, 128)
                            assert smem <= 232448
                            assert spc == (2 if bn == 64 and (n // 256) % 2 == 0 else 1)
                            assert kern == (0 if bm <= 64 else 1)
                            assert 1 <= ks <= min(8, k // 128) and (ks == 1 or (bm <= 32 and spc == 1 and nblocks == 9))
    assert capi.plan(7168, 16, 5)[0] == 5
    # A handful of live blocks at the DeepSeek shard shape (two slices each): the largest cluster along K whose
    # copies all fit the device at once, modelled here as 8 GPCs of 18 SMs (a positive num_sms touches no device).
    for nblocks, want in ((1, 8), (8, 8), (9, 6), (12, 6), (13, 4), (16, 4), (17, 3), (24, 3), (25, 2), (36, 2), (37, 1)):
        assert capi.plan(7168, 16, 5, 32, N=512, num_blocks=nblocks)[4] == want, nblocks
    assert capi.plan(256, 16, 5, 32, N=512, num_blocks=1)[4] == 2       # never more CTAs than K chunks
    # a ring shallow enough for two CTAs per SM doubles the room: clusters of an even size fill half as many SMs
    for nblocks, want in ((9, 8), (16, 8), (17, 6), (24, 6), (29, 4), (36, 4), (37, 3), (48, 3), (49, 2), (74, 2), (75, 1)):
        depth, _, smem, _, ks, _ = capi.plan(7168, 16, 2, 32, N=512, num_blocks=nblocks)
        assert ks == want and depth == 2 and smem <= 105 * 1024, nblocks
    with pytest.raises(capi.AlphaMoeError):
        capi.set_ksplit(9)


def test_out_alignment_is_checked_per_kernel_before_anything_is_launched():
    """block_m > 64 accumulates with 16-byte vector reductions: an `out` that is only 4-byte aligned must be
    rejected with an argument error (it would fault on the device); block_m <= 64 accepts it.  The call with
    block_m = 16 gets past the argument checks and fails later (no CUDA device / fake pointers), not with the alignment message."""
    from alpha_moe_b200 import capi
    p = 0x10000
    args = dict(x=p, x_scale=p, w=p, w_scale=p, w2=p, w2_scale=p, out=p + 4, sid=p, eid=p, npp=p, tw=p, top_k=2, M=4,
                K=512, N=256, E=8, sorted_num=128, block_m=128, block_n=64, warp_n=4, stages=3, scaling=1.0)
    with pytest.raises(capi.AlphaMoeError, match="16-byte aligned"):
        capi.fused_moe_w8a8_up_down(*args.values())
    args["out"] = p + 2
    args["block_m"] = 16
    with pytest.raises(capi.AlphaMoeError, match="4-byte aligned"):
        capi.fused_moe_w8a8_up_down(*args.values())


def test_torch_operator_schema_is_the_reference_schema():
    import alpha_moe  # noqa: F401
    schema = str(torch.ops.alpha_moe.fused_moe_w8a8_up_down.default._schema)
    want = ("alpha_moe::fused_moe_w8a8_up_down(Tensor x, Tensor x_scale, Tensor w, Tensor w_scale, Tensor w2, "
            "Tensor w2_scale, Tensor sorted_token_ids, Tensor expert_ids, Tensor num_tokens_post_padded, "
            "Tensor topk_weights, Tensor(a!) out, int top_k, int block_m, int block_n, int warp_n, int stages, "
            "float scaling_factor) -> ()")
    assert schema == want
    # CUDA-only: calling it with CPU tensors must fail, never fall back
    x = torch.zeros(2, 128, dtype=torch.float8_e4m3fn)
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops.alpha_moe.fused_moe_w8a8_up_down(
            x, torch.zeros(2, 1), torch.zeros(1, 256, 128, dtype=torch.float8_e4m3fn), torch.zeros(1, 2, 1),
            torch.zeros(1, 128, 128, dtype=torch.float8_e4m3fn), torch.zeros(1, 1, 1),
            torch.zeros(32, dtype=torch.int32), torch.zeros(2, dtype=torch.int32), torch.zeros(1, dtype=torch.int32),
            torch.zeros(2, 1), torch.zeros(2, 128, dtype=torch.bfloat16), 1, 16, 32, 8, 3, 1.0)


def test_no_product_module_imports_the_oracle():
    pkg = os.path.join(ROOT, "alpha_moe_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "oracle" not in text.replace("# oracle", ""), f"{fn} mentions the oracle"


def test_layer_entry_checks_shapes_strides_and_dtypes_before_taking_pointers():
    """alpha_moe_b200.layer.fused_experts_impl hands raw addresses to the C ABI, so it makes the operator's
    tensor checks itself: a mismatched shard, a non-contiguous view or a wrong dtype raises, nothing is launched."""
    from alpha_moe_b200.layer import _check_layer_arguments, fused_experts_impl
    e, n, k, m, top_k = 4, 256, 256, 3, 2
    good = dict(
        hidden_states=torch.zeros(m, k, dtype=torch.bfloat16),
        w1=torch.zeros(e, n, k, dtype=torch.float8_e4m3fn), w1_scale=torch.zeros(e, n // 128, k // 128),
        w2=torch.zeros(e, k, n // 2, dtype=torch.float8_e4m3fn), w2_scale=torch.zeros(e, k // 128, n // 256),
        topk_weights=torch.zeros(m, top_k), topk_ids=torch.zeros(m, top_k, dtype=torch.int32))
    _check_layer_arguments(**good)
    bad = [
        dict(hidden_states=torch.zeros(m, k)),                                              # dtype
        dict(hidden_states=torch.zeros(m, 2 * k, dtype=torch.bfloat16)[:, ::2]),            # strided view
        dict(w1=torch.zeros(e, n, k // 2, dtype=torch.float8_e4m3fn)),                      # K mismatch
        dict(w1=torch.zeros(e, 2 * n, k, dtype=torch.float8_e4m3fn)[:, ::2]),               # non-contiguous shard
        dict(w2=torch.zeros(e, k, n, dtype=torch.float8_e4m3fn)),                           # w2 != [E, K, N/2]
        dict(w2=torch.zeros(e, k, n // 2, dtype=torch.uint8)),                              # dtype
        dict(w1_scale=torch.zeros(e, n // 128, k // 128 + 1)),
        dict(w2_scale=torch.zeros(e, k // 128, n // 256, dtype=torch.float64)),
        dict(topk_ids=torch.zeros(m + 1, top_k, dtype=torch.int32)),
        dict(topk_weights=torch.zeros(m, top_k + 1)),
    ]
    for change in bad:
        with pytest.raises(RuntimeError):
            _check_layer_arguments(**dict(good, **change))
    with pytest.raises(RuntimeError, match="CUDA"):
        fused_experts_impl(good["hidden_states"], good["w1"], good["w1_scale"], good["w2"], good["w2_scale"],
                           good["topk_weights"], good["topk_ids"], config=dict(block_m=16, block_n=32, warp_n=8, stages=3))


def test_tensor_parallel_entry_points_reject_bad_arguments_before_any_launch():
    from alpha_moe_b200 import capi
    p = 0x10000
    base = dict(x=p, x_scale=p, w=p, w_scale=p, w2=p, w2_scale=p, outs=[p, p], tp_rank=0, sid=p, eid=p, npp=p, tw=p,
                top_k=2, M=4, K=512, N=256, E=8, sorted_num=128, block_m=16, block_n=32, warp_n=8, stages=3, scaling=1.0)
    for bad, msg in ((dict(block_m=128, block_n=64, warp_n=4), "block_m <= 64"), (dict(tp_rank=2), "tp_rank"),
                     (dict(outs=[p] * 9), "tp_world"), (dict(outs=[p, 0]), "null"), (dict(outs=[p, p + 2]), "aligned")):
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.fused_moe_w8a8_up_down_tp(*dict(base, **bad).values())
    for flags, rank, tmo, msg in (([p] * 9, 0, 100, "tp_world"), ([p, p], 3, 100, "tp_rank"), ([p, 0], 0, 100, "null"),
                                  ([p, p], 0, 0, "timeout_ms"), ([p, p], 0, 5000, "timeout_ms")):
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.tp_barrier(flags, rank, tmo)
    for kw, msg in ((dict(count=12), "multiples of 8"), (dict(partials=[p, p + 4]), "misaligned"), (dict(result=0), "null"),
                    (dict(clear_next=0, clear_count=64), "clear_next")):
        a = dict(partials=[p, p], result=p, clear_next=p, count=64, clear_count=64, flags=[p, p], tp_rank=0)
        a.update(kw)
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.tp_exchange_sum(*a.values())
    for bufs, count, msg in (([p, p], 12, "multiple of 8"), ([p, p + 8], 64, "misaligned"), ([p] * 9, 64, "tp_world")):
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.tp_allreduce(bufs, count, [p] * len(bufs), 0)
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.tp_reduce_scatter(bufs, count, [p] * len(bufs), 0)


def test_quant_and_align_entry_rejects_bad_arguments_before_any_launch():
    """alpha_moe_b200_quant_and_align (both steps in front of the operator in one call): argument errors come back as
    error codes from both of its forms - one launch (M * top_k <= 1024) and two launches - without touching a GPU."""
    from alpha_moe_b200 import capi
    p = 0x10000
    base = dict(x_bf16=p, x_fp8=p, x_scale=p, M=4, K=512, zero_src=1, topk_ids=p, top_k=2, num_experts=8, block_m=16,
                sorted_token_ids=p, expert_ids=p, num_tokens_post_padded=p)
    for bad, msg in ((dict(M=0), "positive"), (dict(top_k=0), "positive"), (dict(x_fp8=0), "null"), (dict(topk_ids=0), "null"),
                     (dict(K=500), "multiple of 128"), (dict(x_bf16=p + 8), "aligned"), (dict(num_experts=5000), "num_experts"),
                     (dict(block_m=0), "block_m"),
                     (dict(M=4096, x_scale=0), "null"), (dict(M=4096, K=100), "multiple of 128"),
                     (dict(M=4096, x_bf16=p + 8), "aligned")):
        with pytest.raises(capi.AlphaMoeError, match=msg):
            capi.quant_and_align(*dict(base, **bad).values())
