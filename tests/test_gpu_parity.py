"""GPU parity tests: the sm_100a kernel, called through the C ABI, against the CPU oracle on the
same seeded inputs.  Tolerances (floating point, bf16 output accumulated with atomics):
  vs faithful oracle : rel-L2 <= 2e-2 and |d| <= 0.25*rms(ref) + 0.1*|ref| element-wise
  vs ideal oracle    : rel-L2 <= 4e-2
  reference's own    : allclose(atol=2e-2, rtol=1e-1) under its own input distribution
                       (test/test_moe_correctness.py:47-48,106-110,147-155)
"""
import dataclasses
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.harness import check_close, run_capi, run_torch_op, to_device

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")

KNOBS = [(bm, bn, wn, st) for bm in range(8, 129, 8) for bn, wn in ((64, 4), (32, 8)) for st in range(1, 6)]


@pytest.fixture(scope="module")
def cfg0():
    case = orc.make_case(8, 512, 128, 16, 2, seed=0)
    return case, to_device(case)


def test_cfg0_every_knob_combination(cfg0):
    """Config 0 with all 160 (block_m, block_n, warp_n, stages) combinations the operator accepts
    (the reference's sweep, test_moe_correctness.py:171-179), against the oracle and the committed pin."""
    case, dcase = cfg0
    pin = torch.from_numpy(np.load(os.path.join(GOLD, "cfg0_oracle.npz"))["out_faithful"])
    ideal = orc.run_oracle(case, 16, faithful=False, out_fp32=True)
    refs = {}
    for bm, bn, wn, st in KNOBS:
        if bm not in refs:
            refs[bm] = orc.run_oracle(case, bm, out_fp32=True)
            assert orc.rel_l2(refs[bm], pin) < 1e-5
        got = run_capi(case, bm, bn, wn, st, dcase=dcase)
        check_close(got, refs[bm], tag=f"cfg0 {bm},{bn},{wn},{st}")
        assert orc.rel_l2(got, ideal) <= 4e-2


@pytest.mark.parametrize("m", [1, 8, 64, 300])
def test_deepseek_shard_shape_small_expert_count(m):
    """K=7168, I=256, scaling 2.5 as the DeepSeek-V3 TP8 shard, with 16 experts so that the oracle
    finishes in seconds; shared expert always on."""
    w = test_deepseek_shard_shape_small_expert_count.weights
    case = orc.make_case(16, 7168, 256, m, 5, seed=10 + m, shared=True, scaling=2.5, weights=w)
    dcase = to_device(case)
    for bm, st in ((8, 3), (16, 5), (32, 2), (64, 5), (128, 4), (72, 1)):
        if m < bm and bm != 16:
            continue
        ref = orc.run_oracle(case, bm)
        for bn, wn in ((32, 8), (64, 4)):      # one / two intermediate slices per CTA
            got = run_capi(case, bm, bn, wn, st, dcase=dcase)
            check_close(got, ref, tag=f"ds16 M={m} bm={bm} bn={bn}")


test_deepseek_shard_shape_small_expert_count.weights = None


@pytest.fixture(autouse=True, scope="module")
def _ds_weights():
    g = torch.Generator().manual_seed(77)
    test_deepseek_shard_shape_small_expert_count.weights = orc.make_weights(16, 7168, 256, g)
    yield
    test_deepseek_shard_shape_small_expert_count.weights = None


@pytest.mark.parametrize("e,k,inter,m,top_k,bm", [
    (32, 2048, 256, 33, 10, 16),     # Qwen3-Next-like shard
    (8, 128, 128, 5, 2, 8),          # a single K chunk, a single slice
    (8, 384, 128, 40, 3, 24),        # odd number of K chunks: last w2 slot is half empty
    (4, 256, 512, 17, 2, 16),        # four intermediate slices
    (37, 4096, 256, 32, 9, 32),      # reference sweep shape (E=37, K=4096)
    (8, 1280, 384, 64, 4, 128),      # three slices, token-major kernel
    (8, 1024, 512, 200, 4, 128),     # token-major kernel, two slices per CTA
    (8, 1024, 512, 200, 4, 96),      # same, blocks only three quarters full
])
def test_shapes(e, k, inter, m, top_k, bm):
    case = orc.make_case(e, k, inter, m, top_k, seed=e + k + m, scaling=1.0)
    ref = orc.run_oracle(case, bm)
    check_close(run_capi(case, bm, 64, 4, 3), ref, tag=f"E{e} K{k} I{inter} M{m}")


@pytest.mark.parametrize("bm,bn,wn,stages", [(64, 64, 4, 2), (64, 32, 8, 2), (48, 64, 4, 1), (64, 64, 4, 3)])
def test_sixty_four_wide_blocks_two_ctas_per_sm(bm, bn, wn, stages):
    """Blocks of 33..64 assignments with a ring of at most two slots run the single-warpgroup shape of the
    weight-major kernel (two CTAs per SM); deeper rings run the two-warpgroup shape.  Both against the oracle,
    with full blocks, a ragged tail and more CTAs than one wave."""
    case = orc.make_case(24, 2048, 256, 900, 6, seed=64 + stages, shared=True, scaling=2.5)
    check_close(run_capi(case, bm, bn, wn, stages), orc.run_oracle(case, bm), tag=f"bm={bm} bn={bn} st={stages}")


def test_skewed_routing_with_empty_experts():
    """Zipf(1.2) routing: several experts receive nothing, a few receive >10% of the tokens, so the
    schedule has empty experts, multi-block experts and ragged padding."""
    case = orc.make_case(129, 1024, 256, 200, 5, seed=1, shared=True, scaling=2.5, zipf=1.2)
    counts = torch.bincount(case.topk_ids.reshape(-1).long(), minlength=129)
    assert (counts == 0).any() and counts[:-1].max() > 0.1 * 200
    for bm in (16, 64, 128):
        check_close(run_capi(case, bm, 32, 8, 4), orc.run_oracle(case, bm), tag=f"zipf bm={bm}")


# one knob tuple per kernel shape: 16/32/64-wide weight-major (64 in both its shapes), token-major with one and two slices
_GRID_KNOBS = [(8, 32, 8, 3), (16, 64, 4, 5), (32, 32, 8, 2), (64, 64, 4, 2), (64, 32, 8, 4), (128, 64, 4, 3), (96, 32, 8, 2)]


@pytest.mark.parametrize("e", [257, 8, 37])
@pytest.mark.parametrize("n", [256, 512])
@pytest.mark.parametrize("k", [7168, 4096])
def test_reference_input_distribution_and_literal_tolerance(e, n, k):
    """The reference's own sweep grid (test/test_moe_correctness.py:118-140: E in {257,8,37} x N in {256,512} x
    K in {7168,4096} x M in {8,32,128,256}, top_k = 9), its own generator (duplicates of an expert inside a token
    included, negative block scales) and its own pass criterion, against the faithful oracle.  Each case runs three
    knob tuples, rotating so that every kernel shape meets every (E, N, K)."""
    weights = None
    for i, m in enumerate((8, 32, 128, 256)):
        case = orc.make_reference_style_case(m, e, n, k, 9, seed=42 + m, weights=weights)
        weights = (case.w, case.w_scale, case.w2, case.w2_scale)
        dcase = to_device(case)
        refs = {}
        base = (i * 3 + e + n // 256 + k // 4096) % len(_GRID_KNOBS)
        for j in range(3):
            bm, bn, wn, st = _GRID_KNOBS[(base + j) % len(_GRID_KNOBS)]
            if m < bm and bm != 16:          # the reference skips these too (:189-190)
                bm, bn, wn, st = 16, bn, wn, st
            if bm not in refs:
                refs[bm] = orc.run_oracle(case, bm).float()
            got = run_capi(case, bm, bn, wn, st, dcase=dcase).float()
            tag = f"M={m} E={e} N={n} K={k} knobs={bm},{bn},{wn},{st}"
            assert torch.allclose(got, refs[bm], atol=2e-2, rtol=1e-1), tag
            assert orc.rel_l2(got, refs[bm]) <= 2e-2, tag


def test_schedule_is_followed_and_padding_rows_untouched():
    """Blocks past num_tokens_post_padded and sentinel slots contribute nothing; rows of `out`
    outside [0, M) are never written (canary rows around the output)."""
    case = orc.make_case(8, 512, 128, 12, 2, seed=5)
    sid, eid, npp = case.schedule(8)
    cut = torch.tensor([int(npp) - 8], dtype=torch.int32)
    ref = orc.fused_moe_w8a8_up_down_oracle(case.x, case.x_scale, case.w, case.w_scale, case.w2, case.w2_scale,
                                            sid, eid, cut, case.topk_weights, 2, 8, 1.0)
    big = torch.full((12 + 2, 512), 3.0, dtype=torch.bfloat16, device="cuda:0")
    big[1:13].zero_()
    got = run_capi(case, 8, 32, 8, 2, schedule=(sid, eid, cut), out=big[1:13])
    check_close(got, ref, tag="cut schedule")
    assert (big[0] == 3.0).all() and (big[13] == 3.0).all()


def test_accumulates_into_out_and_is_linear_in_scaling():
    case = orc.make_case(8, 512, 128, 16, 2, seed=0, scaling=1.0)
    base = run_capi(case, 16).float()
    case2 = orc.make_case(8, 512, 128, 16, 2, seed=0, scaling=2.0)
    assert orc.rel_l2(run_capi(case2, 16).float(), 2 * base) < 1e-2
    # a second call on the same buffer adds the result again (out is accumulated, not overwritten)
    out = torch.zeros(16, 512, dtype=torch.bfloat16, device="cuda:0")
    run_capi(case, 16, out=out)
    twice = run_capi(case, 16, out=out).float()
    assert orc.rel_l2(twice, 2 * base) < 1e-2


def test_torch_operator_path_and_errors():
    case = orc.make_case(8, 512, 128, 16, 2, seed=0)
    ref = orc.run_oracle(case, 16)
    check_close(run_torch_op(case, 16, 64, 4, 5), ref, tag="torch op")
    import alpha_moe_ops
    d = to_device(case)
    sid, eid, npp = [t.cuda() for t in case.schedule(16)]
    out = torch.zeros(16, 512, dtype=torch.bfloat16, device="cuda:0")
    ret = alpha_moe_ops.fused_moe_w8a8_up_down(d["x"], d["x_scale"], d["w"], d["w_scale"], d["w2"], d["w2_scale"],
                                               sid, eid, npp, d["topk_weights"], out, 2, 16, 32, 8, 3, 1.0)
    assert ret is out
    torch.cuda.synchronize()
    check_close(out.cpu(), ref, tag="alpha_moe_ops")
    for bad in (dict(block_n=64, warp_n=8), dict(stages=6), dict(block_m=20)):
        kn = dict(block_m=16, block_n=32, warp_n=8, stages=3)
        kn.update(bad)
        with pytest.raises(RuntimeError):
            torch.ops.alpha_moe.fused_moe_w8a8_up_down(
                d["x"], d["x_scale"], d["w"], d["w_scale"], d["w2"], d["w2_scale"], sid, eid, npp,
                d["topk_weights"], out, 2, kn["block_m"], kn["block_n"], kn["warp_n"], kn["stages"], 1.0)
    with pytest.raises(RuntimeError):   # wrong dtype of out
        torch.ops.alpha_moe.fused_moe_w8a8_up_down(
            d["x"], d["x_scale"], d["w"], d["w_scale"], d["w2"], d["w2_scale"], sid, eid, npp,
            d["topk_weights"], out.float(), 2, 16, 32, 8, 3, 1.0)


@pytest.fixture
def ksplit_override():
    from alpha_moe_b200 import capi
    yield capi.set_ksplit
    capi.set_ksplit(0)


@pytest.mark.parametrize("ks", [1, 2, 3, 4, 5, 6, 7, 8])
def test_k_split_over_a_cluster_small_batches(ks, ksplit_override):
    """Small batches: each (block, slice) is shared by a cluster of ks CTAs that split K and exchange partial
    sums through distributed shared memory.  alpha_moe_b200_set_ksplit overrides the automatic choice."""
    ksplit_override(ks)
    w = test_deepseek_shard_shape_small_expert_count.weights
    for m, top_k in ((1, 5), (3, 5), (7, 3)):
        case = orc.make_case(16, 7168, 256, m, top_k, seed=50 + m, shared=True, scaling=2.5, weights=w)
        dcase = to_device(case)
        for bm, st in ((16, 2), (8, 5), (32, 3)):
            if m < bm and bm != 16:
                continue
            check_close(run_capi(case, bm, 32, 8, st, dcase=dcase), orc.run_oracle(case, bm), tag=f"ks={ks} M={m} bm={bm}")
    # K with a chunk count that does not divide by ks, and an odd number of hidden tiles
    case = orc.make_case(8, 1152, 128, 2, 2, seed=9)
    check_close(run_capi(case, 16, 32, 8, 3), orc.run_oracle(case, 16), tag=f"ks={ks} K=1152")


def test_automatic_cluster_size_follows_the_devices_cluster_capacity():
    """The launcher asks the driver how many clusters of 2..8 CTAs the device holds at once and takes the largest
    size at which every (block, slice) unit gets its cluster in one round; plan(num_sms=0) reports that choice.  It
    must be monotone in the number of blocks, stay within the K chunks, and the operator must be right with it."""
    from alpha_moe_b200 import capi
    capi.set_ksplit(0)
    chosen = [capi.plan(7168, 16, 5, 32, N=512, num_blocks=nb, num_sms=0)[4] for nb in range(1, 80)]
    assert all(1 <= ks <= 8 for ks in chosen) and chosen == sorted(chosen, reverse=True)
    assert chosen[0] >= 4 and chosen[-1] == 1
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for nb, ks in enumerate(chosen, start=1):
        assert ks == 1 or 2 * nb * ks <= sms            # one CTA per SM: never more CTAs than SMs
    assert capi.plan(256, 16, 5, 32, N=512, num_blocks=1, num_sms=0)[4] == 2
    w = test_deepseek_shard_shape_small_expert_count.weights
    for m, top_k in ((1, 5), (2, 5), (3, 5), (5, 4)):
        case = orc.make_case(16, 7168, 256, m, top_k, seed=70 + m, shared=True, scaling=2.5, weights=w)
        check_close(run_capi(case, 16, 32, 8, 5), orc.run_oracle(case, 16), tag=f"auto ks M={m}")


def test_every_token_to_one_expert_many_blocks_of_the_same_weights():
    """Maximum imbalance: all assignments land on two experts, so one expert owns dozens of consecutive blocks
    (narrow, 64-wide and token-major shapes)."""
    case = orc.make_case(6, 1024, 256, 700, 2, seed=21, scaling=1.5)
    ids = torch.zeros_like(case.topk_ids)
    ids[:, 1] = 3
    case = dataclasses.replace(case, topk_ids=ids.contiguous())
    for bm, bn, wn, st in ((16, 32, 8, 3), (64, 64, 4, 2), (128, 64, 4, 3), (128, 32, 8, 2)):
        check_close(run_capi(case, bm, bn, wn, st), orc.run_oracle(case, bm), tag=f"one expert bm={bm} bn={bn}")


@pytest.mark.parametrize("e,k,inter,m,top_k,bm,bn,wn", [
    (4, 128, 128, 150, 2, 128, 64, 4),     # a single K chunk and a single slice in the token-major kernel
    (4, 128, 128, 150, 2, 64, 64, 4),      # same in the 64-wide shape (block_n = 64 falls back to one slice per CTA)
    (4, 256, 384, 260, 3, 128, 64, 4),     # three slices: odd slice count, so one slice per CTA despite block_n = 64
    (4, 2304, 256, 129, 2, 128, 64, 4),    # 18 K chunks, second block of every expert almost empty
    (3, 640, 128, 9, 3, 72, 32, 8),        # fewer tokens than the block size, every token to every expert
])
def test_edge_shapes_of_the_wide_kernels(e, k, inter, m, top_k, bm, bn, wn):
    case = orc.make_case(e, k, inter, m, top_k, seed=e * k + m, scaling=0.5)
    check_close(run_capi(case, bm, bn, wn, 3), orc.run_oracle(case, bm), tag=f"E{e} K{k} I{inter} M{m} bm={bm}")


def test_zero_and_negative_routing_weights_and_scales():
    """topk_weights of zero cancel an assignment, negative ones and negative weight scales (the reference's own
    generator produces them) flip signs; nothing in the kernel may assume positivity."""
    case = orc.make_case(8, 512, 256, 90, 3, seed=33, scaling=2.0)
    wts = case.topk_weights.clone()
    wts[::3, 0] = 0.0
    wts[1::3, 1] *= -1.0
    ws = case.w_scale.clone()
    ws[::2] *= -1.0
    w2s = case.w2_scale.clone()
    w2s[1::2] *= -1.0
    case = dataclasses.replace(case, topk_weights=wts.contiguous(), w_scale=ws.contiguous(), w2_scale=w2s.contiguous())
    for bm, bn, wn in ((16, 32, 8), (64, 64, 4), (128, 64, 4)):
        check_close(run_capi(case, bm, bn, wn, 2), orc.run_oracle(case, bm), tag=f"signs bm={bm}")


@pytest.mark.parametrize("m,bm,bn,wn,st", [(8, 16, 32, 8, 3), (300, 128, 64, 4, 3)])
def test_operator_replays_from_a_cuda_graph(m, bm, bn, wn, st):
    """Serving engines capture the decode step in a CUDA graph: after one eager call (which sets the kernel's
    shared-memory attribute and builds the tensor maps) the operator is captured together with the clearing of
    `out` and replayed; every replay must give the eager result (up to the order of the bf16 reductions)."""
    import alpha_moe  # noqa: F401
    case = orc.make_case(16, 1024, 256, m, 4, seed=70 + m, scaling=2.5)
    d = to_device(case)
    sid, eid, npp = [t.cuda() for t in case.schedule(bm)]
    out = torch.zeros(m, 1024, dtype=torch.bfloat16, device="cuda")

    def layer():
        out.zero_()
        torch.ops.alpha_moe.fused_moe_w8a8_up_down(d["x"], d["x_scale"], d["w"], d["w_scale"], d["w2"], d["w2_scale"],
                                                   sid, eid, npp, d["topk_weights"], out, case.top_k, bm, bn, wn, st, 2.5)
    layer()
    torch.cuda.synchronize()
    eager = out.clone()
    check_close(eager.cpu(), orc.run_oracle(case, bm), tag="eager")
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        layer()                      # warm-up on the capture stream
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            layer()
    for _ in range(3):
        out.fill_(7.0)               # the captured clear must take care of this
        g.replay()
        torch.cuda.synchronize()
        assert orc.rel_l2(out.cpu(), eager.cpu()) <= 1e-2


@pytest.mark.parametrize("balancedness", [0.8, 0.5])
def test_reference_timing_scripts_imbalance_model(balancedness):
    """Routing of the reference's timing script (test/test_moe_performance.py:42-49): every routed assignment drawn
    independently from balancedness x uniform + (1 - balancedness) x expert 0 - one hot expert that owns dozens of
    blocks, duplicates inside a token, experts that receive nothing - through every kernel shape."""
    import bench
    e, k, inter, m, top_k = 24, 1024, 256, 300, 6
    base = orc.make_case(e, k, inter, m, top_k, seed=31, shared=True, scaling=2.5)
    ids, wts = bench.route_mixture(m, e - 1, top_k - 1, balancedness, torch.Generator().manual_seed(5), e - 1)
    case = dataclasses.replace(base, topk_ids=ids, topk_weights=wts)
    assert float((ids[:, :-1] == 0).float().mean()) > (1 - balancedness) * 0.8        # expert 0 is hot
    for bm, bn, wn, st in ((8, 64, 4, 3), (16, 32, 8, 5), (32, 64, 4, 2), (64, 64, 4, 2), (64, 32, 8, 4), (128, 64, 4, 3)):
        check_close(run_capi(case, bm, bn, wn, st), orc.run_oracle(case, bm), tag=f"mixture {balancedness} bm={bm} bn={bn}")
