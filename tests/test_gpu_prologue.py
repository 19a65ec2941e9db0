"""GPU tests of the two pre-operator kernels, bit-exact against the CPU restatement (integer and
byte work): block schedule and per-token-group fp8 quantisation, then the whole call-site sequence
of extra/sglang.patch:25-41 end to end."""
import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,e,k,block", [(1, 257, 9, 16), (4, 8, 2, 8), (16, 8, 2, 16), (64, 257, 9, 8),
                                         (113, 257, 9, 16), (114, 257, 9, 16), (300, 37, 9, 32),
                                         (1024, 512, 10, 64), (4096, 257, 9, 128), (8192, 257, 9, 72)])
def test_moe_align_block_size_matches_oracle_exactly(m, e, k, block):
    from alpha_moe_b200.prologue import moe_align_block_size
    g = torch.Generator().manual_seed(m + e)
    ids, _ = orc.route_topk(torch.randn(m, e, generator=g), k)
    want = orc.moe_align_block_size(ids, block, e)
    got = moe_align_block_size(ids.cuda(), block, e)
    torch.cuda.synchronize()
    for a, b, name in zip(got, want, ("sorted_token_ids", "expert_ids", "num_tokens_post_padded")):
        assert torch.equal(a.cpu(), b), name


def test_moe_align_more_chunks_than_fit_on_the_gpu_and_many_experts():
    """About a million assignments are more 1024-assignment chunks than can be resident at once, so the schedule is
    built by two launches instead of one cooperative launch; 1000 experts exercises several experts per thread in
    the offset computation.  Both bit-exact against the CPU restatement."""
    from alpha_moe_b200.prologue import moe_align_block_size
    g = torch.Generator().manual_seed(11)
    for m, e, k, block in ((130000, 257, 9, 128), (3000, 1000, 6, 16)):
        ids = torch.randint(0, e, (m, k), generator=g, dtype=torch.int32)
        want = orc.moe_align_block_size(ids, block, e)
        got = moe_align_block_size(ids.cuda(), block, e)
        torch.cuda.synchronize()
        for a, b, name in zip(got, want, ("sorted_token_ids", "expert_ids", "num_tokens_post_padded")):
            assert torch.equal(a.cpu(), b), f"{name} M={m} E={e}"


def test_moe_align_duplicates_skew_and_out_of_range_ids():
    from alpha_moe_b200.prologue import moe_align_block_size
    g = torch.Generator().manual_seed(0)
    # everything routed to two experts, duplicates inside a token (reference test generator draws with replacement)
    ids = torch.randint(0, 2, (700, 9), generator=g, dtype=torch.int32) * 5
    want = orc.moe_align_block_size(ids, 16, 8)
    got = moe_align_block_size(ids.cuda(), 16, 8)
    for a, b in zip(got, want):
        assert torch.equal(a.cpu(), b)
    # ids outside [0, E) are ignored (they never reach a block)
    bad = ids.clone()
    bad[::7, 0] = -1
    bad[3::11, 1] = 8
    sid, eid, npp = [t.cpu() for t in moe_align_block_size(bad.cuda(), 16, 8)]
    flat = bad.reshape(-1)
    live = sid[: int(npp)]
    real = live[live < flat.numel()]
    assert sorted(real.tolist()) == [i for i in range(flat.numel()) if 0 <= int(flat[i]) < 8]


@pytest.mark.parametrize("m,k", [(1, 128), (3, 512), (64, 7168), (1000, 2048), (8192, 7168)])
def test_group_quant_matches_oracle_bit_for_bit(m, k):
    from alpha_moe_b200.prologue import per_token_group_quant_fp8
    g = torch.Generator().manual_seed(m * 7 + k)
    x = (torch.randn(m, k, generator=g) * torch.rand(m, 1, generator=g) * 3).to(torch.bfloat16)
    x[0, :128] = 0                                     # an all-zero group: scale = 1e-10 / 448
    if m > 2:
        x[2, 5] = 300.0                                # an outlier
    want_q, want_s = orc.quant_token_groups(x)
    xd = x.cuda()
    q, s = per_token_group_quant_fp8(xd)
    torch.cuda.synchronize()
    assert torch.equal(s.cpu(), want_s)
    assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8))
    assert torch.equal(xd.cpu(), x)                    # source untouched
    q2, s2 = per_token_group_quant_fp8(xd, zero_input=True)
    torch.cuda.synchronize()
    assert torch.equal(q2.cpu().view(torch.uint8), want_q.view(torch.uint8)) and torch.equal(s2.cpu(), want_s)
    assert (xd == 0).all()


@pytest.mark.parametrize("m,e,k,hidden,block", [(1, 257, 9, 7168, 16), (7, 8, 2, 128, 8), (64, 512, 10, 2048, 16),
                                                (113, 257, 9, 7168, 32), (114, 257, 9, 7168, 16), (500, 37, 9, 1024, 64)])
def test_quant_and_align_in_one_call_matches_oracle_bit_for_bit(m, e, k, hidden, block):
    """Quantisation and schedule as one launch (M * top_k <= 1024: the first four cases) or as the two separate
    launches (the last two), against the CPU restatement of each; with and without clearing the source."""
    from alpha_moe_b200.prologue import quant_and_align
    g = torch.Generator().manual_seed(3 * m + e)
    x = (torch.randn(m, hidden, generator=g) * torch.rand(m, 1, generator=g) * 3).to(torch.bfloat16)
    x[0, :128] = 0
    ids, _ = orc.route_topk(torch.randn(m, e, generator=g), k)
    want_q, want_s = orc.quant_token_groups(x)
    want_sched = orc.moe_align_block_size(ids, block, e)
    for zero in (False, True):
        xd = x.cuda()
        q, s, sid, eid, npp = quant_and_align(xd, ids.cuda(), block, e, zero_input=zero)
        torch.cuda.synchronize()
        assert torch.equal(q.cpu().view(torch.uint8), want_q.view(torch.uint8)) and torch.equal(s.cpu(), want_s)
        for a, b, name in zip((sid, eid, npp), want_sched, ("sorted_token_ids", "expert_ids", "num_tokens_post_padded")):
            assert torch.equal(a.cpu(), b), name
        assert (xd == 0).all() if zero else torch.equal(xd.cpu(), x)


def test_call_site_sequence_end_to_end():
    """quantise -> zero the activations -> schedule -> fused operator accumulating into the activation
    buffer, exactly the sequence of the reference's call site (extra/sglang.patch:30-41)."""
    import alpha_moe  # noqa: F401
    from alpha_moe_b200.prologue import moe_align_block_size, sglang_per_token_group_quant_fp8
    e, k, inter, m, top_k = 16, 1024, 256, 50, 4
    g = torch.Generator().manual_seed(3)
    w, w_scale, w2, w2_scale = orc.make_weights(e, k, inter, g)
    hidden = torch.randn(m, k, generator=g).to(torch.bfloat16)
    ids, wts = orc.route_topk(torch.randn(m, e, generator=g), top_k)
    xq, xs = orc.quant_token_groups(hidden)
    sid, eid, npp = orc.moe_align_block_size(ids, 16, e)
    ref = orc.fused_moe_w8a8_up_down_oracle(xq, xs, w, w_scale, w2, w2_scale, sid, eid, npp, wts, top_k, 16, 2.5)

    hs = hidden.cuda()
    a, a_scale = sglang_per_token_group_quant_fp8(hs, 128, zero_input=True)
    s_ids, e_ids, n_pad = moe_align_block_size(ids.cuda(), 16, e)
    torch.ops.alpha_moe.fused_moe_w8a8_up_down(a, a_scale, w.cuda(), w_scale.cuda(), w2.cuda(), w2_scale.cuda(),
                                               s_ids, e_ids, n_pad, wts.cuda(), hs, top_k, 16, 32, 8, 3, 2.5)
    torch.cuda.synchronize()
    assert orc.rel_l2(hs.cpu(), ref) <= 2e-2


@pytest.mark.parametrize("m,conf", [(50, {"block_m": 16, "block_n": 32, "warp_n": 8, "stages": 3}),
                                     (300, {"block_m": 128, "block_n": 64, "warp_n": 4, "stages": 3})])
def test_fused_experts_single_call_matches_the_step_by_step_sequence(m, conf, tmp_path):
    """alpha_moe_b200.layer.fused_experts_impl (one C-ABI call for the body of the reference's patched
    fused_experts_impl, extra/sglang.patch:25-40) against the oracle, with the knobs given directly and
    through a table file + ALPHA_MOE_CONFIG-style look-up."""
    import json
    from alpha_moe_b200.layer import fused_experts_impl
    e, k, inter, top_k = 16, 1024, 256, 4
    g = torch.Generator().manual_seed(5 + m)
    w, w_scale, w2, w2_scale = orc.make_weights(e, k, inter, g)
    hidden = torch.randn(m, k, generator=g).to(torch.bfloat16)
    ids, wts = orc.route_topk(torch.randn(m, e, generator=g), top_k)
    xq, xs = orc.quant_token_groups(hidden)
    bm = conf["block_m"]
    sid, eid, npp = orc.moe_align_block_size(ids, bm, e)
    ref = orc.fused_moe_w8a8_up_down_oracle(xq, xs, w, w_scale, w2, w2_scale, sid, eid, npp, wts, top_k, bm, 2.5)
    dw = [t.cuda() for t in (w, w_scale, w2, w2_scale)]

    hs = hidden.cuda()
    out = fused_experts_impl(hs, *dw, wts.cuda(), ids.cuda(), routed_scaling_factor=2.5, config=conf)
    torch.cuda.synchronize()
    assert out.data_ptr() == hs.data_ptr()            # result in place, as at the reference's call site
    assert orc.rel_l2(hs.cpu(), ref) <= 2e-2

    table = tmp_path / "moe.json"
    table.write_text(json.dumps({str(m): conf}))
    hs2 = hidden.cuda()
    fused_experts_impl(hs2, *dw, wts.cuda(), ids.cuda(), routed_scaling_factor=2.5, config=str(table))
    torch.cuda.synchronize()
    assert torch.equal(hs2.cpu(), hs.cpu()) or orc.rel_l2(hs2.cpu(), hs.cpu()) <= 1e-2   # reduction order may differ


def test_back_to_back_layers_with_changing_inputs_eager_and_from_a_graph():
    """The operator is launched with programmatic stream serialisation (its CTAs may be scheduled while the
    quantise/schedule kernel in front of it is still running, and wait for that kernel's completion before reading
    anything).  Several layers in a row, each with its own activations and routing but through the same scratch
    memory, must each see their own schedule and activations - eagerly and replayed from one CUDA graph."""
    from alpha_moe_b200.layer import fused_experts_impl
    e, k, inter, top_k = 16, 1024, 256, 4
    g = torch.Generator().manual_seed(77)
    w, w_scale, w2, w2_scale = orc.make_weights(e, k, inter, g)
    dw = [t.cuda() for t in (w, w_scale, w2, w2_scale)]
    steps = []
    for m, bm, bn, wn in ((3, 16, 32, 8), (50, 16, 32, 8), (50, 32, 64, 4), (200, 128, 64, 4), (7, 8, 32, 8)):
        hidden = torch.randn(m, k, generator=g).to(torch.bfloat16)
        ids, wts = orc.route_topk(torch.randn(m, e, generator=g), top_k)
        xq, xs = orc.quant_token_groups(hidden)
        sid, eid, npp = orc.moe_align_block_size(ids, bm, e)
        ref = orc.fused_moe_w8a8_up_down_oracle(xq, xs, w, w_scale, w2, w2_scale, sid, eid, npp, wts, top_k, bm, 2.5)
        conf = {"block_m": bm, "block_n": bn, "warp_n": wn, "stages": 3}
        steps.append((hidden, ids.cuda(), wts.cuda(), conf, ref))

    def run_all(bufs):
        for (hidden, ids, wts, conf, _), hs in zip(steps, bufs):
            fused_experts_impl(hs, *dw, wts, ids, routed_scaling_factor=2.5, config=conf)

    bufs = [s[0].cuda() for s in steps]
    run_all(bufs)
    torch.cuda.synchronize()
    for (_, _, _, conf, ref), hs in zip(steps, bufs):
        assert orc.rel_l2(hs.cpu(), ref) <= 2e-2, conf

    static = [s[0].cuda() for s in steps]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run_all([b.clone() for b in static])              # warm-up on the capture stream
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all(static)
    for rep in range(2):
        for (hidden, _, _, _, _), hs in zip(steps, static):
            hs.copy_(hidden.cuda())
        graph.replay()
        torch.cuda.synchronize()
        for (_, _, _, conf, ref), hs in zip(steps, static):
            assert orc.rel_l2(hs.cpu(), ref) <= 2e-2, (rep, conf)
    from alpha_moe_b200 import capi
    assert capi.read_status(reset=True)[0] == 0
