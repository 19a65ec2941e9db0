"""CPU tests of the oracle: golden vectors generated from the reference's Python utilities,
the committed config-0 pin, and invariants of the restated pieces."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _digest(case):
    h = hashlib.sha256()
    for name in ("x", "x_scale", "w", "w_scale", "w2", "w2_scale", "topk_ids", "topk_weights"):
        t = getattr(case, name).contiguous()
        if t.dtype == torch.float8_e4m3fn:
            t = t.view(torch.uint8)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def test_interleave_matches_reference_goldens():
    g = np.load(os.path.join(GOLD, "ref_interleave.npz"))
    for src, rep, key in (("a", 8, "a_rep8"), ("a", 2, "a_rep2"), ("b", 8, "b_rep8"), ("s", 1, "s_rep1")):
        t = torch.from_numpy(g[src])
        want = torch.from_numpy(g[key])
        assert torch.equal(orc.interleave_rows(t, rep), want)
        assert torch.equal(orc.deinterleave_rows(want, rep), t)


def test_cfg0_inputs_and_oracle_match_committed_pin():
    g = np.load(os.path.join(GOLD, "cfg0_oracle.npz"))
    case = orc.make_case(8, 512, 128, 16, 2, seed=0)
    assert _digest(case) == str(g["inputs_sha256"])
    sid, eid, npp = case.schedule(16)
    assert np.array_equal(sid.numpy(), g["sorted_token_ids"])
    assert np.array_equal(eid.numpy(), g["expert_ids"])
    assert np.array_equal(npp.numpy(), g["num_tokens_post_padded"])
    out_b = orc.run_oracle(case, 16, faithful=True, out_fp32=True)
    out_a = orc.run_oracle(case, 16, faithful=False, out_fp32=True)
    assert torch.allclose(out_b, torch.from_numpy(g["out_faithful"]), rtol=1e-5, atol=1e-7)
    assert torch.allclose(out_a, torch.from_numpy(g["out_ideal"]), rtol=1e-5, atol=1e-7)
    # the two oracles bracket what a correct kernel may produce
    assert orc.rel_l2(out_b, out_a) < 4e-2


@pytest.mark.parametrize("block", [8, 16, 24, 64, 128])
@pytest.mark.parametrize("m,e,k", [(1, 8, 2), (16, 8, 2), (33, 37, 9), (300, 257, 9), (5, 512, 10)])
def test_moe_align_block_size_properties(m, e, k, block):
    gen = torch.Generator().manual_seed(m * 131 + e)
    ids = torch.stack([torch.randperm(e, generator=gen)[:k] for _ in range(m)]).to(torch.int32)
    sid, eid, npp = orc.moe_align_block_size(ids, block, e)
    numel = m * k
    assert sid.numel() == numel + e * (block - 1)
    n = int(npp)
    assert n % block == 0 and n <= sid.numel()
    live = sid[:n]
    assert (sid[n:] == numel).all()                      # tail is sentinel only
    real = live[live < numel]
    assert sorted(real.tolist()) == list(range(numel))   # every assignment exactly once
    flat = ids.reshape(-1)
    for b in range(n // block):
        blk = live[b * block:(b + 1) * block]
        vals = blk[blk < numel]
        assert vals.numel() > 0                          # no all-padding block inside the schedule
        assert (flat[vals.long()] == eid[b]).all()       # one expert per block
        pad = (blk >= numel).nonzero()
        if pad.numel():                                  # padding only at the end of a block
            assert int(pad.min()) == vals.numel()
    used = eid[: n // block]
    assert (used[1:] >= used[:-1]).all()                 # experts in ascending order


def test_quantisers_round_trip_and_saturate():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(7, 256, generator=gen).to(torch.bfloat16)
    q, s = orc.quant_token_groups(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (7, 2)
    deq = q.float().reshape(7, 2, 128) * s[:, :, None]
    err = (deq.reshape(7, 256) - x.float()).abs()
    assert float((err / (s.repeat_interleave(128, 1) * 448)).max()) <= 0.0625 + 1e-6   # half an e4m3 step at the top
    assert float(q.float().abs().max()) <= 448
    assert torch.isfinite(orc.to_fp8_sat(torch.tensor([1e9, -1e9, 465.0])).float()).all()
    z, zs = orc.quant_token_groups(torch.zeros(2, 128, dtype=torch.bfloat16))
    assert (z.float() == 0).all() and torch.allclose(zs, torch.full_like(zs, 1e-10 / 448))
    w = (torch.randn(2, 256, 128, generator=gen) * 0.02).to(torch.bfloat16)
    qw, sw = orc.quant_weight_blocks(w)
    assert sw.shape == (2, 2, 1)
    assert float(qw.float().abs().amax()) == 448.0


def test_oracle_follows_schedule_not_topk_ids():
    """Blocks beyond num_tokens_post_padded and sentinel slots contribute nothing (kernel :678, :758)."""
    case = orc.make_case(8, 256, 128, 12, 2, seed=5)
    sid, eid, npp = case.schedule(8)
    full = orc.fused_moe_w8a8_up_down_oracle(case.x, case.x_scale, case.w, case.w_scale, case.w2, case.w2_scale,
                                             sid, eid, npp, case.topk_weights, 2, 8, 1.0, out_fp32=True)
    cut = torch.tensor([int(npp) - 8], dtype=torch.int32)
    part = orc.fused_moe_w8a8_up_down_oracle(case.x, case.x_scale, case.w, case.w_scale, case.w2, case.w2_scale,
                                             sid, eid, cut, case.topk_weights, 2, 8, 1.0, out_fp32=True)
    dropped = sid[int(cut):int(npp)]
    rows = torch.unique(dropped[dropped < 24] // 2)
    other = torch.ones(12, dtype=torch.bool)
    other[rows.long()] = False
    assert torch.equal(full[other], part[other])
    assert not torch.equal(full[rows.long()], part[rows.long()])
    # block size does not change the result beyond summation order
    a = orc.run_oracle(case, 8, out_fp32=True)
    b = orc.run_oracle(case, 64, out_fp32=True)
    assert orc.rel_l2(a, b) < 1e-5


def test_reference_style_inputs_meet_the_reference_tolerance_between_oracles():
    """Under the reference's own input distribution its literal check allclose(atol=2e-2, rtol=1e-1)
    (test/test_moe_correctness.py:106-110) holds between the faithful and the ideal oracle."""
    case = orc.make_reference_style_case(8, 10, 512, 1024, 9)
    assert (case.topk_ids[:, -1] == 9).all()
    b = orc.run_oracle(case, 16).float()
    a = orc.run_oracle(case, 16, faithful=False).float()
    assert torch.allclose(b, a, atol=2e-2, rtol=1e-1)


def test_tp_split_of_the_oracle_is_exact():
    """Summing the oracle over I/tp shards reproduces the unsharded result (the property the
    tensor-parallel path relies on)."""
    from alpha_moe_b200.tp import shard_weights
    case = orc.make_case(4, 256, 256, 9, 2, seed=7)
    sid, eid, npp = case.schedule(16)
    full = orc.run_oracle(case, 16, out_fp32=True)
    acc = torch.zeros_like(full)
    for r in range(2):
        w, ws, w2, w2s = shard_weights(case.w, case.w_scale, case.w2, case.w2_scale, r, 2)
        acc += orc.fused_moe_w8a8_up_down_oracle(case.x, case.x_scale, w, ws, w2, w2s, sid, eid, npp,
                                                 case.topk_weights, 2, 16, 1.0, out_fp32=True)
    assert orc.rel_l2(acc, full) < 1e-5
