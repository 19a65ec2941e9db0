"""CPU tests that hold the oracle against results this repository's authors did not compute: outputs of
vLLM's Triton block-fp8 fused-MoE pipeline (the upstream of the comparator in the reference's correctness
script, test/test_moe_correctness.py:77-110), its group quantiser and its moe_align_block_size, captured on a
B200 by tests/golden/make_vllm_goldens.py and committed as tests/golden/vllm_comparator.npz.

Tolerances: operator output rel-L2 <= 2e-2 and |d| <= 0.25*rms + 0.1*|ref| (the comparator accumulates with a
different summation order and rounds the weighted sum to bf16 before the routed scaling); under the reference's
own input distribution also its literal allclose(atol=2e-2, rtol=1e-1).  Quantiser and schedule: bit-exact."""
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc
from tests.golden.make_vllm_goldens import CASES, digest

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "vllm_comparator.npz"))


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_matches_vllm_fixture(name):
    case = CASES[name]()
    assert digest(case) == str(GOLD[f"{name}_sha256"]), "the seeded input generator has drifted from the fixture"
    truth = torch.from_numpy(GOLD[f"{name}_out_bf16"]).view(torch.bfloat16).float()
    for bm in (16, 64):
        ref = orc.run_oracle(case, bm).float()
        r = orc.rel_l2(ref, truth)
        assert r <= 2e-2, f"{name}: rel-L2 {r}"
        bound = 0.25 * truth.pow(2).mean().sqrt() + 0.1 * truth.abs()
        assert float(((ref - truth).abs() - bound).max()) <= 0
        if name == "refdist":
            assert torch.allclose(ref, truth, atol=2e-2, rtol=1e-1)
    # the ideal (unrounded) oracle brackets it from the other side
    assert orc.rel_l2(orc.run_oracle(case, 16, faithful=False, out_fp32=True), truth) <= 4e-2


@pytest.mark.parametrize("name", sorted(CASES))
def test_group_quantiser_matches_vllm_fixture_bit_for_bit(name):
    case = CASES[name]()
    q, s = orc.quant_token_groups(case.x_bf16)
    assert np.array_equal(s.numpy(), GOLD[f"{name}_xs"])
    assert np.array_equal(q.view(torch.uint8).numpy(), GOLD[f"{name}_xq"])


@pytest.mark.parametrize("name", sorted(CASES))
def test_block_schedule_matches_vllm_fixture(name):
    case = CASES[name]()
    sid, eid, npp = orc.moe_align_block_size(case.topk_ids, 16, case.num_experts)
    n = int(npp)
    assert n == int(GOLD[f"{name}_npp"].reshape(-1)[0])
    nb = n // 16
    assert np.array_equal(eid[:nb].numpy(), GOLD[f"{name}_eid"][:nb])
    sid_v = torch.from_numpy(GOLD[f"{name}_sid"])
    # ids of one expert's segment as a set (the comparator promises no order inside a segment)
    for ex in torch.unique(eid[:nb]).tolist():
        sel = eid[:nb] == ex
        a = sid[:n].reshape(nb, 16)[sel].reshape(-1).sort().values
        b = sid_v[:n].reshape(nb, 16)[sel].reshape(-1).sort().values
        assert torch.equal(a, b)
