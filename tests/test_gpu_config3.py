"""The unsharded DeepSeek-V3-like layer and its tensor-parallel shards on one GPU: E=257, K=7168 and
I = 2048 (tp=1: 16 intermediate slices per block, 11.3 GB of fp8 weights behind one pair of tensor maps),
1024 (tp=2) and 512 (tp=4).  The serving engine hands the operator an N = 2*I/tp shard (reference
README.md:1, csrc/torch_interface.cpp:91-95) and sums the partial outputs afterwards; here the shards run
back to back on one device.  Checked: sampled tokens against the oracle for every shard size (rel-L2 <= 2e-2),
and the sum of the shards' bf16 outputs against the unsharded result (rel-L2 <= 1e-2)."""
import pytest
import torch

from oracle import moe_oracle as orc
from tests.test_gpu_fullsize import E, K, TOP_K, _inputs, _run, _weights

pytestmark = pytest.mark.gpu
I_FULL = 2048


@pytest.fixture(scope="module")
def layer():
    return _weights(torch.device("cuda:0"), inter=I_FULL, seed=11)


def _oracle_on_sample(weights, x, xs, ids, wts, sample):
    experts = torch.unique(ids[sample]).tolist()
    remap = {e: i for i, e in enumerate(experts)}
    sub_ids = torch.tensor([[remap[int(e)] for e in row] for row in ids[sample]], dtype=torch.int32)
    idx = torch.tensor(experts)
    wc = [t[idx.to(t.device)].cpu() for t in weights]
    ssid, seid, snpp = orc.moe_align_block_size(sub_ids, 16, len(experts))
    return orc.fused_moe_w8a8_up_down_oracle(x[sample], xs[sample], wc[0], wc[1], wc[2], wc[3], ssid, seid, snpp,
                                             wts[sample].contiguous(), TOP_K, 16, 2.5)


@pytest.mark.parametrize("m,bm,bn", [(1, 16, 32), (64, 16, 64), (1024, 64, 64), (8192, 128, 64)])
def test_unsharded_layer_sampled_tokens_match_the_oracle(layer, m, bm, bn):
    x, xs, ids, wts = _inputs(m, "cuda:0", 300 + m)
    got = _run(layer, x, xs, ids, wts, bm, 2.5, bn=bn)
    assert torch.isfinite(got.float()).all()
    g = torch.Generator().manual_seed(m)
    sample = torch.randperm(m, generator=g)[: min(m, 2)]
    ref = _oracle_on_sample(layer, x, xs, ids, wts, sample)
    r = orc.rel_l2(got[sample], ref)
    assert r <= 2e-2, f"I={I_FULL} M={m}: rel-L2 {r}"


@pytest.mark.parametrize("tp", [2, 4])
@pytest.mark.parametrize("m,bm,bn", [(64, 16, 64), (1024, 128, 64)])
def test_tp_shards_sum_to_the_unsharded_layer_and_match_the_oracle(layer, tp, m, bm, bn):
    from alpha_moe_b200.tp import shard_weights
    x, xs, ids, wts = _inputs(m, "cuda:0", 500 + m)
    full = _run(layer, x, xs, ids, wts, bm, 2.5, bn=bn).float()
    g = torch.Generator().manual_seed(m + tp)
    sample = torch.randperm(m, generator=g)[:2]
    acc = torch.zeros_like(full)
    for r in range(tp):
        shard = shard_weights(*layer, r, tp)
        part = _run(shard, x, xs, ids, wts, bm, 2.5, bn=bn)
        acc += part.float()
        if r == tp - 1:      # one shard of each size also directly against the oracle
            ref = _oracle_on_sample(shard, x, xs, ids, wts, sample)
            rr = orc.rel_l2(part[sample], ref)
            assert rr <= 2e-2, f"I={I_FULL // tp} M={m}: rel-L2 {rr}"
        del shard
    rel = orc.rel_l2(acc, full)
    assert rel <= 1e-2, f"tp={tp} M={m}: sum of shards vs unsharded {rel}"
