"""Full-size checks at the Qwen3-Next-like TP2 shard shape (E=512, K=2048, I=256, top_k=10 of softmax-renormalised
N(0,1) logits, no shared expert, scaling 1.0): sampled tokens against the oracle with the knobs the shipped table
gives for each batch size (every kernel shape gets exercised at K/128 = 16 chunks), and invariance to block_m."""
import os

import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu
E, K, I, TOP_K = 512, 2048, 256, 10
TABLE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs",
                     "moe_b200_E512_I256_K2048.json")


@pytest.fixture(scope="module")
def weights():
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(11)

    def quant(shape):
        w = (torch.randn(shape, generator=g, device=dev) * 0.02).to(torch.bfloat16).float()
        e, r, c = shape
        v = w.view(e, r // 128, 128, c // 128, 128)
        s = v.abs().amax(dim=(2, 4)).clamp_min(1e-10) / 448.0
        q = (v / s[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(e, r, c)
        return q, s
    parts = [quant((64, 2 * I, K)) for _ in range(E // 64)]
    w13 = torch.cat([p[0] for p in parts]); s13 = torch.cat([p[1] for p in parts])
    parts = [quant((64, K, I)) for _ in range(E // 64)]
    w2 = torch.cat([p[0] for p in parts]); s2 = torch.cat([p[1] for p in parts])
    from alpha_moe_b200.utils import interleave_tensor
    w = interleave_tensor(w13.view(torch.uint8), 8).view(torch.float8_e4m3fn)
    return w, interleave_tensor(s13, 1), w2.contiguous(), s2.contiguous()


def _run(wd, x, xs, ids, wts, bm, bn, wn, stages):
    import alpha_moe  # noqa: F401
    from alpha_moe_b200 import capi
    from alpha_moe_b200.prologue import moe_align_block_size
    dev = wd[0].device
    sid, eid, npp = moe_align_block_size(ids.to(dev), bm, E)
    out = torch.zeros(x.shape[0], K, dtype=torch.bfloat16, device=dev)
    torch.ops.alpha_moe.fused_moe_w8a8_up_down(x.to(dev), xs.to(dev), wd[0], wd[1], wd[2], wd[3], sid, eid, npp,
                                               wts.to(dev), out, TOP_K, bm, bn, wn, stages, 1.0)
    torch.cuda.synchronize()
    assert capi.read_status(reset=True)[0] == 0
    return out.cpu()


def _inputs(m, seed):
    g = torch.Generator().manual_seed(seed)
    x, xs = orc.quant_token_groups(torch.randn(m, K, generator=g).to(torch.bfloat16))
    ids, wts = orc.route_topk(torch.randn(m, E, generator=g), TOP_K)
    return x, xs, ids, wts


@pytest.mark.parametrize("m", [1, 16, 256, 1024, 4096])
def test_sampled_tokens_match_the_oracle_with_the_table_knobs(weights, m):
    from alpha_moe_b200.utils import get_best_config
    conf = get_best_config(TABLE, m)
    x, xs, ids, wts = _inputs(m, 300 + m)
    got = _run(weights, x, xs, ids, wts, conf["block_m"], conf["block_n"], conf["warp_n"], conf["stages"])
    g = torch.Generator().manual_seed(m)
    sample = torch.randperm(m, generator=g)[: min(m, 6)]
    experts = torch.unique(ids[sample]).tolist()
    remap = {e: i for i, e in enumerate(experts)}
    sub_ids = torch.tensor([[remap[int(e)] for e in row] for row in ids[sample]], dtype=torch.int32)
    idx = torch.tensor(experts)
    wc = [t[idx.to(t.device)].cpu() for t in weights]
    ssid, seid, snpp = orc.moe_align_block_size(sub_ids, 16, len(experts))
    ref = orc.fused_moe_w8a8_up_down_oracle(x[sample], xs[sample], wc[0], wc[1], wc[2], wc[3], ssid, seid, snpp,
                                            wts[sample].contiguous(), TOP_K, 16, 1.0)
    r = orc.rel_l2(got[sample], ref)
    assert r <= 2e-2, f"M={m} knobs {conf}: rel-L2 {r}"


def test_result_does_not_depend_on_the_block_size(weights):
    x, xs, ids, wts = _inputs(700, 9)
    a = _run(weights, x, xs, ids, wts, 16, 32, 8, 3)
    b = _run(weights, x, xs, ids, wts, 64, 64, 4, 2)
    c = _run(weights, x, xs, ids, wts, 128, 64, 4, 3)
    assert orc.rel_l2(b, a) <= 1e-2 and orc.rel_l2(c, a) <= 1e-2
