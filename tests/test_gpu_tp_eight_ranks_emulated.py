"""Eight tensor-parallel ranks on ONE GPU, one after the other.

Kernels that wait for one another must never run as separate launches on one GPU, so nothing here waits: every
"rank" owns its buffers and flag array in the same GPU's memory, and the arrivals of the other seven ranks are written
into each flag array beforehand.  Each rank's launch then finds everybody else "already there", does its share of the
work and returns.  This covers what an eight-GPU run adds over the two-GPU tests - eight buffer pointers, eight-way slices,
loops up to the maximum world size - for the parts that do not read another rank's *result*:

* the operator's tensor-parallel form (every partial result added into all eight `out` buffers),
* alpha_moe_b200_tp_exchange_sum (every rank sums all eight partial buffers into its own result buffer),
* alpha_moe_b200_tp_reduce_scatter (every rank sums its own eighth of the rows in place).

(The second phase of the all-reduce copies finished slices from their owners and is covered by the multi-GPU tests.)
"""
import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

WORLD = 8


def _flags(preset: int):
    """One flag array per rank: words 0..7 = the epoch every OTHER rank has 'already announced' (a rank's own word
    starts at zero and is written by its own launch, as in a real run), word 8 = own epoch (0), word 9 = ticket."""
    flags = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(WORLD)]
    for rank, f in enumerate(flags):
        f[:WORLD] = preset
        f[rank] = 0
    return flags


def test_operator_adds_into_all_eight_out_buffers():
    from alpha_moe_b200 import capi
    from alpha_moe_b200.tp import shard_weights
    e, k, inter, m, top_k = 8, 1024, 1024, 24, 3
    g = torch.Generator().manual_seed(808)
    weights = orc.make_weights(e, k, inter, g)
    case = orc.make_case(e, k, inter, m, top_k, seed=809, scaling=1.5, weights=weights)
    full = [t.cuda() for t in weights]
    for bm, bn, wn, st in ((16, 32, 8, 3), (64, 32, 8, 2)):
        sid, eid, npp = [t.cuda() for t in case.schedule(bm)]
        x, xs, wts = case.x.cuda(), case.x_scale.cuda(), case.topk_weights.cuda()
        outs = [torch.zeros(m, k, dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
        ptrs = [o.data_ptr() for o in outs]
        keep = []
        for rank in range(WORLD):
            w, w_scale, w2, w2_scale = shard_weights(*full, rank, WORLD)
            keep.append((w, w_scale, w2, w2_scale))
            capi.fused_moe_w8a8_up_down_tp(x.data_ptr(), xs.data_ptr(), w.data_ptr(), w_scale.data_ptr(), w2.data_ptr(),
                                           w2_scale.data_ptr(), ptrs, rank, sid.data_ptr(), eid.data_ptr(), npp.data_ptr(),
                                           wts.data_ptr(), top_k, m, k, w.shape[1], e, sid.numel(), bm, bn, wn, st, 1.5,
                                           torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert capi.read_status(reset=True)[0] == 0
        ref = orc.run_oracle(case, bm)
        for rank, o in enumerate(outs):
            assert orc.rel_l2(o.cpu(), ref) <= 2e-2, (bm, rank)


@pytest.mark.parametrize("n", [8 * 7, 7168, 64 * 7168 + 8])
def test_exchange_sum_with_eight_ranks(n):
    from alpha_moe_b200 import capi
    g = torch.Generator().manual_seed(n)
    parts = [(torch.randn(n, generator=g) * 3).to(torch.bfloat16).cuda() for _ in range(WORLD)]
    want = parts[0].float()
    for p in parts[1:]:
        want = want + p.float()                       # fp32, rank order: what every rank must compute
    want = want.to(torch.bfloat16)
    flags = _flags(1)
    fp = [f.data_ptr() for f in flags]
    results = [torch.full((n,), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
    nxt = [torch.ones(n, dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
    for rank in range(WORLD):
        capi.tp_exchange_sum([p.data_ptr() for p in parts], results[rank].data_ptr(), nxt[rank].data_ptr(), n, n, fp, rank, 50,
                             torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert capi.read_status(reset=True)[0] == 0
    for rank in range(WORLD):
        assert torch.equal(results[rank], want), rank          # identical bits on every rank
        assert (nxt[rank] == 0).all()                          # the next step's partial buffer was cleared
        assert int(flags[rank][WORLD]) == 1                    # own epoch advanced on the device
        assert int(flags[rank][WORLD + 1]) == 0                # ticket counter back at zero (replayable)


@pytest.mark.parametrize("rows,hidden", [(8, 56), (64, 7168), (40, 1024), (5, 24)])
def test_reduce_scatter_with_eight_ranks(rows, hidden):
    """rows * hidden / 8 vectors in eight slices of ceil(vectors / 8): whole rows when rows is a multiple of eight,
    ragged (the last rank's slice shorter, or empty) otherwise."""
    from alpha_moe_b200 import capi
    n = rows * hidden
    g = torch.Generator().manual_seed(n + 1)
    parts = [(torch.randn(n, generator=g) * 3).to(torch.bfloat16).cuda() for _ in range(WORLD)]
    orig = [p.clone() for p in parts]
    want = orig[0].float()
    for p in orig[1:]:
        want = want + p.float()
    want = want.to(torch.bfloat16)
    flags = _flags(2)
    fp = [f.data_ptr() for f in flags]
    for rank in range(WORLD):
        capi.tp_reduce_scatter([p.data_ptr() for p in parts], n, fp, rank, 50, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert capi.read_status(reset=True)[0] == 0
    per = 8 * (-(-(n // 8) // WORLD))
    for rank in range(WORLD):
        lo, hi = min(n, rank * per), min(n, (rank + 1) * per)
        assert torch.equal(parts[rank][lo:hi], want[lo:hi]), rank                     # my slice: the sum
        assert torch.equal(parts[rank][:lo], orig[rank][:lo]) and torch.equal(parts[rank][hi:], orig[rank][hi:])
        assert int(flags[rank][WORLD]) == 2 and int(flags[rank][WORLD + 1]) == 0
