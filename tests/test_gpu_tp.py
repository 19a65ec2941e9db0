"""Tensor-parallel run on real GPUs: two ranks (one process per GPU, NCCL) each run the fused operator on
their I/2 shard and all-reduce the partial bf16 outputs; rank 0 compares with the unsharded single-GPU
result (rel-L2 <= 1e-2).  Skipped with fewer than two GPUs."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import alpha_moe  # noqa: F401
    from alpha_moe_b200.tp import shard_weights, tp_layer
    from oracle import moe_oracle as orc
    case = orc.make_case(16, 1024, 512, 70, 5, seed=31, shared=True, scaling=2.5)
    sid, eid, npp = case.schedule(16)
    full = [t.to(dev) for t in (case.w, case.w_scale, case.w2, case.w2_scale)]
    shard = shard_weights(*full, rank, world)
    x, xs, wts = case.x.to(dev), case.x_scale.to(dev), case.topk_weights.to(dev)
    sid, eid, npp = sid.to(dev), eid.to(dev), npp.to(dev)

    def run(weights):
        def compute(out):
            torch.ops.alpha_moe.fused_moe_w8a8_up_down(x, xs, *weights, sid, eid, npp, wts, out, case.top_k,
                                                       16, 64, 4, 3, 2.5)
        return compute
    out = torch.full((70, 1024), 5.0, dtype=torch.bfloat16, device=dev)
    tp_layer(run(shard), out)
    torch.cuda.synchronize()
    if rank == 0:
        ref = torch.zeros(70, 1024, dtype=torch.bfloat16, device=dev)
        run(full)(ref)
        torch.cuda.synchronize()
        torch.save({"rel": orc.rel_l2(out.cpu(), ref.cpu()),
                    "rel_oracle": orc.rel_l2(out.cpu(), orc.run_oracle(case, 16))}, result_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_nccl_allreduce_equals_single_gpu(tmp_path):
    import torch.multiprocessing as mp
    result = str(tmp_path / "r.pt")
    mp.spawn(_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    r = torch.load(result)
    assert r["rel"] <= 1e-2 and r["rel_oracle"] <= 2e-2


def _worker_fused(rank, world, port, result_path, mode):
    """Fused exchange: every rank's kernel adds into all ranks' peer-mapped outputs, then this library's barrier."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import alpha_moe  # noqa: F401
    from alpha_moe_b200 import capi
    from alpha_moe_b200.tp import PeerReducedLayer, shard_weights
    from oracle import moe_oracle as orc
    layer = PeerReducedLayer(64, 1024, mode=mode)
    g = torch.Generator().manual_seed(77)
    weights = orc.make_weights(16, 1024, 512, g)
    full = [t.to(dev) for t in weights]
    shard = shard_weights(*full, rank, world)
    results = {}
    # consecutive steps of different sizes: the two buffers alternate, stale rows of a larger earlier batch must be gone
    for step, (m, bm, bn, wn, st) in enumerate(((40, 16, 64, 4, 3), (1, 16, 32, 8, 5), (64, 64, 64, 4, 2), (7, 8, 32, 8, 2))):
        case = orc.make_case(16, 1024, 512, m, 5, seed=100 + m, shared=True, scaling=2.5, weights=weights)
        sid, eid, npp = [t.to(dev) for t in case.schedule(bm)]
        x, xs, wts = case.x.to(dev), case.x_scale.to(dev), case.topk_weights.to(dev)
        out = layer.run(x, xs, *shard, sid, eid, npp, wts, case.top_k, bm, bn, wn, st, 2.5)
        torch.cuda.synchronize()
        assert capi.read_status(reset=True)[0] == 0
        got = out.cpu().clone()
        if rank == 0:
            ref = torch.zeros(m, 1024, dtype=torch.bfloat16, device=dev)
            torch.ops.alpha_moe.fused_moe_w8a8_up_down(x, xs, *full, sid, eid, npp, wts, ref, case.top_k, bm, bn, wn, st, 2.5)
            torch.cuda.synchronize()
            results[step] = {"rel": orc.rel_l2(got, ref.cpu()), "got": got, "case": case, "bm": bm}
        # every rank must hold the same sums (up to the order of the bf16 additions)
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out.contiguous())
        for other in gathered:
            assert orc.rel_l2(other.cpu(), got) <= 1e-2
    if rank == 0:
        for v in results.values():      # the CPU oracle only after the last step (bounded cross-GPU waits)
            v["rel_oracle"] = orc.rel_l2(v.pop("got"), orc.run_oracle(v.pop("case"), v.pop("bm")))
        torch.save(results, result_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["exchange", "epilogue"])
def test_tp2_exchange_without_a_collective_equals_single_gpu(tmp_path, mode):
    """The exchange step done by this library's own kernels over peer-mapped memory, no collective call: either one
    barrier + sum + clear kernel after the operator ("exchange"), or reductions into every rank's `out` from the
    operator's epilogue plus a barrier kernel ("epilogue").  Against the unsharded single-GPU result and the oracle,
    over four consecutive steps of different batch sizes (the two buffers alternate)."""
    import torch.multiprocessing as mp
    result = str(tmp_path / "rf.pt")
    mp.spawn(_worker_fused, args=(2, _free_port(), result, mode), nprocs=2, join=True)
    r = torch.load(result)
    assert len(r) == 4
    for step, v in r.items():
        assert v["rel"] <= 1e-2 and v["rel_oracle"] <= 2e-2, (step, v)


def _worker_allreduce(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import alpha_moe  # noqa: F401
    from alpha_moe_b200 import capi
    from alpha_moe_b200.tp import PeerAllReduce, shard_weights
    from oracle import moe_oracle as orc
    ar = PeerAllReduce(300, 1024)
    g = torch.Generator().manual_seed(78)
    weights = orc.make_weights(16, 1024, 512, g)
    full = [t.to(dev) for t in weights]
    shard = shard_weights(*full, rank, world)
    results = {}
    for step, (m, bm, bn, wn, st) in enumerate(((300, 128, 64, 4, 3), (33, 16, 32, 8, 3), (257, 64, 64, 4, 2))):
        case = orc.make_case(16, 1024, 512, m, 5, seed=200 + m, shared=True, scaling=2.5, weights=weights)
        sid, eid, npp = [t.to(dev) for t in case.schedule(bm)]
        x, xs, wts = case.x.to(dev), case.x_scale.to(dev), case.topk_weights.to(dev)
        out = ar.next_buffer(m)
        torch.ops.alpha_moe.fused_moe_w8a8_up_down(x, xs, *shard, sid, eid, npp, wts, out, case.top_k, bm, bn, wn, st, 2.5)
        part = out.float().clone()
        ar.all_reduce()
        torch.cuda.synchronize()
        assert capi.read_status(reset=True)[0] == 0
        dist.all_reduce(part)                       # fp32 sum of the partial outputs
        got = out.cpu().clone()
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out.contiguous())
        for other in gathered:
            assert torch.equal(other.cpu(), got)    # summed in rank order: every rank holds the same bits
        if rank == 0:
            results[step] = {"rel_sum": orc.rel_l2(got, part.cpu()), "got": got, "case": case, "bm": bm}
        dist.barrier()      # the cross-GPU waits are bounded (1 s): no rank may run ahead while another does host work
    # the reduce-scatter form: every rank ends up with the summed rows of its own share only
    for step, (m, bm, bn, wn, st) in enumerate(((300, 128, 64, 4, 3), (34, 16, 32, 8, 3))):
        case = orc.make_case(16, 1024, 512, m, 5, seed=300 + m, shared=True, scaling=2.5, weights=weights)
        sid, eid, npp = [t.to(dev) for t in case.schedule(bm)]
        x, xs, wts = case.x.to(dev), case.x_scale.to(dev), case.topk_weights.to(dev)
        out = ar.next_buffer(m)
        torch.ops.alpha_moe.fused_moe_w8a8_up_down(x, xs, *shard, sid, eid, npp, wts, out, case.top_k, bm, bn, wn, st, 2.5)
        part = out.float().clone()
        mine = ar.reduce_scatter()
        torch.cuda.synchronize()
        assert capi.read_status(reset=True)[0] == 0
        assert mine.shape == (m // world, 1024)
        dist.all_reduce(part)
        per = m // world
        rel_sum = orc.rel_l2(mine.cpu(), part[rank * per:(rank + 1) * per].cpu())
        rows = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(rows, mine.contiguous())
        worst = torch.tensor([rel_sum], device=dev)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        if rank == 0:
            results[f"rs{step}"] = {"rel_sum": float(worst), "got": torch.cat(rows).cpu(), "case": case, "bm": bm}
        dist.barrier()
    if rank == 0:
        # the CPU oracle takes seconds: only after the last step, when no rank is waiting in a kernel
        for v in results.values():
            v["rel_oracle"] = orc.rel_l2(v.pop("got"), orc.run_oracle(v.pop("case"), v.pop("bm")))
        torch.save(results, result_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_own_all_reduce_over_peer_mapped_buffers(tmp_path):
    """alpha_moe_b200_tp_allreduce (slice sums + slice fetches over NVLink, two flag barriers) after the operator:
    against the fp32 sum of the ranks' partial outputs (only the bf16 rounding of the sum may differ) and the oracle;
    every rank must hold identical bits.  Three steps of different sizes over the two alternating buffers, then two
    steps with alpha_moe_b200_tp_reduce_scatter, whose row shards put together must give the same layer output."""
    import torch.multiprocessing as mp
    result = str(tmp_path / "ra.pt")
    mp.spawn(_worker_allreduce, args=(2, _free_port(), result), nprocs=2, join=True)
    r = torch.load(result)
    assert len(r) == 5 and "rs0" in r and "rs1" in r      # three all-reduce steps, two reduce-scatter steps
    for step, v in r.items():
        assert v["rel_sum"] <= 5e-3 and v["rel_oracle"] <= 2e-2, (step, v)
