"""world_size-2 gloo test of the tensor-parallel plumbing on CPU: each rank runs the restated
operator on its shard of the intermediate dimension, the partial outputs are summed by the same
tp_layer() helper the GPU path uses, and the result equals the unsharded one."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_path):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from alpha_moe_b200.tp import shard_weights, tp_layer
    from oracle import moe_oracle as orc
    torch.set_num_threads(1)
    case = orc.make_case(4, 256, 256, 10, 2, seed=11, scaling=2.5)
    sid, eid, npp = case.schedule(16)
    w, ws, w2, w2s = shard_weights(case.w, case.w_scale, case.w2, case.w2_scale, rank, world)

    def compute(out):
        out += orc.fused_moe_w8a8_up_down_oracle(case.x, case.x_scale, w, ws, w2, w2s, sid, eid, npp,
                                                 case.topk_weights, 2, 16, 2.5, out_fp32=True)
    out = torch.full((10, 256), 7.0)          # tp_layer must zero it first
    tp_layer(compute, out)
    if rank == 0:
        full = orc.run_oracle(case, 16, out_fp32=True)
        torch.save({"rel": orc.rel_l2(out, full)}, result_path)
    dist.destroy_process_group()


def test_tp2_sum_equals_unsharded(tmp_path):
    port = _free_port()
    result = str(tmp_path / "r.pt")
    mp.spawn(_worker, args=(2, port, result), nprocs=2, join=True)
    assert torch.load(result)["rel"] < 1e-5


def test_shard_shapes_and_errors():
    import pytest
    from alpha_moe_b200.tp import shard_weights
    w = torch.zeros(3, 1024, 256, dtype=torch.uint8)
    ws = torch.zeros(3, 8, 2)
    w2 = torch.zeros(3, 256, 512, dtype=torch.uint8)
    w2s = torch.zeros(3, 2, 4)
    a, b, c, d = shard_weights(w, ws, w2, w2s, 1, 4)
    assert a.shape == (3, 256, 256) and b.shape == (3, 2, 2) and c.shape == (3, 256, 128) and d.shape == (3, 2, 1)
    assert c.is_contiguous()
    with pytest.raises(ValueError):
        shard_weights(w, ws, w2, w2s, 0, 8)
