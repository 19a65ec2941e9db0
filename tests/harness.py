"""Shared helpers of the GPU parity tests: move a seeded oracle case to the device, call the
operator through the C ABI (ctypes) or through torch.ops, read the kernel status word."""
from __future__ import annotations

import torch

from oracle import moe_oracle as orc


def to_device(case: orc.MoeCase, dev="cuda:0"):
    d = {}
    for name in ("x", "x_scale", "w", "w_scale", "w2", "w2_scale", "topk_weights"):
        d[name] = getattr(case, name).to(dev).contiguous()
    return d


def run_capi(case: orc.MoeCase, block_m: int, block_n=32, warp_n=8, stages=4, dev="cuda:0",
             dcase=None, schedule=None, out=None):
    """One call through alpha_moe_b200_fused_moe_w8a8_up_down; returns the bf16 result on CPU."""
    from alpha_moe_b200 import capi
    d = dcase if dcase is not None else to_device(case, dev)
    sid, eid, npp = schedule if schedule is not None else case.schedule(block_m)
    sid_d, eid_d, npp_d = sid.to(dev), eid.to(dev), npp.to(dev)
    m, k = case.x.shape
    e, n, _ = case.w.shape
    if out is None:
        out = torch.zeros(m, k, dtype=torch.bfloat16, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        capi.fused_moe_w8a8_up_down(
            d["x"].data_ptr(), d["x_scale"].data_ptr(), d["w"].data_ptr(), d["w_scale"].data_ptr(),
            d["w2"].data_ptr(), d["w2_scale"].data_ptr(), out.data_ptr(), sid_d.data_ptr(),
            eid_d.data_ptr(), npp_d.data_ptr(), d["topk_weights"].data_ptr(), case.top_k, m, k, n, e,
            sid.numel(), block_m, block_n, warp_n, stages, float(case.scaling_factor), stream)
        status = capi.read_status(reset=True)
    assert status[0] == 0, f"kernel status {status}"
    return out.cpu()


def run_torch_op(case: orc.MoeCase, block_m: int, block_n=32, warp_n=8, stages=4, dev="cuda:0"):
    import alpha_moe  # noqa: F401  registers the operator
    d = to_device(case, dev)
    sid, eid, npp = case.schedule(block_m)
    m, k = case.x.shape
    out = torch.zeros(m, k, dtype=torch.bfloat16, device=dev)
    torch.ops.alpha_moe.fused_moe_w8a8_up_down(
        d["x"], d["x_scale"], d["w"], d["w_scale"], d["w2"], d["w2_scale"], sid.to(dev), eid.to(dev),
        npp.to(dev), d["topk_weights"], out, case.top_k, block_m, block_n, warp_n, stages,
        float(case.scaling_factor))
    torch.cuda.synchronize()
    return out.cpu()


def check_close(got: torch.Tensor, ref: torch.Tensor, rel=2e-2, tag=""):
    """Gate against the faithful oracle: rel-L2 <= rel and |d| <= 0.25*rms(ref) + 0.1*|ref|."""
    got, ref = got.float(), ref.float()
    assert torch.isfinite(got).all(), f"{tag}: non-finite output"
    r = orc.rel_l2(got, ref)
    rms = ref.pow(2).mean().sqrt()
    bound = 0.25 * rms + 0.1 * ref.abs()
    worst = float(((got - ref).abs() - bound).max())
    assert r <= rel, f"{tag}: rel-L2 {r:.4f} > {rel}"
    assert worst <= 0, f"{tag}: element outside 0.25*rms+0.1*|ref| by {worst:.4g}"
    return r
