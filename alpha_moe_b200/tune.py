"""Knob search for the fused MoE operator on the GPU at hand; writes a table in the reference's
format ({"<M>": {"block_m", "block_n", "warp_n", "stages"}}) that `get_best_config` /
`ALPHA_MOE_CONFIG` consume.

Counterpart of the reference's jit_moe.py:104-184 (brute force over the knob space per token count,
arg-min per M).  Differences: timing uses CUDA events with the L2 flushed between calls by default
(`--timing kineto` takes the reference's method instead: mean device time of the kernels whose name contains
"moe" in a torch.profiler trace, jit_moe.py:15-32); the schedule and the activation quantisation come from this
library's own kernels instead of SGLang's; by default only knob values that map to distinct kernel
configurations are tried (`--full` sweeps all 160 combinations like the reference).

    python -m alpha_moe_b200.tune --E 256 --N 512 --K 7168 --top-k 8            # DeepSeek-V3 TP8 shard
    python -m alpha_moe_b200.tune --E 512 --N 512 --K 2048 --top-k 10 --no-shared-expert
"""
from __future__ import annotations

import argparse
import json
import os

import torch

DEFAULT_MS = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192]


def knob_space(full: bool):
    if full:
        return [(bm, bn, wn, st) for bm in range(8, 129, 8) for bn, wn in ((64, 4), (32, 8)) for st in range(1, 6)]
    # block_m pads to 16 / 32 / 64 (weight-major kernel) or runs the token-major kernel (> 64);
    # 96 is kept because a three-quarters-full token-major block wastes less than a half-empty 128 one.
    return [(bm, bn, wn, st) for bm in (8, 16, 32, 64, 96, 128) for bn, wn in ((64, 4), (32, 8)) for st in (2, 3, 4, 5)]


def rand_fp8(shape, gen, dev):
    b = torch.randint(0, 0x78, shape, generator=gen, device=dev, dtype=torch.uint8)
    s = torch.randint(0, 2, shape, generator=gen, device=dev, dtype=torch.uint8) * 128
    return (b | s).view(torch.float8_e4m3fn)


def time_call(fn, flush, iters: int, warmup: int = 2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e3   # median, microseconds


def time_call_kineto(fn, flush, iters: int, kernel_name: str = "moe") -> float:
    """The reference's timing method (jit_moe.py:15-32): one warm-up cycle and one recorded cycle of `iters` calls
    under torch.profiler (CUDA activity), the L2 evicted before every call, mean device time of the kernels whose
    name contains `kernel_name`; microseconds."""
    from torch.profiler import ProfilerActivity, profile, schedule
    with profile(activities=[ProfilerActivity.CUDA], schedule=schedule(wait=0, warmup=1, active=1, repeat=1)) as prof:
        for _ in range(2):
            for _ in range(iters):
                flush.zero_()
                fn()
                torch.cuda.synchronize()
            prof.step()
    times = [e.device_time_total for e in prof.profiler.function_events if kernel_name in e.name]
    if not times:
        raise RuntimeError(f"no kernel with '{kernel_name}' in its name in the profile")
    return sum(times) / len(times)


def parse_knobs(items):
    """'16,32,8,3' -> (16, 32, 8, 3) for every item."""
    out = []
    for it in items:
        parts = tuple(int(v) for v in it.split(","))
        if len(parts) != 4:
            raise ValueError(f"a knob tuple is block_m,block_n,warp_n,stages - got '{it}'")
        out.append(parts)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description="B200 knob search for alpha_moe::fused_moe_w8a8_up_down")
    ap.add_argument("--E", type=int, default=256, help="routed experts (the shared expert is added on top)")
    ap.add_argument("--N", type=int, default=512, help="rows of w per expert = 2 x intermediate size of the shard")
    ap.add_argument("--K", type=int, default=7168, help="hidden size")
    ap.add_argument("--top-k", type=int, default=8, help="routed experts per token")
    ap.add_argument("--shared-expert", default=True, action=argparse.BooleanOptionalAction)
    ap.add_argument("--batch-sizes", type=int, nargs="+", default=DEFAULT_MS)
    ap.add_argument("--routings", type=int, default=2, help="random routings averaged per token count")
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--full", action="store_true", help="sweep all 160 knob combinations")
    ap.add_argument("--knobs", nargs="+", default=None, metavar="BM,BN,WN,ST", help="search these tuples only")
    ap.add_argument("--timing", choices=["events", "kineto"], default="events",
                    help="CUDA events (default) or the reference's torch.profiler method")
    ap.add_argument("--scaling-factor", type=float, default=2.5)
    ap.add_argument("--out-file", default=None)
    args = ap.parse_args(argv)

    import alpha_moe  # noqa: F401
    from .prologue import moe_align_block_size
    op = torch.ops.alpha_moe.fused_moe_w8a8_up_down

    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(42)
    e_total = args.E + int(args.shared_expert)
    top_k = args.top_k + int(args.shared_expert)
    n, k = args.N, args.K
    w = rand_fp8((e_total, n, k), gen, dev)
    w2 = rand_fp8((e_total, k, n // 2), gen, dev)
    w_scale = torch.rand(e_total, n // 128, k // 128, generator=gen, device=dev) * 1e-3 + 1e-4
    w2_scale = torch.rand(e_total, k // 128, n // 256, generator=gen, device=dev) * 1e-3 + 1e-4
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    table, report = {}, {}
    for m in args.batch_sizes:
        x = rand_fp8((m, k), gen, dev)
        x_scale = torch.rand(m, k // 128, generator=gen, device=dev) * 0.02 + 0.01
        out = torch.zeros(m, k, dtype=torch.bfloat16, device=dev)
        routings = []
        for _ in range(args.routings):
            logits = torch.randn(m, args.E, generator=gen, device=dev)
            vals, ids = torch.topk(logits, args.top_k, dim=-1)
            wts = torch.softmax(vals, -1)
            ids = ids.to(torch.int32)
            if args.shared_expert:
                ids = torch.cat([ids, torch.full((m, 1), args.E, dtype=torch.int32, device=dev)], 1)
                wts = torch.cat([wts, torch.ones(m, 1, device=dev)], 1)
            routings.append((ids.contiguous(), wts.float().contiguous()))
        best, best_us = None, float("inf")
        for bm, bn, wn, st in (parse_knobs(args.knobs) if args.knobs else knob_space(args.full)):
            if m < bm and bm != 16:          # same pruning as the reference sweep (jit_moe.py:153-154)
                continue
            total = 0.0
            for ids, wts in routings:
                sid, eid, npp = moe_align_block_size(ids, bm, e_total)

                def call():
                    op(x, x_scale, w, w_scale, w2, w2_scale, sid, eid, npp, wts, out, top_k, bm, bn, wn, st,
                       args.scaling_factor)
                total += (time_call_kineto if args.timing == "kineto" else time_call)(call, flush, args.iters)
            us = total / len(routings)
            if us < best_us:
                best, best_us = (bm, bn, wn, st), us
        if best is None:
            raise RuntimeError(f"no knob tuple is admissible for M={m}")
        table[str(m)] = {"block_m": best[0], "block_n": best[1], "warp_n": best[2], "stages": best[3]}
        report[m] = best_us
        print(f"M={m:5d}: best {best} {best_us:9.1f} us", flush=True)
    out_file = args.out_file or f"moe_b200_E{e_total}_I{n // 2}_K{k}.json"
    os.makedirs(os.path.dirname(os.path.abspath(out_file)), exist_ok=True)
    with open(out_file, "w") as f:
        json.dump(table, f)
    print("wrote", out_file)
    return table, report


if __name__ == "__main__":
    main()
