#!/usr/bin/env python
"""Benchmark of the fused W8A8 MoE layer (torch.ops.alpha_moe.fused_moe_w8a8_up_down) on B200.

One "step" = one MoE layer call on one batch of M tokens: zero `out`, run the fused kernel on this
rank's shard of the intermediate dimension, and (N > 1) all-reduce the partial bf16 outputs.
Workload at every N: the DeepSeek-V3 TP8 shard per GPU (E=257 incl. the shared expert, K=7168,
I=256 per GPU, top_k=8+1, routed_scaling_factor=2.5), i.e. N GPUs serve a layer whose
intermediate size is 256*N ("weak" scaling; N=8 is the real DeepSeek-V3 layer, I=2048, TP8).
Inputs are synthetic: random fp8 weights / activations and seeded N(0,1) router logits -> top-8
-> softmax -> renormalise, plus the always-on shared expert.

Prints ONE JSON line (rank 0).  `--impl reference` instead times the CPU restatement of the
operator (oracle/, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

E, K, I_PER_GPU, TOP_K, SCALING = 257, 7168, 256, 9, 2.5
SWEEP_MS = [1, 4, 16, 64, 256, 1024, 4096]
FP8_MAX_BYTE = 0x78   # random bytes below this are finite e4m3 values

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused kernel, from the ncu
# capture summarised under profiles/ (bytes per launch, keyed by M); None = not captured.
NCU_DRAM_TRAFFIC = {1: 49.66e6 + 0.04e6, 64: 1.2302e9 + 5.9e6, 4096: 1.8186e9 + 139.9e6}


def best_knobs(m: int):
    """(block_m, block_n, warp_n, stages) per token count, from the tuned table if present."""
    from alpha_moe_b200.utils import get_best_config
    path = os.environ.get("ALPHA_MOE_CONFIG") or os.path.join(
        ROOT, "configs", f"moe_b200_E{E}_I{I_PER_GPU}_K{K}.json")
    if os.path.exists(path):
        c = get_best_config(path, m)
        return c["block_m"], c["block_n"], c["warp_n"], c["stages"]
    if m <= 8:
        return 16, 32, 8, 5
    if m <= 256:
        return 16, 32, 8, 3
    if m <= 1024:
        return 64, 64, 4, 5
    return 128, 64, 4, 3


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            pk = json.load(f)
        return {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops": float(pk["bf16_tflops"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def rand_fp8(shape, gen, dev):
    b = torch.randint(0, FP8_MAX_BYTE, shape, generator=gen, device=dev, dtype=torch.uint8)
    s = torch.randint(0, 2, shape, generator=gen, device=dev, dtype=torch.uint8) * 128
    return (b | s).view(torch.float8_e4m3fn)


def route(logits: torch.Tensor, k_routed: int, shared_expert: int):
    """Synthetic router: top-k of N(0,1) logits -> softmax over the k -> renormalise, plus the
    always-selected shared expert with weight 1."""
    vals, ids = torch.topk(logits.float(), k_routed, dim=-1)
    wts = torch.softmax(vals, dim=-1)
    wts = wts / wts.sum(dim=-1, keepdim=True)
    m = logits.shape[0]
    ids = torch.cat([ids.to(torch.int32), torch.full((m, 1), shared_expert, dtype=torch.int32)], 1)
    wts = torch.cat([wts, torch.ones(m, 1)], 1)
    return ids.contiguous(), wts.float().contiguous()


def align_block_size(topk_ids: torch.Tensor, block: int, num_experts: int):
    """Input generator for the benchmark: block schedule with the layout moe_align_block_size
    produces (each expert's assignments padded with the sentinel M*top_k to a multiple of block)."""
    flat = topk_ids.reshape(-1).to(torch.int64)
    numel = flat.numel()
    total = numel + num_experts * (block - 1)
    sorted_ids = torch.full((total,), numel, dtype=torch.int32)
    expert_ids = torch.zeros(((total + block - 1) // block,), dtype=torch.int32)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + block - 1) // block * block
    starts = torch.cumsum(padded, 0) - padded
    first = torch.cumsum(counts, 0) - counts
    e_of = flat[order]
    sorted_ids[starts[e_of] + torch.arange(numel) - first[e_of]] = order.to(torch.int32)
    n_pad = int(padded.sum())
    expert_ids[: n_pad // block] = torch.repeat_interleave(
        torch.arange(num_experts, dtype=torch.int32), padded // block)
    return sorted_ids, expert_ids, torch.tensor([n_pad], dtype=torch.int32)


class Workload:
    """Device-resident weights of this rank's shard and per-M inputs (identical on every rank)."""

    def __init__(self, dev, rank: int):
        self.dev = dev
        g = torch.Generator(device=dev).manual_seed(1234 + rank)
        self.w = rand_fp8((E, 2 * I_PER_GPU, K), g, dev)
        self.w2 = rand_fp8((E, K, I_PER_GPU), g, dev)
        self.w_scale = torch.rand(E, 2 * I_PER_GPU // 128, K // 128, generator=g, device=dev) * 2e-4 + 1e-4
        self.w2_scale = torch.rand(E, K // 128, I_PER_GPU // 128, generator=g, device=dev) * 2e-4 + 1e-4

    def inputs(self, m: int, block_m: int):
        gc = torch.Generator().manual_seed(99 + m)
        gd = torch.Generator(device=self.dev).manual_seed(99 + m)
        x = rand_fp8((m, K), gd, self.dev)
        x_scale = torch.rand(m, K // 128, generator=gd, device=self.dev) * 0.02 + 0.01
        logits = torch.randn(m, E - 1, generator=gc)
        ids, wts = route(logits, TOP_K - 1, E - 1)
        sid, eid, npp = align_block_size(ids, block_m, E)
        return {"x": x, "x_scale": x_scale, "ids": ids, "topk_weights": wts, "sid": sid, "eid": eid,
                "npp": npp, "e_active": int(torch.unique(ids).numel())}


def algorithmic_bytes(m: int, e_active: int, sorted_num: int) -> float:
    """Bytes one layer call must move: fp8 weights + block scales of the experts hit, x, x_scale,
    out written once, topk weights and the block schedule."""
    inter = I_PER_GPU
    per_expert = 3 * inter * K + 4 * ((2 * inter // 128) * (K // 128) + (K // 128) * (inter // 128))
    return float(e_active * per_expert + m * K + 4 * m * K // 128 + 2 * m * K + 8 * m * TOP_K + 4 * sorted_num)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


def cpu_sample(wl_cpu, inp, m, n_experts_sample, reps, threads):
    """Times the CPU restatement on the sub-problem 'assignments routed to the first
    n_experts_sample experts' of the bench workload; returns (TFLOP/s, seconds per rep, n_assign)."""
    from oracle import moe_oracle as orc
    torch.set_num_threads(threads)
    ids = inp["ids"]
    keep = ids < n_experts_sample
    n_assign = int(keep.sum())
    # Assignments to other experts are sent to a dummy last expert whose blocks are then cut off.
    ids_s = torch.where(keep, ids, torch.full_like(ids, n_experts_sample))
    sid, eid, npp = align_block_size(ids_s, 16, n_experts_sample + 1)
    n_real_blocks = int((eid[: int(npp) // 16] < n_experts_sample).sum())
    npp = torch.tensor([n_real_blocks * 16], dtype=torch.int32)
    args = (inp["x_cpu"], inp["x_scale_cpu"], wl_cpu["w"], wl_cpu["w_scale"], wl_cpu["w2"], wl_cpu["w2_scale"],
            sid, eid, npp, inp["topk_weights"], TOP_K, 16, SCALING)
    orc.fused_moe_w8a8_up_down_oracle(*args)            # warm-up
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.fused_moe_w8a8_up_down_oracle(*args)
    dt = (time.perf_counter() - t0) / reps
    flops = 6.0 * n_assign * I_PER_GPU * K
    return flops / dt / 1e12, dt, n_assign


def run_reference(args, rank, world):
    """CPU arm: the oracle restatement (kind 'port'; the reference has no CPU implementation and its
    CUDA kernel is Hopper-only) on a bounded sample, all host threads, rank 0 only."""
    if rank != 0:
        return
    m = args.m
    threads = os.cpu_count() or 1
    n_s = args.cpu_experts
    g = torch.Generator().manual_seed(1234)
    shape_w, shape_w2 = (n_s, 2 * I_PER_GPU, K), (n_s, K, I_PER_GPU)
    wl_cpu = {
        "w": torch.randint(0, FP8_MAX_BYTE, shape_w, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn),
        "w2": torch.randint(0, FP8_MAX_BYTE, shape_w2, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn),
        "w_scale": torch.rand(n_s, 4, K // 128, generator=g) * 2e-4 + 1e-4,
        "w2_scale": torch.rand(n_s, K // 128, 2, generator=g) * 2e-4 + 1e-4,
    }
    gc = torch.Generator().manual_seed(99 + m)
    logits = torch.randn(m, E - 1, generator=gc)
    ids, wts = route(logits, TOP_K - 1, E - 1)
    inp = {"ids": ids, "topk_weights": wts,
           "x_cpu": torch.randint(0, FP8_MAX_BYTE, (m, K), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn),
           "x_scale_cpu": torch.rand(m, K // 128, generator=g) * 0.02 + 0.01}
    for _ in range(max(args.warmup - 1, 0)):
        cpu_sample(wl_cpu, inp, m, n_s, 1, threads)
    tf, dt, n_assign = cpu_sample(wl_cpu, inp, m, n_s, max(args.steps, 1), threads)
    sample = (f"assignments routed to the first {n_s} of {E} experts at M={m} "
              f"({n_assign} of {m * TOP_K}), dequantise + matmul per expert")
    line = {
        "impl": "reference", "metric": "fused_moe_layer_tflops", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dequantised fp8)",
        "data": "synthetic",
        "config": workload_config(m, args.gpus),
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(m, n_gpus):
    return {"workload": f"DeepSeek-V3 TP8 MoE shard per GPU: E={E} (256 routed + shared), K={K}, "
                        f"I={I_PER_GPU} per GPU (layer I={I_PER_GPU * n_gpus}), top_k=8+1, scaling={SCALING}, M={m}",
            "M": m, "E": E, "K": K, "I_per_gpu": I_PER_GPU, "top_k": TOP_K,
            "parallelism": f"tp{n_gpus} over the intermediate dimension + all-reduce" if n_gpus > 1 else "single GPU",
            "l2": "weights (1.4 GB) exceed L2 and a 256 MB buffer is overwritten between timed steps"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=4096, help="tokens per step of the headline number")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-experts", type=int, default=257, help="experts in the CPU sample (257 = the whole workload)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback of the operator)")
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner on stdout while the communicator comes up (when NCCL_DEBUG asks for
        # one); stdout must carry the one JSON line only, so it points at stderr until the first collective is done
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)

    import alpha_moe  # noqa: F401  registers torch.ops.alpha_moe.fused_moe_w8a8_up_down
    from alpha_moe_b200 import capi
    op = torch.ops.alpha_moe.fused_moe_w8a8_up_down
    peaks = load_peaks()
    wl = Workload(dev, rank)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def prepare(m):
        bm, bn, wn, st = best_knobs(m)
        inp = wl.inputs(m, bm)
        d = {k: inp[k].to(dev) for k in ("sid", "eid", "npp", "topk_weights")}
        out = torch.zeros(m, K, dtype=torch.bfloat16, device=dev)

        def call():
            op(inp["x"], inp["x_scale"], wl.w, wl.w_scale, wl.w2, wl.w2_scale, d["sid"], d["eid"], d["npp"],
               d["topk_weights"], out, TOP_K, bm, bn, wn, st, SCALING)
        return inp, d, out, call, (bm, bn, wn, st)

    def time_steps(m, steps, warmup):
        """Returns (ms per whole step, ms per fused-kernel launch), max over ranks."""
        inp, d, out, call, knobs = prepare(m)
        for _ in range(warmup):
            out.zero_()
            call()
            if world > 1:
                dist.all_reduce(out)
        barrier()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        for i in range(steps):
            flush.fill_(i & 0xFF)                     # evict L2 between timed steps (not timed)
            ev[i][0].record()
            out.zero_()
            ev[i][1].record()
            call()
            ev[i][2].record()
            if world > 1:
                dist.all_reduce(out)
            ev[i][3].record()
        barrier()
        step_ms = sum(e[0].elapsed_time(e[3]) for e in ev) / steps
        kern_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
        if world > 1:
            t = torch.tensor([step_ms, kern_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            step_ms, kern_ms = float(t[0]), float(t[1])
        return step_ms, kern_ms, inp, knobs

    def time_e2e(m, steps, warmup):
        """Same step through the public operator with HOST inputs: every step copies its pinned x / scales /
        routing to the device, runs the layer and copies `out` back, all inside the timed region.  The three
        stages of consecutive steps run on three streams over two sets of buffers (copy-in of step i+1 and
        copy-out of step i-1 overlap the layer of step i), as a serving loop would issue them."""
        inp, d, out, _, (bm, bn, wn, st) = prepare(m)
        host = {"x": inp["x"].cpu().pin_memory(), "x_scale": inp["x_scale"].cpu().pin_memory(),
                "topk_weights": inp["topk_weights"].pin_memory(), "sid": inp["sid"].pin_memory(),
                "eid": inp["eid"].pin_memory(), "npp": inp["npp"].pin_memory()}
        depth = 2
        dbuf = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(depth)]
        outs = [out] + [torch.empty_like(out) for _ in range(depth - 1)]
        out_host = [torch.empty(m, K, dtype=torch.bfloat16).pin_memory() for _ in range(depth)]
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        d2h = out_host[0].numel() * out_host[0].element_size()
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(depth)]
        ev_run = [torch.cuda.Event() for _ in range(depth)]
        ev_out = [torch.cuda.Event() for _ in range(depth)]
        main = torch.cuda.current_stream()

        def step(i):
            j = i % depth
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_run[j])            # the layer that last read this input set has finished
                for k, v in host.items():
                    dbuf[j][k].copy_(v, non_blocking=True)
                ev_in[j].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[j])
                s_run.wait_event(ev_out[j])           # the previous result in this output buffer has been copied out
                outs[j].zero_()
                op(dbuf[j]["x"], dbuf[j]["x_scale"], wl.w, wl.w_scale, wl.w2, wl.w2_scale, dbuf[j]["sid"],
                   dbuf[j]["eid"], dbuf[j]["npp"], dbuf[j]["topk_weights"], outs[j], TOP_K, bm, bn, wn, st, SCALING)
                if world > 1:
                    dist.all_reduce(outs[j])
                ev_run[j].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[j])
                out_host[j].copy_(outs[j], non_blocking=True)
                ev_out[j].record(s_out)

        def drain():
            for s_ in (s_in, s_run, s_out):
                main.wait_stream(s_)

        for s_ in (s_in, s_run, s_out):
            s_.wait_stream(main)
        for i in range(warmup):
            step(i)
        drain()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        for s_ in (s_in, s_run, s_out):
            s_.wait_event(e0)
        for i in range(steps):
            step(warmup + i)
        drain()
        e1.record(main)
        barrier()
        ms = e0.elapsed_time(e1) / steps
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms, h2d, d2h

    m = args.m
    sampler = ClockSampler(physical_gpu_index(local_rank)) if rank == 0 else None
    if sampler:
        sampler.start()
    step_ms, kern_ms, inp, knobs = time_steps(m, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    e2e_ms, h2d, d2h = time_e2e(m, args.steps, args.warmup)

    flops_per_gpu = 6.0 * m * TOP_K * I_PER_GPU * K
    flops_job = flops_per_gpu * world
    abytes = algorithmic_bytes(m, inp["e_active"], inp["sid"].numel())
    wbytes = inp["e_active"] * 3.0 * I_PER_GPU * K
    fp8_peak = 2.0 * peaks["bf16_tflops"]             # dense fp8 = 2 x the measured bf16 GEMM rate
    t_hbm = abytes / (peaks["hbm_gbs"] * 1e9)
    t_fp8 = flops_per_gpu / (fp8_peak * 1e12)
    bound = "hbm" if t_hbm >= t_fp8 else "tensor"
    if bound == "hbm":
        achieved, peak, unit = abytes / (kern_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = flops_per_gpu / (kern_ms * 1e-3) / 1e12, fp8_peak, "TFLOP/s"

    sweep = []
    if not args.no_sweep:
        for ms_ in SWEEP_MS:
            s_ms, k_ms, sinp, sk = time_steps(ms_, 10, 3)
            fl = 6.0 * ms_ * TOP_K * I_PER_GPU * K
            wb = sinp["e_active"] * 3.0 * I_PER_GPU * K
            sweep.append({"M": ms_, "us_kernel": round(k_ms * 1e3, 1), "us_step": round(s_ms * 1e3, 1),
                          "tflops_job": round(fl * world / (s_ms * 1e-3) / 1e12, 2),
                          "e_active": sinp["e_active"],
                          "frac_hbm_weights": round(wb / (k_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 3),
                          "frac_fp8": round(fl / (k_ms * 1e-3) / 1e12 / fp8_peak, 3),
                          "knobs": list(sk)})

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n_s = args.cpu_experts
        wl_cpu = {"w": wl.w[:n_s].cpu(), "w2": wl.w2[:n_s].cpu(), "w_scale": wl.w_scale[:n_s].cpu(),
                  "w2_scale": wl.w2_scale[:n_s].cpu()}
        inp["x_cpu"], inp["x_scale_cpu"] = inp["x"].cpu(), inp["x_scale"].cpu()
        threads = os.cpu_count() or 1
        tf, dt, n_assign = cpu_sample(wl_cpu, inp, m, n_s, 8, threads)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"assignments routed to the first {n_s} of {E} experts at M={m} "
                         f"({n_assign} of {m * TOP_K}), {dt:.2f} s per pass"}

    status = capi.read_status(reset=True)
    if rank == 0:
        line = {
            "metric": "fused_moe_layer_tflops", "value": flops_job / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate)",
            "data": "synthetic", "config": workload_config(m, world),
            "us_per_layer_kernel": kern_ms * 1e3,
            "knobs": {"block_m": knobs[0], "block_n": knobs[1], "warp_n": knobs[2], "stages": knobs[3]},
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                         "frac": achieved / peak, "traffic": NCU_DRAM_TRAFFIC.get(m),
                         "peak_source": peaks["source"] + ("" if bound == "hbm" else "; fp8 = 2 x bf16"),
                         "algorithmic_bytes": abytes, "weight_bytes": wbytes,
                         "frac_hbm_weights_only": wbytes / (kern_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                         "frac_fp8_tensor": flops_per_gpu / (kern_ms * 1e-3) / 1e12 / fp8_peak,
                         "t_hbm_us": t_hbm * 1e6, "t_fp8_us": t_fp8 * 1e6},
            "e2e": {"value": flops_job / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "pipeline": "copy-in / layer / copy-out of consecutive steps on three streams, two buffer sets"},
            "gpu_launches": args.steps,
            "clocks": clocks, "kernel_status": list(status), "sweep": sweep,
        }
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
