#!/usr/bin/env python
"""Benchmark of the fused W8A8 MoE layer (torch.ops.alpha_moe.fused_moe_w8a8_up_down) on B200.

One "step" = one MoE layer call on one batch of M tokens: zero `out`, run the fused kernel on this
rank's shard of the intermediate dimension, and (N > 1) all-reduce the partial bf16 outputs (with NCCL or with
this library's own all-reduce kernel over peer-mapped buffers; the headline takes the faster, `exchange` says which).

Headline workload at every N: the DeepSeek-V3 TP8 shard per GPU (E=257 incl. the shared expert,
K=7168, I=256 per GPU, top_k=8+1, routed_scaling_factor=2.5), M=4096, i.e. N GPUs serve a layer whose
intermediate size is 256*N ("weak" scaling; N=8 is the real DeepSeek-V3 layer, I=2048, TP8).
Beside the headline the JSON line carries sub-records for the rest of the metric:
  sweep    the headline shape over M = 1 ... 8192 (at N > 1 and M <= 64 also with this library's own
           exchange kernel over peer-mapped memory instead of the all-reduce call: us_step_own_exchange; *_graph =
           the step replayed from a CUDA graph)
  qwen3    the Qwen3-Next TP2 shard (E=512, K=2048, I=256, top_k=10) over M      (1 GPU only)
  zipf     the headline shape at M=8192 with Zipf(1.2) routing                   (1 GPU only)
  imbalance  the headline shape at M=256 and 4096 under the reference script's balancedness levels 0.8 ... 0.5 (1 GPU only)
  tp_fixed the unsharded layer I=2048 split I/N per GPU ("strong" scaling) at M = 1, 64, 1024, 8192
  layer    the whole call-site sequence from bf16 activations and topk_ids (quantise + clear + schedule
           + operator, one C-ABI call) over M
Inputs are synthetic: random fp8 weights / activations and seeded N(0,1) router logits -> top-k
-> softmax -> renormalise, plus the always-on shared expert where the shape has one.

Prints ONE JSON line (rank 0).  `--impl reference` instead times the CPU restatement of the
operator (oracle/, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FP8_MAX_BYTE = 0x78   # random bytes below this are finite e4m3 values


class Shape:
    """One MoE shard shape: E experts (the last one shared and always selected if `shared`), hidden K,
    intermediate I per GPU, top_k (counting the shared expert), routed scaling factor."""

    def __init__(self, name, e, k, inter, top_k, scaling, shared):
        self.name, self.e, self.k, self.inter, self.top_k, self.scaling, self.shared = name, e, k, inter, top_k, scaling, shared

    def table(self):
        return os.path.join(ROOT, "configs", f"moe_b200_E{self.e}_I{self.inter}_K{self.k}.json")

    def flops(self, m):
        return 6.0 * m * self.top_k * self.inter * self.k

    def expert_bytes(self):
        i, k = self.inter, self.k
        return 3 * i * k + 4 * ((2 * i // 128) * (k // 128) + (k // 128) * (i // 128))

    def algorithmic_bytes(self, m, e_active, sorted_num):
        """Bytes one layer call must move: fp8 weights + block scales of the experts hit, x, x_scale, out written
        once, topk weights and the block schedule."""
        k = self.k
        return float(e_active * self.expert_bytes() + m * k + 4 * m * k // 128 + 2 * m * k + 8 * m * self.top_k + 4 * sorted_num)


DEEPSEEK = Shape("DeepSeek-V3 TP8 MoE shard", 257, 7168, 256, 9, 2.5, True)
QWEN3 = Shape("Qwen3-Next TP2 MoE shard", 512, 2048, 256, 10, 1.0, False)
SWEEP_MS = [1, 4, 16, 64, 256, 1024, 2048, 4096, 8192]
QWEN_MS = [1, 16, 64, 256, 1024, 4096]
TP_FIXED_MS = [1, 64, 1024, 8192]
LAYER_MS = [1, 64, 1024, 4096]
GRAPH_MAX_M = 256          # step times at or below this M are also taken from CUDA-graph replays
I_FULL = 2048              # intermediate size of the unsharded DeepSeek-V3-like layer (tp_fixed)
# legacy names used by development scripts
E, K, I_PER_GPU, TOP_K, SCALING = DEEPSEEK.e, DEEPSEEK.k, DEEPSEEK.inter, DEEPSEEK.top_k, DEEPSEEK.scaling


def best_knobs(shape: Shape, m: int):
    """(block_m, block_n, warp_n, stages) per token count: from the tuned table of the shape if there is one
    ($ALPHA_MOE_CONFIG overrides the DeepSeek shard's), else a rule of thumb."""
    from alpha_moe_b200.utils import get_best_config
    path = shape.table()
    if shape is DEEPSEEK and os.environ.get("ALPHA_MOE_CONFIG"):
        path = os.environ["ALPHA_MOE_CONFIG"]
    if os.path.exists(path):
        c = get_best_config(path, m)
        return c["block_m"], c["block_n"], c["warp_n"], c["stages"]
    if m <= 8:
        return 16, 32, 8, 5
    if m <= 256:
        return 16, 32, 8, 3
    if m <= 1024:
        return 64, 64, 4, 2
    return 128, 64, 4, 3


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            pk = json.load(f)
        return {"hbm_gbs": float(pk["hbm_gbs"]), "bf16_tflops": float(pk["bf16_tflops"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def load_ncu_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the fused kernel from the committed ncu summary
    (profiles/fused_moe_dram_traffic.md: table rows `| shape | M | kernel | read bytes | written bytes |`)."""
    out = {}
    path = os.path.join(ROOT, "profiles", "fused_moe_dram_traffic.md")
    if not os.path.exists(path):
        return out
    row = re.compile(r"^\|\s*(\w+)\s*\|\s*(\d+)\s*\|\s*([^|]+?)\s*\|\s*([0-9.eE+]+)\s*\|\s*([0-9.eE+]+)\s*\|")
    with open(path) as f:
        for line in f:
            mt = row.match(line)
            if mt:
                out[(mt.group(1), int(mt.group(2)))] = {"kernel": mt.group(3), "bytes": float(mt.group(4)) + float(mt.group(5))}
    return out


def rand_fp8(shape, gen, dev):
    b = torch.randint(0, FP8_MAX_BYTE, shape, generator=gen, device=dev, dtype=torch.uint8)
    s = torch.randint(0, 2, shape, generator=gen, device=dev, dtype=torch.uint8) * 128
    return (b | s).view(torch.float8_e4m3fn)


def route(logits: torch.Tensor, k_routed: int, shared_expert):
    """Synthetic router: top-k of N(0,1) logits -> softmax over the k -> renormalise, plus (if given) the
    always-selected shared expert with weight 1."""
    vals, ids = torch.topk(logits.float(), k_routed, dim=-1)
    wts = torch.softmax(vals, dim=-1)
    wts = wts / wts.sum(dim=-1, keepdim=True)
    ids = ids.to(torch.int32)
    if shared_expert is not None:
        m = logits.shape[0]
        ids = torch.cat([ids, torch.full((m, 1), shared_expert, dtype=torch.int32)], 1)
        wts = torch.cat([wts, torch.ones(m, 1)], 1)
    return ids.contiguous(), wts.float().contiguous()


def route_zipf(m, n_routed, k_routed, s, gen, shared_expert):
    """Skewed routing: routed expert ids drawn without replacement inside a token from a Zipf(s) law."""
    p = 1.0 / torch.arange(1, n_routed + 1, dtype=torch.float64) ** s
    ids = torch.multinomial((p / p.sum()).float().expand(m, -1), k_routed, replacement=False, generator=gen).to(torch.int32)
    wts = torch.softmax(torch.randn(m, k_routed, generator=gen), -1)
    if shared_expert is not None:
        ids = torch.cat([ids, torch.full((m, 1), shared_expert, dtype=torch.int32)], 1)
        wts = torch.cat([wts, torch.ones(m, 1)], 1)
    return ids.contiguous(), wts.float().contiguous()


def route_mixture(m, n_routed, k_routed, balancedness, gen, shared_expert):
    """The imbalance model of the reference's timing script (test/test_moe_performance.py:42-49): every routed
    assignment is drawn independently - so an expert may repeat inside a token - from balancedness x uniform +
    (1 - balancedness) x "always expert 0"."""
    p = torch.full((n_routed,), balancedness / n_routed, dtype=torch.float32)
    p[0] += 1.0 - balancedness
    ids = torch.multinomial(p, m * k_routed, replacement=True, generator=gen).view(m, k_routed).to(torch.int32)
    wts = torch.softmax(torch.randn(m, k_routed, generator=gen), -1)
    if shared_expert is not None:
        ids = torch.cat([ids, torch.full((m, 1), shared_expert, dtype=torch.int32)], 1)
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

    def __init__(self, shape: Shape, dev, rank: int):
        self.shape, self.dev = shape, dev
        e, k, i = shape.e, shape.k, shape.inter
        g = torch.Generator(device=dev).manual_seed(1234 + rank)
        self.w = rand_fp8((e, 2 * i, k), g, dev)
        self.w2 = rand_fp8((e, k, i), g, dev)
        self.w_scale = torch.rand(e, 2 * i // 128, k // 128, generator=g, device=dev) * 2e-4 + 1e-4
        self.w2_scale = torch.rand(e, k // 128, i // 128, generator=g, device=dev) * 2e-4 + 1e-4

    def inputs(self, m: int, block_m: int, zipf: float | None = None):
        sh = self.shape
        gc = torch.Generator().manual_seed(99 + m)
        gd = torch.Generator(device=self.dev).manual_seed(99 + m)
        x = rand_fp8((m, sh.k), gd, self.dev)
        x_scale = torch.rand(m, sh.k // 128, generator=gd, device=self.dev) * 0.02 + 0.01
        n_routed = sh.e - 1 if sh.shared else sh.e
        k_routed = sh.top_k - 1 if sh.shared else sh.top_k
        shared = sh.e - 1 if sh.shared else None
        if isinstance(zipf, tuple):        # ("balancedness", b): the reference script's imbalance model
            ids, wts = route_mixture(m, n_routed, k_routed, zipf[1], torch.Generator().manual_seed(2), shared)
        elif zipf is None:
            ids, wts = route(torch.randn(m, n_routed, generator=gc), k_routed, shared)
        else:
            # the law covers the first 240 routed experts: the other 16 receive nothing (empty experts in the schedule)
            ids, wts = route_zipf(m, min(n_routed, 240), k_routed, zipf, torch.Generator().manual_seed(1), shared)
        sid, eid, npp = align_block_size(ids, block_m, sh.e)
        return {"x": x, "x_scale": x_scale, "ids": ids, "topk_weights": wts, "sid": sid, "eid": eid,
                "npp": npp, "e_active": int(torch.unique(ids).numel())}


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


def cpu_sample(shape: Shape, wl_cpu, inp, m, n_experts_sample, reps, threads):
    """Times the CPU restatement on the sub-problem 'assignments routed to the first n_experts_sample experts' of
    the bench workload (one I-per-GPU shard); returns (TFLOP/s, seconds per rep, n_assign)."""
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
            sid, eid, npp, inp["topk_weights"], shape.top_k, 16, shape.scaling)
    orc.fused_moe_w8a8_up_down_oracle(*args)            # warm-up
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.fused_moe_w8a8_up_down_oracle(*args)
    dt = (time.perf_counter() - t0) / reps
    return 6.0 * n_assign * shape.inter * shape.k / dt / 1e12, dt, n_assign


def workload_config(shape: Shape, m, n_gpus):
    return {"workload": f"{shape.name} per GPU: E={shape.e} (256 routed + shared), K={shape.k}, "
                        f"I={shape.inter} per GPU (layer I={shape.inter * n_gpus}), top_k=8+1, scaling={shape.scaling}, M={m}",
            "M": m, "E": shape.e, "K": shape.k, "I_per_gpu": shape.inter, "top_k": shape.top_k,
            "parallelism": f"tp{n_gpus} over the intermediate dimension + all-reduce" if n_gpus > 1 else "single GPU",
            "l2": "weights (1.4 GB) exceed L2 and a 256 MB buffer is overwritten between timed steps"}


def run_reference(args, rank, world):
    """CPU arm: the oracle restatement (kind 'port'; the reference has no CPU implementation and its CUDA kernel is
    Hopper-only) on a bounded sample, all host threads, rank 0 only.  It always runs ONE shard of the headline
    shape (I=256): at N > 1 that is rank 0's share of the layer, without the exchange step."""
    if rank != 0:
        return
    sh, m = DEEPSEEK, args.m
    threads = os.cpu_count() or 1
    n_s = args.cpu_experts
    g = torch.Generator().manual_seed(1234)
    shape_w, shape_w2 = (n_s, 2 * sh.inter, sh.k), (n_s, sh.k, sh.inter)
    wl_cpu = {
        "w": torch.randint(0, FP8_MAX_BYTE, shape_w, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn),
        "w2": torch.randint(0, FP8_MAX_BYTE, shape_w2, generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn),
        "w_scale": torch.rand(n_s, 4, sh.k // 128, generator=g) * 2e-4 + 1e-4,
        "w2_scale": torch.rand(n_s, sh.k // 128, 2, generator=g) * 2e-4 + 1e-4,
    }
    gc = torch.Generator().manual_seed(99 + m)
    ids, wts = route(torch.randn(m, sh.e - 1, generator=gc), sh.top_k - 1, sh.e - 1)
    inp = {"ids": ids, "topk_weights": wts,
           "x_cpu": torch.randint(0, FP8_MAX_BYTE, (m, sh.k), generator=g, dtype=torch.uint8).view(torch.float8_e4m3fn),
           "x_scale_cpu": torch.rand(m, sh.k // 128, generator=g) * 0.02 + 0.01}
    for _ in range(max(args.warmup - 1, 0)):
        cpu_sample(sh, wl_cpu, inp, m, n_s, 1, threads)
    tf, dt, n_assign = cpu_sample(sh, wl_cpu, inp, m, n_s, max(args.steps, 1), threads)
    sample = (f"one I={sh.inter} shard on rank 0: assignments routed to the first {n_s} of {sh.e} experts at M={m} "
              f"({n_assign} of {m * sh.top_k}), dequantise + matmul per expert"
              + ("" if args.gpus == 1 else f"; the other {args.gpus - 1} shards and the exchange step are not run"))
    cfg = workload_config(sh, m, args.gpus)
    cfg["cpu_arm_runs"] = "one shard (I=256) of the layer on rank 0's host cores, no exchange step"
    line = {
        "impl": "reference", "metric": "fused_moe_layer_tflops", "value": tf, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dequantised fp8)",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=4096, help="tokens per step of the headline number")
    ap.add_argument("--no-sweep", action="store_true", help="skip the M sweep and the other sub-records")
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
    fp8_peak = 2.0 * peaks["bf16_tflops"]             # dense fp8 taken as 2 x the measured bf16 GEMM rate
    fp8_note = "dense fp8 peak = 2 x the measured bf16 GEMM rate (no fp8 measurement exists)"
    traffic = load_ncu_traffic()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    launches = [0]                                    # launches of this library's kernels inside timed regions

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        if world == 1:
            return vals
        t = torch.tensor(vals, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return tuple(float(v) for v in t)

    def prepare(wl, m, zipf=None):
        sh = wl.shape
        bm, bn, wn, st = best_knobs(sh, m)
        inp = wl.inputs(m, bm, zipf)
        d = {k: inp[k].to(dev) for k in ("sid", "eid", "npp", "topk_weights")}
        out = torch.zeros(m, sh.k, dtype=torch.bfloat16, device=dev)

        def call(o=out):
            op(inp["x"], inp["x_scale"], wl.w, wl.w_scale, wl.w2, wl.w2_scale, d["sid"], d["eid"], d["npp"],
               d["topk_weights"], o, sh.top_k, bm, bn, wn, st, sh.scaling)
        return inp, d, out, call, (bm, bn, wn, st)

    own_ar, own_notes = {}, {}

    def make_on_all_ranks(what, fn):
        """Creates a peer-mapped helper on every rank; if it fails on any rank (symmetric memory not available, ...)
        every rank drops it, so that the ranks keep issuing the same collectives.  Returns the object or None."""
        try:
            obj, err = fn(), ""
        except Exception as e:      # noqa: BLE001 - reported in the JSON line, the NCCL path still runs
            obj, err = None, f"{type(e).__name__}: {str(e)[:200]}"
        ok = torch.tensor([1 if obj is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok) == 0:
            own_notes[what] = err or "failed on another rank"
            return None
        return obj

    def peer_all_reduce(hidden):
        """This library's all-reduce over peer-mapped output buffers (alpha_moe_b200.tp.PeerAllReduce), made once."""
        if hidden not in own_ar:
            from alpha_moe_b200.tp import PeerAllReduce
            own_ar[hidden] = make_on_all_ranks("own_allreduce", lambda: PeerAllReduce(max(SWEEP_MS), hidden, timeout_ms=2000))
        return own_ar[hidden]

    last_median = [0.0]

    def time_steps(wl, m, steps, warmup, zipf=None, own_exchange=False):
        """(ms per whole step, ms per fused-kernel launch) as the max over ranks, inputs, knobs.  The exchange step at
        N > 1 is the NCCL all-reduce, or with own_exchange this library's all-reduce kernel over peer-mapped buffers."""
        inp, d, out, call, knobs = prepare(wl, m, zipf)
        ar = peer_all_reduce(wl.shape.k) if (own_exchange and world > 1) else None

        def one(ev=None):
            if ev:
                ev[0].record()
            buf = ar.next_buffer(m) if ar else out.zero_()
            if ev:
                ev[1].record()
            call(buf)
            if ev:
                ev[2].record()
            if ar:
                ar.reduce_scatter() if own_exchange == "reduce_scatter" else ar.all_reduce()
            elif world > 1:
                dist.all_reduce(out)
            if ev:
                ev[3].record()
        for _ in range(warmup):
            one()
        barrier()
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
        for i in range(steps):
            flush.fill_(i & 0xFF)                     # evict L2 between timed steps (not timed)
            one(ev[i])
        barrier()
        launches[0] += steps
        per_step = sorted(e[0].elapsed_time(e[3]) for e in ev)
        step_ms = sum(per_step) / steps
        kern_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / steps
        step_ms, kern_ms, med = max_over_ranks(step_ms, kern_ms, per_step[steps // 2])
        last_median[0] = med                         # one late host thread on one rank moves the mean of ten steps a lot
        return step_ms, kern_ms, inp, knobs

    def host_us_per_call(wl, m, calls=300):
        """CPU time of one operator call (no synchronisation inside the loop): through the torch dispatcher and
        through the C ABI directly.  At M = 1 the kernel's HBM bound is a few microseconds, so this matters."""
        inp, d, out, call, (bm, bn, wn, st) = prepare(wl, m)
        sh = wl.shape
        stream = torch.cuda.current_stream().cuda_stream
        ptrs = (inp["x"].data_ptr(), inp["x_scale"].data_ptr(), wl.w.data_ptr(), wl.w_scale.data_ptr(), wl.w2.data_ptr(),
                wl.w2_scale.data_ptr(), out.data_ptr(), d["sid"].data_ptr(), d["eid"].data_ptr(), d["npp"].data_ptr(),
                d["topk_weights"].data_ptr())

        def raw():
            capi.fused_moe_w8a8_up_down(*ptrs, sh.top_k, m, sh.k, 2 * sh.inter, sh.e, inp["sid"].numel(), bm, bn, wn, st,
                                        sh.scaling, stream)
        res = {}
        for name, fn in (("torch_op", call), ("c_abi", raw)):
            fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(calls):
                fn()
            res[name] = round((time.perf_counter() - t0) / calls * 1e6, 2)
            torch.cuda.synchronize()
        launches[0] += 2 * calls
        return res

    fused_tp = {}

    def time_graph_step(wl, m, steps, own_exchange=False):
        """The step replayed from a CUDA graph, as a serving engine's decode loop issues it: below a few hundred
        tokens the eager step is bound by the host's launch path, not by the GPU.  A step is: clear `out` +
        fused kernel (+ NCCL all-reduce at N > 1), or with own_exchange (N > 1) this library's PeerReducedLayer: fused
        kernel + barrier / sum / clear kernel over peer-mapped memory.  Returns ms per step, max over ranks."""
        inp, d, out, call, (bm, bn, wn, st) = prepare(wl, m)
        sh = wl.shape
        if own_exchange:
            from alpha_moe_b200.tp import PeerReducedLayer
            if "layer" not in fused_tp:
                fused_tp["layer"] = make_on_all_ranks("own_exchange", lambda: PeerReducedLayer(64, sh.k, timeout_ms=2000))
            lay = fused_tp["layer"]
            if lay is None:
                return None

            def one():
                lay.run(inp["x"], inp["x_scale"], wl.w, wl.w_scale, wl.w2, wl.w2_scale, d["sid"], d["eid"], d["npp"],
                        d["topk_weights"], sh.top_k, bm, bn, wn, st, sh.scaling)
        else:
            def one():
                out.zero_()
                call()
                if world > 1:
                    dist.all_reduce(out)
        # One step per graph, two graphs replayed alternately (the own exchange alternates between two buffers), the
        # L2 flushed before every replay: a second step inside the same graph would find the first one's weights in L2.
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        graphs = [torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()]
        with torch.cuda.stream(s):
            one()
            one()                                    # first calls outside the capture: attributes, tensor maps
            torch.cuda.synchronize()
            for g in graphs:
                with torch.cuda.graph(g, stream=s):
                    one()
        torch.cuda.current_stream().wait_stream(s)
        for i in range(4):
            graphs[i & 1].replay()
        barrier()
        ts = []
        for i in range(2 * steps):
            flush.fill_(i & 0xFF)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graphs[i & 1].replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        launches[0] += 2 * steps
        del graphs, g                                # before any communicator is torn down
        ts.sort()
        (ms,) = max_over_ranks(ts[len(ts) // 2])     # median: the ranks are re-aligned on the host before every replay
        return ms

    def time_fused_tp(wl, m, steps, warmup):
        """Small batches on N > 1 ranks with this library's own exchange step instead of the all-reduce call: the
        operator accumulates into a peer-mapped partial buffer, one kernel then waits for all ranks, sums all ranks'
        partials over NVLink and clears the next buffer (alpha_moe_b200.tp.PeerReducedLayer)."""
        from alpha_moe_b200.tp import PeerReducedLayer
        sh = wl.shape
        if "layer" not in fused_tp:
            fused_tp["layer"] = make_on_all_ranks("own_exchange", lambda: PeerReducedLayer(64, sh.k, timeout_ms=2000))
        lay = fused_tp["layer"]
        if lay is None:
            return None
        inp, d, _, _, (bm, bn, wn, st) = prepare(wl, m)
        tot = 0.0
        for i in range(warmup + steps):
            flush.fill_(i & 0xFF)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            lay.run(inp["x"], inp["x_scale"], wl.w, wl.w_scale, wl.w2, wl.w2_scale, d["sid"], d["eid"], d["npp"],
                    d["topk_weights"], sh.top_k, bm, bn, wn, st, sh.scaling)
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                tot += e0.elapsed_time(e1)
        launches[0] += 2 * steps
        (ms,) = max_over_ranks(tot / steps)
        return ms

    def time_fused_tp_train(wl, m, per_graph=8, replays=5):
        """The own-exchange step as a decode loop sees it: eight steps in ONE graph, the L2 overwritten between them
        inside the graph.  Only the first step of a replay absorbs the ranks' launch skew; from then on the exchange
        itself keeps the ranks together, as it does layer after layer in a model.  Per step = (the graph's time - the
        time of a graph that holds the eight L2 overwrites alone) / 8; medians over the replays, max over ranks.
        None if the peer-memory layer is unavailable or anything in here fails (on every rank alike)."""
        lay = fused_tp.get("layer")
        if lay is None:
            return None
        sh = wl.shape
        inp, d, _, _, (bm, bn, wn, st) = prepare(wl, m)

        def one():
            lay.run(inp["x"], inp["x_scale"], wl.w, wl.w_scale, wl.w2, wl.w2_scale, d["sid"], d["eid"], d["npp"],
                    d["topk_weights"], sh.top_k, bm, bn, wn, st, sh.scaling)

        def build():
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            g_steps, g_flush = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.stream(s):
                one()
                one()
                torch.cuda.synchronize()
                with torch.cuda.graph(g_steps, stream=s):
                    for k in range(per_graph):
                        flush.fill_(k)
                        one()
                with torch.cuda.graph(g_flush, stream=s):
                    for k in range(per_graph):
                        flush.fill_(k)
            torch.cuda.current_stream().wait_stream(s)
            return g_steps, g_flush
        graphs = make_on_all_ranks("own_exchange_train", build)
        if graphs is None:
            return None
        g_steps, g_flush = graphs

        def med(g):
            ts = []
            for _ in range(replays):
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ts.sort()
            return ts[len(ts) // 2]
        med(g_steps)                                 # warm-up replays
        t_steps, t_flush = med(g_steps), med(g_flush)
        launches[0] += 2 * per_graph * replays
        del graphs, g_steps, g_flush
        (ms,) = max_over_ranks((t_steps - t_flush) / per_graph)
        return ms

    def time_layer(wl, m, steps, warmup):
        """The call-site sequence as one C-ABI call (alpha_moe_b200_fused_experts): bf16 activations and topk_ids in,
        layer output in the same buffer: group quantisation + clearing + block schedule + fused operator."""
        sh = wl.shape
        bm, bn, wn, st = best_knobs(sh, m)
        inp = wl.inputs(m, bm)
        g = torch.Generator(device=dev).manual_seed(7 + m)
        x0 = torch.randn(m, sh.k, generator=g, device=dev).to(torch.bfloat16)
        hs = torch.empty_like(x0)
        ids, wts = inp["ids"].to(dev), inp["topk_weights"].to(dev)
        numel = m * sh.top_k
        total = numel + sh.e * (bm - 1)
        x_q = torch.empty(m, sh.k, dtype=torch.float8_e4m3fn, device=dev)
        x_s = torch.empty(m, sh.k // 128, dtype=torch.float32, device=dev)
        sid = torch.empty(total, dtype=torch.int32, device=dev)
        eid = torch.empty((total + bm - 1) // bm, dtype=torch.int32, device=dev)
        npp = torch.empty(1, dtype=torch.int32, device=dev)
        ws = torch.empty(max(capi.align_workspace_bytes(numel, sh.e), 4), dtype=torch.uint8, device=dev)
        stream = torch.cuda.current_stream().cuda_stream

        def call():
            capi.fused_experts(hs.data_ptr(), x_q.data_ptr(), x_s.data_ptr(), wl.w.data_ptr(), wl.w_scale.data_ptr(),
                               wl.w2.data_ptr(), wl.w2_scale.data_ptr(), ids.data_ptr(), wts.data_ptr(), sh.top_k, m, sh.k,
                               2 * sh.inter, sh.e, sid.data_ptr(), eid.data_ptr(), npp.data_ptr(), ws.data_ptr(), bm, bn, wn,
                               st, sh.scaling, stream)
        tot = 0.0
        for i in range(warmup + steps):
            hs.copy_(x0)
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            if i >= warmup:
                tot += e0.elapsed_time(e1)
        launches[0] += 3 * steps
        if m > GRAPH_MAX_M:
            return tot / steps, None
        # the same sequence replayed from a CUDA graph (the three launches of the eager call are host-bound at this size)
        s_ = torch.cuda.Stream()
        s_.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(s_):
            stream = s_.cuda_stream
            with torch.cuda.graph(g, stream=s_):
                call()
        torch.cuda.current_stream().wait_stream(s_)
        gtot = 0.0
        for i in range(steps):
            hs.copy_(x0)
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            gtot += e0.elapsed_time(e1)
        launches[0] += 3 * steps
        return tot / steps, gtot / steps

    def time_e2e(wl, m, steps, warmup):
        """Same step through the public operator with HOST inputs: every step copies its pinned x / scales / routing
        to the device, runs the layer and copies the result back, all inside the timed region.  The three stages of
        consecutive steps run on three streams over two sets of buffers (copy-in of step i+1 and copy-out of step i-1
        overlap the layer of step i), as a serving loop would issue them.  With N > 1 ranks each rank moves only its
        1/N of the token rows over PCIe: the rows are all-gathered over NVLink before the layer, and the partial
        outputs are reduce-scattered, so that each rank copies out the rows it copied in.
        Returns (ms per step, host->device bytes, device->host bytes) for the whole job."""
        sh = wl.shape
        inp, d, out, _, (bm, bn, wn, st) = prepare(wl, m)
        split = world > 1 and m % world == 0
        rows = m // world if split else m
        r0 = rank * rows if split else 0
        host = {"x": inp["x"][r0:r0 + rows].cpu().pin_memory(), "x_scale": inp["x_scale"][r0:r0 + rows].cpu().pin_memory(),
                "topk_weights": inp["topk_weights"][r0:r0 + rows].contiguous().pin_memory(), "sid": inp["sid"].pin_memory(),
                "eid": inp["eid"].pin_memory(), "npp": inp["npp"].pin_memory()}
        depth = 2
        dbuf = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(depth)]
        full = [{"x": torch.empty(m, sh.k, dtype=torch.uint8, device=dev),
                 "x_scale": torch.empty(m, sh.k // 128, dtype=torch.float32, device=dev),
                 "topk_weights": torch.empty(m, sh.top_k, dtype=torch.float32, device=dev)} for _ in range(depth)] if split else None
        outs = [out] + [torch.empty_like(out) for _ in range(depth - 1)]
        out_part = [torch.empty(rows, sh.k, dtype=torch.bfloat16, device=dev) for _ in range(depth)] if split else outs
        out_host = [torch.empty(rows, sh.k, dtype=torch.bfloat16).pin_memory() for _ in range(depth)]
        h2d = sum(v.numel() * v.element_size() for v in host.values()) * (world if split else 1)
        d2h = out_host[0].numel() * out_host[0].element_size() * (world if split else 1)
        if world > 1 and not split:      # every rank moves the whole batch
            h2d, d2h = h2d * world, d2h * world
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(depth)]
        ev_run = [torch.cuda.Event() for _ in range(depth)]
        ev_out = [torch.cuda.Event() for _ in range(depth)]
        main_stream = torch.cuda.current_stream()

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
                if split:
                    f = full[j]
                    dist.all_gather_into_tensor(f["x"], dbuf[j]["x"].view(torch.uint8))
                    dist.all_gather_into_tensor(f["x_scale"], dbuf[j]["x_scale"])
                    dist.all_gather_into_tensor(f["topk_weights"], dbuf[j]["topk_weights"])
                    xin, xsc, tw = f["x"].view(torch.float8_e4m3fn), f["x_scale"], f["topk_weights"]
                else:
                    xin, xsc, tw = dbuf[j]["x"], dbuf[j]["x_scale"], dbuf[j]["topk_weights"]
                outs[j].zero_()
                op(xin, xsc, wl.w, wl.w_scale, wl.w2, wl.w2_scale, dbuf[j]["sid"], dbuf[j]["eid"], dbuf[j]["npp"], tw,
                   outs[j], sh.top_k, bm, bn, wn, st, sh.scaling)
                if split:
                    dist.reduce_scatter_tensor(out_part[j], outs[j])
                elif world > 1:
                    dist.all_reduce(outs[j])
                ev_run[j].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[j])
                out_host[j].copy_(out_part[j], non_blocking=True)
                ev_out[j].record(s_out)

        def drain():
            for s_ in (s_in, s_run, s_out):
                main_stream.wait_stream(s_)

        for s_ in (s_in, s_run, s_out):
            s_.wait_stream(main_stream)
        for i in range(warmup):
            step(i)
        drain()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main_stream)
        for s_ in (s_in, s_run, s_out):
            s_.wait_event(e0)
        for i in range(steps):
            step(warmup + i)
        drain()
        e1.record(main_stream)
        barrier()
        launches[0] += steps
        (ms,) = max_over_ranks(e0.elapsed_time(e1) / steps)
        return ms, h2d, d2h, ("each rank copies 1/N of the rows, all-gather in, reduce-scatter out" if split else
                              "whole batch per rank")

    def tp_parity(wl, m, own_exchange=False):
        """Correctness record of a multi-GPU run: after one step the all-reduced `out` is compared on sampled token rows
        with (a) the fp32 sum of the ranks' partial outputs and (b) the CPU restatement of the operator, which every
        rank evaluates for its own shard on those rows (summed over ranks).  Returns (rel-L2 a, rel-L2 b)."""
        from oracle import moe_oracle as orc
        sh = wl.shape
        inp, d, out, call, (bm, _, _, _) = prepare(wl, m)
        ar = peer_all_reduce(sh.k) if (own_exchange and world > 1) else None
        if ar:
            out = ar.next_buffer(m)
        else:
            out.zero_()
        call(out)
        part = out.float()
        if ar:
            ar.all_reduce()
        elif world > 1:
            dist.all_reduce(out)
        torch.cuda.synchronize()
        rows = torch.randperm(m, generator=torch.Generator().manual_seed(5))[: min(m, 2)]
        rows_d = rows.to(dev)
        got = out[rows_d].float()
        shard_sum = part[rows_d].clone()
        if world > 1:
            dist.all_reduce(shard_sum)
        ids = inp["ids"][rows]
        experts = torch.unique(ids).tolist()
        remap = {e: i for i, e in enumerate(experts)}
        sub_ids = torch.tensor([[remap[int(e)] for e in r] for r in ids], dtype=torch.int32)
        idx = torch.tensor(experts, device=dev)
        wc = [t[idx].cpu() for t in (wl.w, wl.w_scale, wl.w2, wl.w2_scale)]
        ssid, seid, snpp = orc.moe_align_block_size(sub_ids, 16, len(experts))
        ref = orc.fused_moe_w8a8_up_down_oracle(inp["x"][rows_d].cpu(), inp["x_scale"][rows_d].cpu(), wc[0], wc[1], wc[2], wc[3],
                                                ssid, seid, snpp, inp["topk_weights"][rows].contiguous(), sh.top_k, 16,
                                                sh.scaling, out_fp32=True).to(dev)
        if world > 1:
            dist.all_reduce(ref)

        def rel(a, b):
            return float((a - b).norm() / b.norm().clamp_min(1e-30))
        return rel(got, shard_sum), rel(got, ref)

    def fractions(sh, m, inp, kern_ms):
        """Roofline figures of one launch: HBM bound on all algorithmic bytes, on the weight bytes alone, fp8 bound."""
        ab = sh.algorithmic_bytes(m, inp["e_active"], inp["sid"].numel())
        wb = inp["e_active"] * 3.0 * sh.inter * sh.k
        fl = sh.flops(m)
        t = kern_ms * 1e-3
        t_hbm, t_fp8 = ab / (peaks["hbm_gbs"] * 1e9), fl / (fp8_peak * 1e12)
        return {"abytes": ab, "wbytes": wb, "flops": fl, "t_hbm": t_hbm, "t_fp8": t_fp8,
                "frac_hbm": ab / t / 1e9 / peaks["hbm_gbs"], "frac_hbm_weights": wb / t / 1e9 / peaks["hbm_gbs"],
                "frac_fp8": fl / t / 1e12 / fp8_peak, "frac_binding": max(t_hbm, t_fp8) / t}

    def sweep_record(sh, m, s_ms, k_ms, inp, knobs, extra=None):
        f = fractions(sh, m, inp, k_ms)
        rec = {"M": m, "us_kernel": round(k_ms * 1e3, 1), "us_step": round(s_ms * 1e3, 1),
               "tflops_job": round(f["flops"] * world / (s_ms * 1e-3) / 1e12, 2), "e_active": inp["e_active"],
               "frac_hbm_weights": round(f["frac_hbm_weights"], 3), "frac_fp8": round(f["frac_fp8"], 3),
               "frac_binding_bound": round(f["frac_binding"], 3), "binding": "hbm" if f["t_hbm"] >= f["t_fp8"] else "fp8",
               "knobs": list(knobs)}
        if extra:
            rec.update(extra)
        return rec

    # ------------------------------------------------------------------ headline: DeepSeek-V3 TP8 shard per GPU
    sh = DEEPSEEK
    m = args.m
    wl = Workload(sh, dev, rank)
    sampler = ClockSampler(physical_gpu_index(local_rank)) if rank == 0 else None
    if sampler:
        sampler.start()
    step_ms, kern_ms, inp, knobs = time_steps(wl, m, args.steps, args.warmup)
    exchange, step_ms_nccl, step_ms_own, step_ms_rs = None, None, None, None
    if world > 1:
        # the exchange step of the headline: the NCCL all-reduce or this library's own kernel, whichever is faster here
        step_ms_nccl, exchange = step_ms, "NCCL all-reduce"
        if peer_all_reduce(sh.k) is not None:
            step_ms_own, kern_own, _, _ = time_steps(wl, m, args.steps, args.warmup, own_exchange=True)
            if step_ms_own < step_ms_nccl:
                step_ms, kern_ms, exchange = step_ms_own, kern_own, "own all-reduce kernel over peer-mapped buffers"
            if m % world == 0:      # for a consumer that takes row shards: the first half of the exchange only (not the headline)
                step_ms_rs = time_steps(wl, m, args.steps, args.warmup, own_exchange="reduce_scatter")[0]
    clocks = sampler.stop() if sampler else None
    e2e_ms, h2d, d2h, e2e_how = time_e2e(wl, m, args.steps, args.warmup)
    parity = tp_parity(wl, m, own_exchange=(exchange is not None and exchange.startswith("own"))) if world > 1 else None

    f = fractions(sh, m, inp, kern_ms)
    bound = "hbm" if f["t_hbm"] >= f["t_fp8"] else "tensor"
    if bound == "hbm":
        achieved, peak, unit = f["abytes"] / (kern_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = f["flops"] / (kern_ms * 1e-3) / 1e12, fp8_peak, "TFLOP/s"
    tr = traffic.get(("deepseek", m))

    sweep, qwen, zipf, tp_fixed, layer, imbalance = [], [], None, [], [], []
    if not args.no_sweep:
        for ms_ in SWEEP_MS:
            s_ms, k_ms, sinp, sk = time_steps(wl, ms_, 10, 3)
            extra = {"us_step_median": round(last_median[0] * 1e3, 1)}
            if ms_ <= GRAPH_MAX_M:
                extra["us_step_graph"] = round(time_graph_step(wl, ms_, 10) * 1e3, 1)
            if world > 1 and ms_ >= 256:
                if peer_all_reduce(sh.k) is not None:
                    extra["us_step_own_allreduce"] = round(time_steps(wl, ms_, 10, 3, own_exchange=True)[0] * 1e3, 1)
            if world > 1 and ms_ <= 64 and sk[0] <= 64:
                t_own = time_fused_tp(wl, ms_, 10, 3)
                if t_own is not None:
                    extra["us_step_own_exchange"] = round(t_own * 1e3, 1)
                    extra["us_step_own_exchange_graph"] = round(time_graph_step(wl, ms_, 10, own_exchange=True) * 1e3, 1)
                    t_train = time_fused_tp_train(wl, ms_)
                    if t_train is not None:
                        extra["us_step_own_exchange_graph8"] = round(t_train * 1e3, 1)
            sweep.append(sweep_record(sh, ms_, s_ms, k_ms, sinp, sk, extra))
        for ms_ in LAYER_MS:
            if world == 1:
                t_eager, t_graph = time_layer(wl, ms_, 6, 3)
                rec = {"M": ms_, "us_layer": round(t_eager * 1e3, 1)}
                if t_graph is not None:
                    rec["us_layer_graph"] = round(t_graph * 1e3, 1)
                layer.append(rec)
        if world == 1:
            s_ms, k_ms, sinp, sk = time_steps(wl, 8192, 6, 3, zipf=1.2)
            counts = torch.bincount(sinp["ids"].reshape(-1).long(), minlength=sh.e)[:-1]
            zipf = sweep_record(sh, 8192, s_ms, k_ms, sinp, sk,
                                {"routing": "Zipf(1.2) over 240 of the 256 routed experts, seed 1",
                                 "empty_experts": int((counts == 0).sum()), "max_share_of_tokens": round(float(counts.max()) / 8192, 3)})
            # the reference's own imbalance levels (its timing script sweeps balancedness 0.8 ... 0.5 at every M)
            for ms_ in (256, 4096):
                for bal in (0.8, 0.7, 0.6, 0.5):
                    s_ms, k_ms, sinp, sk = time_steps(wl, ms_, 5, 3, zipf=("balancedness", bal))
                    counts = torch.bincount(sinp["ids"].reshape(-1).long(), minlength=sh.e)[:-1]
                    imbalance.append(sweep_record(sh, ms_, s_ms, k_ms, sinp, sk,
                                                  {"balancedness": bal,
                                                   "share_of_routed_assignments_on_expert_0": round(float(counts[0]) / float(counts.sum()), 3)}))
            wq = Workload(QWEN3, dev, rank)
            for ms_ in QWEN_MS:
                s_ms, k_ms, sinp, sk = time_steps(wq, ms_, 6, 3)
                qwen.append(sweep_record(QWEN3, ms_, s_ms, k_ms, sinp, sk))
            del wq
        # the unsharded layer (I = 2048) split over the ranks: fixed total work, I / N per GPU + all-reduce
        if I_FULL % world == 0 and (I_FULL // world) % 256 == 0:
            tp_shape = Shape(f"DeepSeek-V3-like layer I={I_FULL} split over tp={world}", sh.e, sh.k, I_FULL // world, sh.top_k,
                             sh.scaling, True)
            del wl
            torch.cuda.empty_cache()
            wt = Workload(tp_shape, dev, rank)
            for ms_ in TP_FIXED_MS:
                s_ms, k_ms, sinp, sk = time_steps(wt, ms_, 6, 3)
                rec = sweep_record(tp_shape, ms_, s_ms, k_ms, sinp, sk, {"I_per_gpu": tp_shape.inter})
                if world > 1 and ms_ == 64:
                    pa = tp_parity(wt, ms_)
                    rec["tp_parity_rel_l2"], rec["tp_parity_vs_oracle"] = round(pa[0], 5), round(pa[1], 5)
                tp_fixed.append(rec)
            del wt
            torch.cuda.empty_cache()
            wl = Workload(sh, dev, rank)

    host_us = host_us_per_call(wl, 1) if (world == 1 and not args.no_sweep) else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        n_s = args.cpu_experts
        wl_cpu = {"w": wl.w[:n_s].cpu(), "w2": wl.w2[:n_s].cpu(), "w_scale": wl.w_scale[:n_s].cpu(),
                  "w2_scale": wl.w2_scale[:n_s].cpu()}
        inp["x_cpu"], inp["x_scale_cpu"] = inp["x"].cpu(), inp["x_scale"].cpu()
        threads = os.cpu_count() or 1
        tf, dt, n_assign = cpu_sample(sh, wl_cpu, inp, m, n_s, 8, threads)
        cpu = {"value": tf, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"assignments routed to the first {n_s} of {sh.e} experts at M={m} "
                         f"({n_assign} of {m * sh.top_k}), {dt:.2f} s per pass"}

    status = capi.read_status(reset=True)
    bad_parity = parity is not None and (parity[0] > 1e-2 or parity[1] > 2e-2)
    if rank == 0:
        line = {
            "metric": "fused_moe_layer_tflops", "value": f["flops"] * world / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (f32 accumulate)",
            "data": "synthetic", "config": workload_config(sh, m, world),
            "us_per_layer_kernel": kern_ms * 1e3,
            "knobs": {"block_m": knobs[0], "block_n": knobs[1], "warp_n": knobs[2], "stages": knobs[3]},
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                         "frac": achieved / peak, "traffic": tr["bytes"] if tr else None,
                         "traffic_source": (f"ncu capture of {tr['kernel']} at M={m}, profiles/fused_moe_dram_traffic.md"
                                            if tr else None),
                         "peak_source": peaks["source"], "fp8_peak_tflops": fp8_peak, "fp8_peak_note": fp8_note,
                         "algorithmic_bytes": f["abytes"], "weight_bytes": f["wbytes"],
                         "frac_hbm_weights_only": f["frac_hbm_weights"], "frac_fp8_tensor": f["frac_fp8"],
                         "t_hbm_us": f["t_hbm"] * 1e6, "t_fp8_us": f["t_fp8"] * 1e6},
            "e2e": {"value": f["flops"] * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "rows": e2e_how,
                    "pipeline": "copy-in / layer / copy-out of consecutive steps on three streams, two buffer sets"},
            "gpu_launches": launches[0], "host_us_per_call_m1": host_us,
            "clocks": clocks, "kernel_status": list(status), "sweep": sweep, "layer": layer, "zipf": zipf, "imbalance": imbalance,
            "qwen3": qwen, "tp_fixed": tp_fixed,
        }
        if parity is not None:
            line["tp_parity_rel_l2"], line["tp_parity_vs_oracle"] = round(parity[0], 5), round(parity[1], 5)
            line["exchange"] = {"used": exchange, "ms_per_step_nccl": step_ms_nccl, "ms_per_step_own_allreduce": step_ms_own,
                                "ms_per_step_own_reduce_scatter": step_ms_rs,
                                "reduce_scatter_note": "same step with the exchange stopped after every rank has summed its own "
                                                       "rows (a consumer that takes row shards); not the headline"}
            if own_notes:
                line["exchange"]["unavailable"] = own_notes
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    # a run-out wait inside a fused kernel (where < 90) or a parity miss fails the run; a run-out cross-GPU wait of the
    # own exchange kernels (where >= 90: a rank arrived more than the time limit late) is reported in kernel_status only
    if bad_parity or (status[0] != 0 and status[2] < 90):
        raise SystemExit(f"tensor-parallel parity {parity} or kernel status {status} out of bounds")


if __name__ == "__main__":
    main()
