#!/usr/bin/env python
"""Benchmark of the attention forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|triton_ref]
                    [--workload 3|2|4|5] [--strong] [--passes P]

A "pass" is one forward + backward of the workload through the public Python API (default:
the headline case B=8, H=16, M=N=2048, D=128, bf16, trainable float bias ~0.5*N(0,1),
non-causal).  A "step" is `passes` passes back to back (24 for the default workload), so that
the K timed steps of a default run cover about 0.7 s: long enough for the GPU to settle at the
clock its power cap allows, which a 30 ms region never shows.  Every step is also timed on its
own with CUDA events; the fastest step is reported as the burst figure.

With N > 1 (launched by torch.distributed.run, one rank per GPU):
  default    every rank runs a workload-sized shard of its own (weak scaling); (batch, head)
             problems are independent, so there is no data-path collective;
  --strong   the ONE global problem of the workload is partitioned over its (batch, head)
             grid: rank r owns sharding.shard_batch_heads(B, H, r, N).  Inputs are seeded per
             (batch, head), so every shard reproduces the 1-GPU tensors exactly.  After the timed
             region the shards are verified: sampled (b, h) problems against the fp32 oracle
             (all_reduce MAX of the errors), out/dq/dk/dv all_gathered and compared bitwise
             with an unsharded run on rank 0.  NCCL carries only that and the barriers.

Rank 0 prints one JSON line:
  value        fwd+bwd TFLOP/s over the K timed steps, inputs resident in HBM
  burst        the same for the fastest single step
  e2e          same metric with HOST (pinned) inputs and outputs: H2D of q,k,v,bias,do and D2H
               of out,dq,dk,dv,dbias inside the timed region
  roofline     dominant kernel (dK/dV) against the measured peaks; "kernels" lists all four, each
               timed alone through the C ABI in a short loop (full clock: held against the burst
               tensor peak) and in a long one (held against the sustained tensor peak)
  cpu_baseline fp32 eager oracle on the host cores, on a bounded sample of (b,h) problems
--impl reference times that CPU oracle alone (the reference project's CPU-runnable path is
exactly this fp32 eager math).  --impl triton_ref times the reference project's own Triton
kernels on the GPU, from the unmodified copy under baseline/_ref/ when it is there.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import re
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, H, M, N, D, dtype, bias kind, causal, bias scale; passes = passes per step
    "2": dict(B=4, H=16, M=1024, N=1024, D=64, dtype="bf16", bias=None, causal=True, bias_scale=0.0, passes=160),
    "3": dict(B=8, H=16, M=2048, N=2048, D=128, dtype="bf16", bias="float", causal=False, bias_scale=0.5, passes=24),
    "4": dict(B=4, H=32, M=4096, N=4096, D=128, dtype="bf16", bias="bool", causal=True, bias_scale=0.0, passes=12),
    "5": dict(B=8, H=32, M=8192, N=8192, D=128, dtype="bf16", bias="float", causal=True, bias_scale=0.5, passes=2),
    # not a benchmark configuration of the reference: the largest head dim its API accepts
    "d256": dict(B=4, H=8, M=2048, N=2048, D=256, dtype="bf16", bias="float", causal=False, bias_scale=0.5, passes=12),
}
WORKLOAD_NAMES = {
    "2": "config2: causal self-attention B4 H16 M=N=1024 D64 bf16, no bias",
    "3": "config3: B8 H16 M=N=2048 D128 bf16, trainable float bias (B,H,M,N), non-causal",
    "4": "config4: bool mask + causal B4 H32 S4096 D128 bf16",
    "5": "config5: B8 H32 M=N=8192 D128 bf16, trainable float bias, causal",
    "d256": "head dim 256: B4 H8 M=N=2048 D256 bf16, trainable float bias, non-causal",
}
# ncu summary of one dK/dV launch of the default workload at a reduced batch (traffic is
# proportional to the batch); parsed for dram__bytes_{read,write}.sum
DKDV_CAPTURE = os.path.join(ROOT, "profiles", "dkdv_kernel_config3_b2_ncu_full.md")
DKDV_CAPTURE_BATCH = 2
REF_PATH = os.path.join(ROOT, "baseline", "_ref", "flash_attention.py")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    tflops_burst=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, tflops_burst=1590.0, source="fallback")


def captured_dkdv_traffic():
    """DRAM bytes (read + written) of one dK/dV launch per batch element, from the committed ncu
    summary; None when the summary is missing or has no such rows."""
    try:
        text = open(DKDV_CAPTURE).read()
    except OSError:
        return None
    vals = {}
    for key in ("dram__bytes_read.sum", "dram__bytes_write.sum"):
        m = re.search(r"\|\s*" + re.escape(key) + r"\s*\|\s*(\w+)\s*\|\s*([0-9.]+)\s*\|", text)
        if not m:
            return None
        mult = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(m.group(1))
        if mult is None:
            return None
        vals[key] = float(m.group(2)) * mult
    return sum(vals.values()) / DKDV_CAPTURE_BATCH


def flops(w, which):
    c = 0.5 if w["causal"] else 1.0
    mult = {"fwd": 4, "bwd": 10, "fwd+bwd": 14, "dkdv": 8, "dq_recompute": 6, "dq_from_ds": 2}[which]
    return mult * w["B"] * w["H"] * w["M"] * w["N"] * w["D"] * c


def kernel_bytes(w, which):
    """Algorithmic (compulsory) HBM bytes of one launch of each kernel."""
    B, H, M, N, D = w["B"], w["H"], w["M"], w["N"], w["D"]
    e = 2
    b = {None: 0, "float": 2, "bool": 1}[w["bias"]]
    c = 0.5 if w["causal"] else 1.0
    bhmn = B * H * M * N
    qd, kd = B * M * H * D * e, B * N * H * D * e
    trainable = w["bias"] == "float"
    if which == "fwd":
        return 2 * qd + 2 * kd + bhmn * b * c + 4 * B * H * M
    if which == "pre":
        return 2 * qd + 4 * B * H * M
    if which == "dkdv":
        return 2 * qd + 4 * kd + bhmn * b * c + (bhmn * 2 if trainable else 0) + 8 * B * H * M
    if which == "dq":
        if trainable:  # streams dS (written as dbias) instead of the bias
            return qd + kd + bhmn * 2 * c
        return 3 * qd + 2 * kd + bhmn * b * c + 8 * B * H * M
    raise KeyError(which)


def make_inputs(w, device, seed):
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    B, H, M, N, D = w["B"], w["H"], w["M"], w["N"], w["D"]

    def rnd(*shape, scale=1.0):
        t = torch.empty(shape, dtype=dt, device=device)
        t.normal_(0.0, scale)
        return t

    torch.manual_seed(seed)
    torch.cuda.manual_seed(seed)
    q, k, v, do = rnd(B, M, H, D), rnd(B, N, H, D), rnd(B, N, H, D), rnd(B, M, H, D)
    bias = None
    if w["bias"] == "float":
        bias = rnd(B, H, M, N, scale=w["bias_scale"])
    elif w["bias"] == "bool":
        bias = torch.rand((B, H, M, N), device=device) < 0.9
        i = torch.arange(min(M, N), device=device)
        bias[:, :, i, i] = True
    return q, k, v, bias, do


def make_inputs_per_pair(w, device, seed, shard):
    """Inputs of the (batch, head) block `shard` of the global problem, drawn from one generator
    per (batch, head): any partition reproduces exactly the tensors of the unsharded problem."""
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    H, M, N, D = w["H"], w["M"], w["N"], w["D"]
    nb, nh = shard.b1 - shard.b0, shard.h1 - shard.h0
    q = torch.empty((nb, M, nh, D), dtype=dt, device=device)
    k = torch.empty((nb, N, nh, D), dtype=dt, device=device)
    v, do = torch.empty_like(k), torch.empty_like(q)
    bias = None
    if w["bias"] == "float":
        bias = torch.empty((nb, nh, M, N), dtype=dt, device=device)
    elif w["bias"] == "bool":
        bias = torch.empty((nb, nh, M, N), dtype=torch.bool, device=device)
    g = torch.Generator(device=device)
    diag = torch.arange(min(M, N), device=device)
    for b in range(shard.b0, shard.b1):
        for h in range(shard.h0, shard.h1):
            g.manual_seed(seed * 1000003 + b * H + h)
            ib, ih = b - shard.b0, h - shard.h0
            q[ib, :, ih] = torch.randn(M, D, generator=g, device=device).to(dt)
            k[ib, :, ih] = torch.randn(N, D, generator=g, device=device).to(dt)
            v[ib, :, ih] = torch.randn(N, D, generator=g, device=device).to(dt)
            do[ib, :, ih] = torch.randn(M, D, generator=g, device=device).to(dt)
            if w["bias"] == "float":
                bias[ib, ih] = (w["bias_scale"] * torch.randn(M, N, generator=g, device=device)).to(dt)
            elif w["bias"] == "bool":
                keep = torch.rand(M, N, generator=g, device=device) < 0.9
                keep[diag, diag] = True
                bias[ib, ih] = keep
    return q, k, v, bias, do


class ClockSampler:
    """SM clock and throttle reasons of one GPU, read in-process through NVML (queries only)
    by a thread every `period` seconds; only samples inside the marked region are used."""

    def __init__(self, device_index, period=0.05):
        self.period = period
        self.samples = []  # (t, sm_mhz, reasons bitmask)
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self.t0 = self.t1 = None
        self.h = None
        self.nv = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.h = None

    def _read(self):
        nv = self.nv
        sm = float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
        except Exception:
            reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
        return (time.perf_counter(), sm, reasons)

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._read())
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.h is None:
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def mark_begin(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def stop(self):
        if self.h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self._thread.join(timeout=2)
        nv = self.nv
        inside = [s for s in self.samples if self.t0 is not None and self.t0 <= s[0] <= self.t1]
        in_region = len(inside)
        if not inside:
            inside = self.samples[-2:]
        names = (("hw_slowdown", nv.nvmlClocksThrottleReasonHwSlowdown),
                 ("hw_thermal_slowdown", nv.nvmlClocksThrottleReasonHwThermalSlowdown),
                 ("sw_thermal_slowdown", nv.nvmlClocksThrottleReasonSwThermalSlowdown),
                 ("sw_power_cap", nv.nvmlClocksThrottleReasonSwPowerCap))
        reasons = sorted({n for s in inside for n, bit in names if s[2] & bit})
        sm = [s[1] for s in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_mhz_min": min(sm) if sm else None,
                "sm_max_mhz": self.sm_max, "samples": len(sm), "in_region": in_region, "reasons": reasons,
                "how": "NVML queries from a thread of this process, every 50 ms"}


def cuda_time_ms(fn, iters):
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def cpu_oracle_sample(w, slices, threads=None, repeats=1):
    """fp32 eager forward+backward of `slices` (b,h) problems of the workload on the host cores;
    returns the best wall-clock seconds for the sample."""
    from oracle import eager_oracle as oracle

    if threads:
        torch.set_num_threads(threads)
    M, N, D = w["M"], w["N"], w["D"]
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, M, slices, D, generator=g)
    k = torch.randn(1, N, slices, D, generator=g)
    v = torch.randn(1, N, slices, D, generator=g)
    do = torch.randn(1, M, slices, D, generator=g)
    bias = None
    if w["bias"] == "float":
        bias = w["bias_scale"] * torch.randn(1, slices, M, N, generator=g)
    elif w["bias"] == "bool":
        bias = torch.rand(1, slices, M, N, generator=g) < 0.9
        i = torch.arange(min(M, N))
        bias[:, :, i, i] = True
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.attention_autograd(q, k, v, bias, w["causal"], None, do)
        best = min(best, time.perf_counter() - t0)
    return best


def config_dict(w, wname, strong):
    return {"workload": wname, "passes_per_step": w["passes"],
            "partition": "one global problem split over (batch, head)" if strong else "per-GPU problem",
            "l2": "inputs larger than L2 (no flush needed)" if w["bias"] else "inputs smaller than L2, no flush"}


def run_reference(args, w, wname, rank):
    """--impl reference: the fp32 eager path on the host cores (rank 0 only).  One step is a
    bounded sample of the workload: `slices` of its B*H (batch, head) problems."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    slices = 2 if w["M"] * w["N"] >= 2048 * 2048 else min(8, w["B"] * w["H"])
    sample_flops = flops(w, "fwd+bwd") * slices / (w["B"] * w["H"])
    for _ in range(args.warmup):
        cpu_oracle_sample(w, slices)
    t0 = time.perf_counter()
    times = [cpu_oracle_sample(w, slices) for _ in range(args.steps)]
    timed_s = time.perf_counter() - t0
    sec = sum(times) / len(times)
    value = sample_flops / sec / 1e12
    sample = (f"each step = fp32 eager fwd+bwd of {slices} of the workload's {w['B'] * w['H']} (b,h) problems; "
              f"value = FLOPs of the sample / its time; the whole workload would take {sec * w['B'] * w['H'] / slices:.2f} s")
    line = {
        "impl": "reference", "metric": "fwd+bwd attention TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "timed_region_s": round(timed_s, 3), "higher_is_better": True,
        "scaling": "strong" if args.strong else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config_dict(w, wname, args.strong), "gpu_launches": 0,
        "note": "CPU arm: one copy on rank 0's host cores whatever --gpus says",
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def load_triton_reference():
    import importlib.util
    if not os.path.exists(REF_PATH):
        raise RuntimeError("baseline/_ref/flash_attention.py is not installed (baseline/install_ref.py)")
    spec = importlib.util.spec_from_file_location("reference_flash_attention", REF_PATH)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def percentile(xs, p):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, max(0, int(math.ceil(p * len(xs))) - 1))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "triton_ref"])
    ap.add_argument("--workload", default="3", choices=sorted(WORKLOADS))
    ap.add_argument("--strong", action="store_true",
                    help="N > 1: partition the ONE global problem over (batch, head) and verify the shards")
    ap.add_argument("--passes", type=int, default=0, help="forward+backward passes per step (0 = workload default)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size B (profiling on a small case)")
    ap.add_argument("--bias", default="", choices=["", "none", "float", "bool"],
                    help="override the bias kind of the workload (profiling)")
    ap.add_argument("--profile", action="store_true",
                    help="profiling run: exactly --warmup/--steps single passes of the public API, nothing else")
    args = ap.parse_args()
    if args.impl != "reference" and not args.profile:
        args.warmup = max(args.warmup, 3)
    if args.profile:
        args.no_e2e = args.no_cpu_baseline = args.no_kernels = True

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    w = dict(WORKLOADS[args.workload])
    wname = WORKLOAD_NAMES[args.workload]
    if args.bias:
        w["bias"] = None if args.bias == "none" else args.bias
        wname += f" [bias overridden to {args.bias}]"
    if args.batch:
        w["B"] = args.batch
        wname += f" [batch overridden to {args.batch}]"
    if args.passes:
        w["passes"] = args.passes
    if args.profile:
        w["passes"] = 1

    if args.impl == "reference":
        run_reference(args, w, wname, rank)
        return

    import torch.distributed as dist

    if world > 1:
        # one slice of the host cores per rank: eight Python main threads, eight autograd threads
        # and eight sampler threads otherwise wander over the same cores
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = max(1, len(cores) // world)
            os.sched_setaffinity(0, cores[local_rank * per:(local_rank + 1) * per] or cores)
        except (AttributeError, OSError):
            pass
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()

    strong = bool(args.strong and world > 1)
    w_local = dict(w)  # the problem this rank runs
    shard = None
    if strong:
        from triton_flashattn_b200.sharding import shard_batch_heads
        shard = shard_batch_heads(w["B"], w["H"], rank, world)
        w_local["B"], w_local["H"] = shard.b1 - shard.b0, shard.h1 - shard.h0
        q, k, v, bias, do = make_inputs_per_pair(w, device, int(args.workload), shard)
    else:
        q, k, v, bias, do = make_inputs(w, device, seed=3 + rank)
    trainable = w["bias"] == "float"

    if args.impl == "triton_ref":
        try:
            ref_mod = load_triton_reference()
            attn = ref_mod.flash_attention_fn
        except Exception as e:
            if rank == 0:
                print(json.dumps({"impl": "triton_ref", "unavailable": f"{type(e).__name__}: {e}"[:300]}), flush=True)
            return
        count_launches = lambda: 0
    else:
        from triton_flashattn_b200 import _cabi, flash_attention_fn as attn
        from triton_flashattn_b200 import flash_attention as fa_mod
        lib = _cabi.load()  # fails loudly if the extension is missing
        count_launches = lambda: int(lib.fa_launch_count())

    q.requires_grad_()
    k.requires_grad_()
    v.requires_grad_()
    if trainable:
        bias.requires_grad_()

    def one_pass():
        out = attn(q, k, v, bias, w["causal"], None)
        out.backward(do)
        q.grad = k.grad = v.grad = None
        if trainable:
            bias.grad = None

    def step():
        for _ in range(w["passes"]):
            one_pass()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    try:
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
    except Exception as e:
        if args.impl == "triton_ref":
            if rank == 0:
                print(json.dumps({"impl": "triton_ref", "unavailable": f"{type(e).__name__}: {e}"[:300]}), flush=True)
            return
        raise
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.06)
    barrier()
    launches0 = count_launches()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    sampler.mark_begin()
    ev[0].record()
    for i in range(args.steps):
        step()
        ev[i + 1].record()
    barrier()
    sampler.mark_end()
    launches = count_launches() - launches0
    ms = ev[0].elapsed_time(ev[-1]) / args.steps
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop()
    ranks = None
    best_step = min(per_step)
    if world > 1:
        # per-rank time and clock, so that a slow rank can be told from a slow program
        mine = torch.tensor([ms, clocks["sm_mhz"] or 0.0, float("sw_power_cap" in clocks["reasons"]),
                             float(any(r != "sw_power_cap" for r in clocks["reasons"])),
                             percentile(per_step, 0.5), percentile(per_step, 0.95), best_step,
                             clocks.get("sm_mhz_min") or 0.0], device=device, dtype=torch.float64)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        ranks = [{"ms": round(x[0].item(), 4), "sm_mhz": x[1].item(), "sm_mhz_min": x[7].item(),
                  "sw_power_cap": bool(x[2].item()), "other_slowdown": bool(x[3].item()),
                  "step_ms_p50": round(x[4].item(), 4), "step_ms_p95": round(x[5].item(), 4),
                  "step_ms_min": round(x[6].item(), 4)} for x in allr]
        ms = max(r["ms"] for r in ranks)
        best_step = max(r["step_ms_min"] for r in ranks)
    if args.impl == "ours":
        st = _cabi.device_status(local_rank)
        if st[0] != 0:
            raise RuntimeError(f"kernel abandoned a bounded wait: {st}")

    pass_flops = flops(w, "fwd+bwd") * (1 if strong else world)  # all ranks together, one pass
    value = pass_flops * w["passes"] / (ms * 1e-3) / 1e12
    burst = {"value": pass_flops * w["passes"] / (best_step * 1e-3) / 1e12, "unit": "TFLOP/s",
             "what": "fastest single step (max over ranks of each rank's fastest)"}

    # ---- --strong: verify the shards (outside the timed region)
    verification = None
    if strong and args.impl == "ours":
        verification = verify_shards(w, w_local, shard, q, k, v, bias, do, attn, device, rank, world,
                                     int(args.workload))

    # ---- per-kernel timing through the C ABI (rank 0 of an N=1 run explains `value`)
    kernels = {}
    roofline = None
    roof_sums = None
    if rank == 0 and args.impl == "ours" and not args.no_kernels:
        kernels, roofline, roof_sums = time_kernels(w_local, q, k, v, bias, do, trainable, peaks, fa_mod, _cabi,
                                                    args.workload == "3" and not args.bias)

    # ---- end to end: host (pinned) inputs and outputs inside the timed region
    e2e = None
    if not args.no_e2e and args.impl == "ours":
        e2e = time_e2e(w, q, k, v, bias, do, trainable, attn, device, args, barrier, world, pass_flops, dist)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.impl == "ours":
        slices = 16 if w["M"] * w["N"] <= 2048 * 2048 else 2
        cores = os.cpu_count() or 1
        sample_s = cpu_oracle_sample(w, slices, threads=cores, repeats=2)
        cpu_baseline = {"value": flops(w, "fwd+bwd") * slices / (w["B"] * w["H"]) / sample_s / 1e12,
                        "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                        "sample": f"fp32 eager fwd+bwd of {slices} of {w['B'] * w['H']} (b,h) problems "
                                  f"({sample_s:.2f} s); value = FLOPs of the sample / its time"}

    if rank == 0:
        line = {
            "metric": "fwd+bwd attention TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "timed_region_s": round(ms * args.steps * 1e-3, 4), "higher_is_better": True,
            "scaling": "strong" if strong else "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": config_dict(w, wname, strong),
            "step_ms": {"p50": round(percentile(per_step, 0.5), 4), "p95": round(percentile(per_step, 0.95), 4),
                        "min": round(min(per_step), 4), "max": round(max(per_step), 4), "of": "rank 0"},
            "ms_per_pass": ms / w["passes"], "burst": burst,
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
            "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu_baseline, "ranks": ranks,
            "frac_of_roofline_sum": roof_sums, "verification": verification,
        }
        if args.impl == "triton_ref":
            line["impl"] = "triton_ref"
            line["gpu_launches"] = None
            line["note"] = "the reference project's own Triton kernels (unmodified copy) on this GPU"
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def verify_shards(w, w_local, shard, q, k, v, bias, do, attn, device, rank, world, seed):
    """Shard against oracle on sampled (b, h) problems; all_gather of out/dq/dk/dv and bitwise
    comparison with an unsharded run on rank 0 (when the whole problem fits there)."""
    import torch.distributed as dist
    from oracle import eager_oracle as oracle
    from triton_flashattn_b200.sharding import shard_batch_heads, BHShard

    trainable = w["bias"] == "float"
    out = attn(q, k, v, bias, w["causal"], None)
    out.backward(do)
    res = {"out": out.detach(), "dq": q.grad, "dk": k.grad, "dv": v.grad}
    if trainable:
        res["dbias"] = bias.grad
    nb, nh = w_local["B"], w_local["H"]
    picks = sorted({(0, 0), (nb - 1, nh - 1), (nb // 2, nh // 3)})
    errs = {}
    with torch.no_grad():
        for ib, ih in picks:
            sl = lambda t: t[ib:ib + 1, :, ih:ih + 1]
            bb = None if bias is None else bias.detach()[ib:ib + 1, ih:ih + 1]
            ref = oracle.attention_backward(sl(q.detach()), sl(k.detach()), sl(v.detach()), bb, w["causal"], None,
                                            sl(do))
            for n, t in res.items():
                mine = t[ib:ib + 1, ih:ih + 1] if n == "dbias" else sl(t)
                r = ref[n].float()
                d = (mine.float() - r).abs()
                # raw max-abs, and the part of it not explained by the 16-bit rounding of the value
                errs[n] = max(errs.get(n, (0.0, 0.0)), (d.max().item(), (d - 2.0 ** -7 * r.abs()).max().item()))
            del ref
    names = sorted(errs)
    t = torch.tensor([[errs[n][0], errs[n][1]] for n in names], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_err = {n: {"raw": t[i, 0].item(), "beyond_rounding": t[i, 1].item()} for i, n in enumerate(names)}

    # gather out/dq/dk/dv (dbias stays local: it is as large as the bias)
    gathered = {}
    for n in ("out", "dq", "dk", "dv"):
        parts = [torch.empty_like(res[n].contiguous()) for _ in range(world)]
        dist.all_gather(parts, res[n].contiguous())
        gathered[n] = parts
    bitwise = None
    need_gb = (w["B"] * w["H"] * w["M"] * w["N"] * (2.0 if trainable else 1.0) * 2.2) / 1e9 * (1 + 1.0 / world)
    if rank == 0:
        if need_gb < 150:
            full = BHShard(0, w["B"], 0, w["H"])
            del res, out
            fq, fk, fv, fb, fdo = make_inputs_per_pair(w, device, seed, full)
            fq.requires_grad_(), fk.requires_grad_(), fv.requires_grad_()
            if trainable:
                fb.requires_grad_()
            fo = attn(fq, fk, fv, fb, w["causal"], None)
            fo.backward(fdo)
            whole = {"out": fo.detach(), "dq": fq.grad, "dk": fk.grad, "dv": fv.grad}
            bitwise = {}
            for n, parts in gathered.items():
                ok = True
                for r, part in enumerate(parts):
                    s = shard_batch_heads(w["B"], w["H"], r, world)
                    ok = ok and torch.equal(s.slice_bshd(whole[n]), part)
                bitwise[n] = ok
            if trainable:
                s0 = shard_batch_heads(w["B"], w["H"], 0, world)
                bitwise["dbias(rank 0's shard)"] = torch.equal(s0.slice_bhmn(fb.grad), bias.grad)
        else:
            bitwise = f"skipped: the unsharded problem needs ~{need_gb:.0f} GB on one GPU"
    checks = {n: [float(p.float().sum().item()) for p in parts] for n, parts in gathered.items()}
    return {"max_abs_err_vs_fp32_oracle": max_err, "sampled_pairs_per_rank": len(picks),
            "gathered_equal_unsharded_bitwise": bitwise, "shard_checksums": checks}


def time_kernels(w, q, k, v, bias, do, trainable, peaks, fa_mod, _cabi, use_capture):
    """Each kernel alone through the C ABI: a short loop (20 launches, full clock; tensor side
    held against the burst peak) and a long one (>= 0.4 s; held against the sustained peak)."""
    kernels = {}
    with torch.no_grad():
        scale = w["D"] ** -0.5
        o, lse = fa_mod._flash_attn_fwd(q, k, v, bias, w["causal"], scale)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dbias = fa_mod._empty_dbias(bias, q.dtype) if trainable else None
        delta = torch.empty_like(lse)
        bias_t, kind = fa_mod._classify_bias(bias.detach() if bias is not None else None, q)
        p = fa_mod._params(q, k, v, o, lse, bias_t, kind, w["causal"], scale)
        p.d_o, p.do_stride = do.data_ptr(), fa_mod._stride3(do)
        p.dq, p.dq_stride = dq.data_ptr(), fa_mod._stride3(dq)
        p.dk, p.dk_stride = dk.data_ptr(), fa_mod._stride3(dk)
        p.dv, p.dv_stride = dv.data_ptr(), fa_mod._stride3(dv)
        p.delta = delta.data_ptr()
        if dbias is not None:
            p.write_dbias = 1
            p.dbias, p.dbias_stride = dbias.data_ptr(), fa_mod._stride3(dbias)
        lib = _cabi.load()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        dq_kind = "dq_from_ds" if trainable else "dq_recompute"
        hbm = peaks["hbm_gbs"] * 1e9
        for name, fn, fl in (("fwd", lib.fa_fwd, flops(w, "fwd")), ("pre", lib.fa_bwd_pre, 0.0),
                             ("dkdv", lib.fa_bwd_dkdv, flops(w, "dkdv")),
                             ("dq", lib.fa_bwd_dq, flops(w, dq_kind))):
            call = lambda fn=fn: _cabi.check(fn(ctypes.byref(p), stream), name)
            for _ in range(3):
                call()
            nbytes = kernel_bytes(w, name)
            # a pause first: right after a long loop the GPU still sits at the clock its power
            # cap forced, and a "short loop" number taken then is not a full-clock number
            torch.cuda.synchronize()
            time.sleep(1.0)
            call()
            t_burst = cuda_time_ms(call, 20)
            t_long = cuda_time_ms(call, max(20, int(400.0 / max(t_burst, 1e-3))))
            roof_b = max(fl / (peaks["tflops_burst"] * 1e12), nbytes / hbm) * 1e3
            roof_s = max(fl / (peaks["tflops"] * 1e12), nbytes / hbm) * 1e3
            kernels[name] = {
                "ms": round(t_burst, 4), "tflops": round(fl / t_burst / 1e9, 1), "gbs": round(nbytes / t_burst / 1e6, 1),
                "roof_ms": round(roof_b, 4), "frac": round(roof_b / t_burst, 3),
                "long": {"ms": round(t_long, 4), "tflops": round(fl / t_long / 1e9, 1),
                         "gbs": round(nbytes / t_long / 1e6, 1), "roof_ms": round(roof_s, 4),
                         "frac": round(roof_s / t_long, 3)}}
        kd = kernels["dkdv"]
        fl, nbytes = flops(w, "dkdv"), kernel_bytes(w, "dkdv")
        tensor_bound = fl / (peaks["tflops"] * 1e12) >= nbytes / hbm
        # the dominant kernel in the long loop (the regime of `value`), against the sustained peaks
        if tensor_bound:
            roofline = {"kernel": "dkdv_kernel", "bound": "tensor", "achieved": kd["long"]["tflops"],
                        "peak": peaks["tflops"], "unit": "TFLOP/s",
                        "frac": round(kd["long"]["tflops"] / peaks["tflops"], 3),
                        "peak_source": peaks["source"] + " sustained bf16"}
        else:
            roofline = {"kernel": "dkdv_kernel", "bound": "hbm", "achieved": kd["long"]["gbs"],
                        "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": round(kd["long"]["gbs"] / peaks["hbm_gbs"], 3), "peak_source": peaks["source"]}
        roofline["burst"] = {"achieved_tflops": kd["tflops"], "achieved_gbs": kd["gbs"], "frac": kd["frac"]}
        roofline["traffic"] = None
        per_batch = captured_dkdv_traffic() if use_capture else None
        if per_batch is not None:
            roofline["traffic"] = int(per_batch * w["B"])
            roofline["traffic_source"] = (f"{os.path.relpath(DKDV_CAPTURE, ROOT)}: one launch at B={DKDV_CAPTURE_BATCH}, "
                                          f"scaled by B (traffic is proportional to the batch)")
        sums = {
            "burst": round(sum(x["roof_ms"] for x in kernels.values()) / sum(x["ms"] for x in kernels.values()), 3),
            "sustained": round(sum(x["long"]["roof_ms"] for x in kernels.values()) /
                               sum(x["long"]["ms"] for x in kernels.values()), 3)}
        roofline["sum_roof_over_sum_measured"] = sums["sustained"]
    return kernels, roofline, sums


def time_e2e(w, q, k, v, bias, do, trainable, attn, device, args, barrier, world, pass_flops, dist):
    hq, hk, hv, hdo = (t.detach().to("cpu").pin_memory() for t in (q, k, v, do))
    hb = bias.detach().to("cpu").pin_memory() if bias is not None else None
    pinned_like = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    ho = pinned_like(hq)
    hdq, hdk, hdv = pinned_like(hq), pinned_like(hk), pinned_like(hv)
    hdb = pinned_like(hb) if trainable else None
    nbytes = lambda t: t.numel() * t.element_size()
    h2d = sum(nbytes(t) for t in (hq, hk, hv, hdo)) + (nbytes(hb) if hb is not None else 0)
    d2h = sum(nbytes(t) for t in (ho, hdq, hdk, hdv)) + (nbytes(hdb) if hdb is not None else 0)

    # Three streams: copies in, compute (the public API call), copies out.  Device inputs are
    # double-buffered, so the H2D copy of pass i+1 and the D2H copy of pass i run while pass
    # i / i+1 computes; every pass still copies all of its inputs in and all of its results out.
    main_s = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    slots = []
    for _ in range(2):
        d = {"q": torch.empty_like(q).requires_grad_(), "k": torch.empty_like(k).requires_grad_(),
             "v": torch.empty_like(v).requires_grad_(), "do": torch.empty_like(do),
             "b": None, "in": torch.cuda.Event(), "done": torch.cuda.Event()}
        if hb is not None:
            d["b"] = torch.empty_like(bias.detach())
            if trainable:
                d["b"].requires_grad_()
        d["done"].record(main_s)
        slots.append(d)

    def e2e_pass(i):
        d = slots[i & 1]
        with torch.cuda.stream(s_in), torch.no_grad():
            s_in.wait_event(d["done"])  # the pass that last used this slot has finished
            d["q"].copy_(hq, non_blocking=True)
            d["k"].copy_(hk, non_blocking=True)
            d["v"].copy_(hv, non_blocking=True)
            d["do"].copy_(hdo, non_blocking=True)
            if hb is not None:
                d["b"].copy_(hb, non_blocking=True)
            d["in"].record(s_in)
        main_s.wait_event(d["in"])
        out = attn(d["q"], d["k"], d["v"], d["b"], w["causal"], None)
        out.backward(d["do"])
        d["done"].record(main_s)
        res = [out.detach(), d["q"].grad, d["k"].grad, d["v"].grad]
        dst = [ho, hdq, hdk, hdv]
        if trainable:
            res.append(d["b"].grad)
            dst.append(hdb)
            d["b"].grad = None
        d["q"].grad = d["k"].grad = d["v"].grad = None
        with torch.cuda.stream(s_out):
            s_out.wait_event(d["done"])
            for src, h in zip(res, dst):
                src.record_stream(s_out)
                h.copy_(src, non_blocking=True)

    def drain():
        main_s.wait_stream(s_in)
        main_s.wait_stream(s_out)

    n = max(2, min(args.steps, 8))
    e2e_pass(0)
    e2e_pass(1)
    drain()
    barrier()
    s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s2.record()
    for i in range(n):
        e2e_pass(i)
    drain()
    e2.record()
    barrier()
    ms2 = s2.elapsed_time(e2) / n
    if world > 1:
        t = torch.tensor([ms2], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms2 = t.item()
    return {"value": pass_flops / (ms2 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_pass": ms2,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "passes": n,
            "what": "one pass per e2e step: every pass copies all inputs in and all results out",
            "pipeline": "3 streams, double-buffered device inputs: H2D of pass i+1 and D2H of pass i "
                        "overlap compute; the drain of the last copies is inside the timed region"}


if __name__ == "__main__":
    main()
