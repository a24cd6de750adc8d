#!/usr/bin/env python
"""Benchmark of the attention forward+backward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload 3|2|4|5]

One "step" is one forward + backward of the workload (default: the headline case
B=8, H=16, M=N=2048, D=128, bf16, trainable float bias ~0.5*N(0,1), non-causal) on
every rank.  With N > 1 (launched by torch.distributed.run) every rank runs its own
shard of that size -- (batch, head) problems are independent, there is no data-path
collective -- and the value is total FLOPs over the slowest rank's time.

Rank 0 prints one JSON line:
  value        fwd+bwd TFLOP/s, inputs resident in HBM, through the public Python API
  e2e          same metric with HOST (pinned) inputs and outputs: H2D of q,k,v,bias,do
               and D2H of out,dq,dk,dv,dbias inside the timed region
  roofline     dominant kernel (dK/dV), timed alone with CUDA events through the C ABI, against
               the measured peaks (burst tensor peak for such a short loop); "kernels" lists all four
  cpu_baseline fp32 eager oracle on the host cores, on a bounded sample of (b,h) slices
--impl reference times that CPU oracle alone (the reference project's own CPU-runnable
path is exactly this fp32 eager math; its Triton kernels need a GPU and the project
files do not travel to the benchmark box).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, H, M, N, D, dtype, bias kind, causal, bias scale, packed
    "2": dict(B=4, H=16, M=1024, N=1024, D=64, dtype="bf16", bias=None, causal=True, bias_scale=0.0),
    "3": dict(B=8, H=16, M=2048, N=2048, D=128, dtype="bf16", bias="float", causal=False, bias_scale=0.5),
    "4": dict(B=4, H=32, M=4096, N=4096, D=128, dtype="bf16", bias="bool", causal=True, bias_scale=0.0),
    "5": dict(B=8, H=32, M=8192, N=8192, D=128, dtype="bf16", bias="float", causal=True, bias_scale=0.5),
}
WORKLOAD_NAMES = {
    "2": "config2: causal self-attention B4 H16 M=N=1024 D64 bf16, no bias",
    "3": "config3: B8 H16 M=N=2048 D128 bf16, trainable float bias (B,H,M,N), non-causal",
    "4": "config4: bool mask + causal B4 H32 S4096 D128 bf16",
    "5": "config5: B8 H32 M=N=8192 D128 bf16, trainable float bias, causal",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    tflops_burst=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, tflops_burst=1590.0, source="fallback")


# dram__bytes_read.sum + dram__bytes_write.sum of one dkdv_kernel launch of config 3 at B=2,
# divided by 2 (ncu capture summarised in profiles/dkdv_kernel_config3_b2_ncu_full.md)
DKDV_DRAM_BYTES_PER_BATCH_CONFIG3 = (340.52e6 + 260.69e6) / 2


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


def make_inputs(w, device, seed, pin=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    dt = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    B, H, M, N, D = w["B"], w["H"], w["M"], w["N"], w["D"]

    def rnd(*shape, scale=1.0):
        # generated on the device in chunks (seeded), then optionally copied to pinned host
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


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 20 ms.  Only samples whose
    time stamp falls inside the marked region (the timed steps) are used; if the region was too
    short to catch one, the nearest samples are used instead and `in_region` says 0."""

    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.first = ""
        self.t0 = self.t1 = None

    def start(self):
        """Starts the sampler and waits (at most 10 s) for its first line, so that the start-up
        of nvidia-smi (driver initialisation on every GPU of the machine) is over before the
        timed region begins and only the cheap periodic queries fall into it."""
        import select
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            if select.select([self.proc.stdout], [], [], 10.0)[0]:
                self.first = self.proc.stdout.readline()
        except OSError:
            self.proc = None

    def mark_begin(self):
        import datetime
        self.t0 = datetime.datetime.now()

    def mark_end(self):
        import datetime
        self.t1 = datetime.datetime.now()

    def stop(self):
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = []
        for line in (self.first + out).strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
                rows.append((ts, float(f[1]), float(f[2]), f[5:9]))
            except ValueError:
                continue
        inside = rows
        if self.t0 is not None and self.t1 is not None:
            pad = datetime.timedelta(milliseconds=10)
            inside = [r for r in rows if self.t0 - pad <= r[0] <= self.t1 + pad]
        in_region = len(inside)
        if not inside and rows and self.t0 is not None:
            mid = self.t0 + (self.t1 - self.t0) / 2
            inside = sorted(rows, key=lambda r: abs((r[0] - mid).total_seconds()))[:2]
        sm = [r[1] for r in inside]
        smax = [r[2] for r in inside]
        reasons = set()
        for r in inside:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 r[3]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "in_region": in_region, "reasons": sorted(reasons)}


def cuda_time_ms(fn, iters, stream_sync=True):
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
    """fp32 eager forward+backward of `slices` (b,h) problems of the workload on the host
    cores; returns (seconds for the sample, seconds extrapolated to the whole workload)."""
    from oracle import eager_oracle as oracle

    if threads:
        torch.set_num_threads(threads)
    B, H, M, N, D = w["B"], w["H"], w["M"], w["N"], w["D"]
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
    return best, best * (B * H) / slices


def run_reference(args, w, wname, rank, world):
    """--impl reference: the fp32 eager path on the host cores (rank 0 only)."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    slices = 2 if w["M"] * w["N"] >= 2048 * 2048 else min(8, w["B"] * w["H"])
    for _ in range(args.warmup):
        cpu_oracle_sample(w, slices)
    times = [cpu_oracle_sample(w, slices)[1] for _ in range(args.steps)]
    sec = sum(times) / len(times)
    # every rank of a weak-scaled job would do the same work; the CPU arm runs one copy
    value = flops(w, "fwd+bwd") / sec / 1e12
    line = {
        "impl": "reference", "metric": "fwd+bwd attention TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": wname},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{slices} of {w['B'] * w['H']} (b,h) slices per step, scaled by B*H/{slices}"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="3", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size B (profiling on a small case)")
    ap.add_argument("--bias", default="", choices=["", "none", "float", "bool"],
                    help="override the bias kind of the workload (profiling)")
    ap.add_argument("--profile", action="store_true",
                    help="profiling run: exactly --warmup/--steps steps of the public API, nothing else")
    args = ap.parse_args()
    if args.impl == "ours" and not args.profile:
        args.warmup = max(args.warmup, 3)
    if args.profile:
        args.no_e2e = args.no_cpu_baseline = True

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

    if args.impl == "reference":
        run_reference(args, w, wname, rank, world)
        return

    import torch.distributed as dist
    from triton_flashattn_b200 import _cabi, flash_attention_fn
    from triton_flashattn_b200 import flash_attention as fa_mod

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = load_peaks()
    _cabi.load()  # fail loudly if the extension is missing

    q, k, v, bias, do = make_inputs(w, device, seed=3 + rank)
    trainable = w["bias"] == "float"
    q.requires_grad_()
    k.requires_grad_()
    v.requires_grad_()
    if trainable:
        bias.requires_grad_()

    def step():
        out = flash_attention_fn(q, k, v, bias, w["causal"], None)
        out.backward(do)
        q.grad = k.grad = v.grad = None
        if trainable:
            bias.grad = None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()  # every rank watches its own GPU
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    sampler.mark_begin()
    start.record()
    for _ in range(args.steps):
        step()
    end.record()
    barrier()
    sampler.mark_end()
    ms = start.elapsed_time(end) / args.steps
    clocks = sampler.stop()
    ranks = None
    if world > 1:
        # per-rank time and clock, so that a slow rank can be told from a slow program
        mine = torch.tensor([ms, clocks["sm_mhz"] or 0.0, float("sw_power_cap" in clocks["reasons"]),
                             float(any(r != "sw_power_cap" for r in clocks["reasons"]))], device=device)
        allr = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        ranks = [{"ms": round(x[0].item(), 4), "sm_mhz": x[1].item(), "sw_power_cap": bool(x[2].item()),
                  "other_slowdown": bool(x[3].item())} for x in allr]
        ms = max(r["ms"] for r in ranks)
    st = _cabi.device_status(local_rank)
    if st[0] != 0:
        raise RuntimeError(f"kernel abandoned a bounded wait: {st}")

    total_flops = flops(w, "fwd+bwd") * world
    value = total_flops / (ms * 1e-3) / 1e12

    # ---- per-kernel timing through the C ABI (rank 0 of an N=1 run explains `value`)
    kernels = {}
    roofline = None
    if rank == 0 and not args.profile:
        with torch.no_grad():
            o, lse = fa_mod._flash_attn_fwd(q, k, v, bias, w["causal"], w["D"] ** -0.5)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            dbias = fa_mod._empty_dbias(bias, q.dtype) if trainable else None
            delta = torch.empty_like(lse)
            bias_t, kind = fa_mod._classify_bias(bias.detach() if bias is not None else None, q)
            p = fa_mod._params(q, k, v, o, lse, bias_t, kind, w["causal"], w["D"] ** -0.5)
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
            iters = max(5, args.steps)
            dq_kind = "dq_from_ds" if trainable else "dq_recompute"
            for name, fn, fl in (("fwd", lib.fa_fwd, flops(w, "fwd")), ("pre", lib.fa_bwd_pre, 0.0),
                                 ("dkdv", lib.fa_bwd_dkdv, flops(w, "dkdv")),
                                 ("dq", lib.fa_bwd_dq, flops(w, dq_kind))):
                call = lambda fn=fn: _cabi.check(fn(ctypes.byref(p), stream), name)
                for _ in range(3):
                    call()
                t_ms = cuda_time_ms(call, iters)
                nbytes = kernel_bytes(w, name)
                # a kernel timed alone for a fraction of a second runs at the full SM clock: it is
                # held against the burst tensor peak; only a loop long enough to reach the power
                # cap is held against the sustained one
                regime = "burst" if iters * t_ms < 250.0 else "sustained"
                tpeak = peaks["tflops_burst"] if regime == "burst" else peaks["tflops"]
                t_roof = max(fl / (tpeak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e3
                kernels[name] = {"ms": round(t_ms, 4), "tflops": round(fl / t_ms / 1e9, 1),
                                 "gbs": round(nbytes / t_ms / 1e6, 1), "roof_ms": round(t_roof, 4),
                                 "frac": round(t_roof / t_ms, 3), "tensor_peak": regime}
            kd = kernels["dkdv"]
            tpeak = peaks["tflops_burst"] if kd["tensor_peak"] == "burst" else peaks["tflops"]
            tensor_bound = flops(w, "dkdv") / (tpeak * 1e12) >= kernel_bytes(w, "dkdv") / (peaks["hbm_gbs"] * 1e9)
            if tensor_bound:
                roofline = {"kernel": "dkdv_kernel", "bound": "tensor", "achieved": kd["tflops"],
                            "peak": tpeak, "unit": "TFLOP/s", "frac": round(kd["tflops"] / tpeak, 3),
                            "traffic": None,
                            "peak_source": peaks["source"] + " " + kd["tensor_peak"] + " bf16"}
            else:
                roofline = {"kernel": "dkdv_kernel", "bound": "hbm", "achieved": kd["gbs"],
                            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(kd["gbs"] / peaks["hbm_gbs"], 3),
                            "traffic": None, "peak_source": peaks["source"]}
            # DRAM traffic of one dK/dV launch: from the ncu capture of this workload at B=2
            # (profiles/dkdv_kernel_config3_b2_ncu_full.md: 340.5 MB read + 260.7 MB written);
            # the kernel's traffic is proportional to B
            if args.workload == "3" and not args.bias:
                roofline["traffic"] = int(DKDV_DRAM_BYTES_PER_BATCH_CONFIG3 * w["B"])
            roofline["sum_roof_over_sum_measured"] = round(
                sum(x["roof_ms"] for x in kernels.values()) / sum(x["ms"] for x in kernels.values()), 3)
            del o, lse, dq, dk, dv, dbias, delta

    # ---- end to end: host (pinned) inputs and outputs inside the timed region
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hdo = (t.detach().to("cpu").pin_memory() for t in (q, k, v, do))
        hb = bias.detach().to("cpu").pin_memory() if bias is not None else None
        pinned_like = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        ho = pinned_like(hq)
        hdq, hdk, hdv = pinned_like(hq), pinned_like(hk), pinned_like(hv)
        hdb = pinned_like(hb) if trainable else None
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo)) + (hb.numel() * hb.element_size() if hb is not None else 0)
        d2h = sum(t.numel() * t.element_size() for t in (ho, hdq, hdk, hdv)) + (hdb.numel() * hdb.element_size() if hdb is not None else 0)

        # Three streams: copies in, compute (the public API call), copies out.  Device inputs are
        # double-buffered, so the H2D copy of step i+1 and the D2H copy of step i run while step
        # i / i+1 computes; every step still copies all of its inputs in and all of its results out.
        main = torch.cuda.current_stream(device)
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        slots = []
        for _ in range(2):
            d = {"q": torch.empty_like(q).requires_grad_(), "k": torch.empty_like(k).requires_grad_(),
                 "v": torch.empty_like(v).requires_grad_(), "do": torch.empty_like(do),
                 "b": None, "in": torch.cuda.Event(), "done": torch.cuda.Event(), "keep": None}
            if hb is not None:
                d["b"] = torch.empty_like(bias.detach())
                if trainable:
                    d["b"].requires_grad_()
            d["done"].record(main)
            slots.append(d)

        def e2e_step(i):
            d = slots[i & 1]
            with torch.cuda.stream(s_in), torch.no_grad():
                s_in.wait_event(d["done"])  # the step that last used this slot has finished
                d["q"].copy_(hq, non_blocking=True)
                d["k"].copy_(hk, non_blocking=True)
                d["v"].copy_(hv, non_blocking=True)
                d["do"].copy_(hdo, non_blocking=True)
                if hb is not None:
                    d["b"].copy_(hb, non_blocking=True)
                d["in"].record(s_in)
            main.wait_event(d["in"])
            out = flash_attention_fn(d["q"], d["k"], d["v"], d["b"], w["causal"], None)
            out.backward(d["do"])
            d["done"].record(main)
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

        def e2e_drain():
            main.wait_stream(s_in)
            main.wait_stream(s_out)

        e2e_steps = max(2, min(args.steps, 8))
        e2e_step(0)
        e2e_step(1)
        e2e_drain()
        barrier()
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for i in range(e2e_steps):
            e2e_step(i)
        e2e_drain()
        e2.record()
        barrier()
        ms2 = s2.elapsed_time(e2) / e2e_steps
        if world > 1:
            t = torch.tensor([ms2], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms2 = t.item()
        e2e = {"value": total_flops / (ms2 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms2,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
               "pipeline": "3 streams, double-buffered device inputs: H2D of step i+1 and D2H of step i "
                           "overlap compute; the drain of the last copies is inside the timed region"}
        del slots

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        slices = 16 if w["M"] * w["N"] <= 2048 * 2048 else 2
        cores = os.cpu_count() or 1
        sample_s, full_s = cpu_oracle_sample(w, slices, threads=cores, repeats=2)
        cpu_baseline = {"value": flops(w, "fwd+bwd") / full_s / 1e12, "unit": "TFLOP/s",
                        "cores": torch.get_num_threads(), "kind": "port",
                        "sample": f"fp32 eager fwd+bwd of {slices} of {w['B'] * w['H']} (b,h) slices "
                                  f"({sample_s:.2f} s), extrapolated by B*H/{slices}"}

    if rank == 0:
        line = {
            "metric": "fwd+bwd attention TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": wname, "per_gpu": True, "l2": "inputs larger than L2 (no flush needed)"
                       if w["bias"] else "inputs smaller than L2, no flush"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": 4 * args.steps,
            "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu_baseline, "ranks": ranks,
            "frac_of_roofline_sum": roofline["sum_roof_over_sum_measured"] if roofline else None,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
