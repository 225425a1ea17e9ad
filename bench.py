#!/usr/bin/env python
"""Benchmark of the scan hot path: forward + backward over one batch of synthetic input.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--algo auto]
    python bench.py --impl reference ...      # the reference's CPU loop on the host cores

One JSON line on stdout (rank 0).  A *step* is one forward scan plus one backward scan of the
workload; ``value`` is elements (batch*seq*d_model, summed over ranks) per second with all
tensors resident in HBM, ``e2e`` the same through ``scan_cu`` + ``.backward`` from pinned host
buffers with the copies inside the timed region.  With N > 1 every rank owns a full-size channel
shard of a d_model*N problem (weak scaling, no collective on the data path).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# DRAM bytes (read + write) per launch of the backward kernel from the committed ncu capture
# (profiles/lookback_c2_ncu_full.md); only known for the workload that was captured
NCU_TRAFFIC = {("c2", "lookback"): 127.9e6}

METRIC = "scan fwd+bwd elems/s"
UNIT = "elems/s"
L2_BYTES = 126 * 1024 * 1024


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=200)
    p.add_argument("--warmup", type=int, default=20)
    p.add_argument("--impl", default="b200", choices=["b200", "reference"])
    p.add_argument("--workload", default="c2")
    p.add_argument("--algo", default="auto", choices=["auto", "chunked", "lookback"])
    p.add_argument("--shape", default=None, help="override batch,seq,d_model of the workload (same gates and dtype)")
    p.add_argument("--mode", default="shard", choices=["shard", "seqpar", "gated"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-graphs", action="store_true", help="launch every step from Python instead of replaying CUDA graphs")
    p.add_argument("--no-cpu", action="store_true")
    p.add_argument("--no-soak", action="store_true", help="skip the extra steps that only feed the clock sampler")
    p.add_argument("--cpu-seconds", type=float, default=12.0)
    return p.parse_args()


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------ CPU legs
def cpu_reference_leg(w, seconds: float, threads: int):
    """The reference's own C++ loop (oracle/_ref) on the host cores, else the C restatement.
    Returns (elems_per_s, kind, cores, sample_text)."""
    import numpy as np
    import torch
    from oracle import oracle
    from fast_sequential_scan_b200.workloads import make_inputs

    a, b, g = (x.float().numpy() for x in make_inputs(w, "cpu", 0))
    job = None
    if oracle.RefLib.available():
        job = oracle.RefLib().job(w.batch, w.seq, w.d_model)
    reps, t_total = 0, 0.0
    if job is not None:
        threads = max(1, min(threads, w.batch))
        job.set(job.ALPHA, a); job.set(job.BETA, b); job.set(job.G, g)
        job.forward(threads); job.backward(threads)          # warm-up
        while t_total < seconds and reps < 50:
            t0 = time.perf_counter()
            job.forward(threads); job.backward(threads)
            t_total += time.perf_counter() - t0
            reps += 1
        job.close()
        kind = "reference"
        sample = (f"{reps} x full {w.name} workload fwd+bwd, fp32, reference_scan_fwd/bwd<1,{w.seq},{w.d_model}> "
                  f"per batch row on {threads} threads")
    else:
        threads = 1
        h = oracle.scan_forward_f32(a, b)
        while t_total < seconds and reps < 50:
            t0 = time.perf_counter()
            h = oracle.scan_forward_f32(a, b)
            oracle.scan_backward_f32(a, h, g)
            t_total += time.perf_counter() - t0
            reps += 1
        kind = "port"
        sample = f"{reps} x full {w.name} workload fwd+bwd, fp32, C restatement, 1 thread"
    return w.elems * reps / t_total, kind, threads, sample, t_total / reps


def run_reference_arm(args):
    from fast_sequential_scan_b200.workloads import CONFIGS
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = CONFIGS[args.workload]
    cores = os.cpu_count() or 1
    # each step = one bounded fwd+bwd sample; warm-up steps are run and discarded
    per_step_seconds = 0.0
    from oracle import oracle
    import numpy as np
    from fast_sequential_scan_b200.workloads import make_inputs
    a, b, g = (x.float().numpy() for x in make_inputs(w, "cpu", 0))
    job = oracle.RefLib().job(w.batch, w.seq, w.d_model) if oracle.RefLib.available() else None
    threads = max(1, min(cores, w.batch)) if job is not None else 1
    if job is not None:
        job.set(job.ALPHA, a); job.set(job.BETA, b); job.set(job.G, g)
        step = lambda: (job.forward(threads), job.backward(threads))
        kind = "reference"
        how = f"reference_scan_fwd/bwd<1,{w.seq},{w.d_model}> per batch row, {threads} threads"
    else:
        def step():
            h = oracle.scan_forward_f32(a, b)
            oracle.scan_backward_f32(a, h, g)
        kind = "port"
        how = "C restatement, 1 thread"
    steps = min(args.steps, 30)
    warm = min(args.warmup, 3)
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    value = w.elems / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{w.name}: B{w.batch} T{w.seq} D{w.d_model} {w.gates} gates, fp32 on CPU",
                   "note": "CPU arm runs the single-GPU workload once regardless of --gpus"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                         "sample": f"{steps} x full {w.name} workload fwd+bwd ({how})"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ sequence-parallel mode
def run_seqpar(args, world, rank, dev):
    """Sequence-parallel configuration (c5): every rank holds 65,536 rows of a (65,536 * N)-row sequence; a step
    is the sequence-parallel forward (local scan, all-gather of carries, fix-up) plus backward."""
    import torch
    import torch.distributed as dist
    import fast_sequential_scan_b200 as pkg
    from fast_sequential_scan_b200 import distributed as fd
    from fast_sequential_scan_b200.workloads import CONFIGS, make_inputs
    w = CONFIGS["c5_rank"]
    a, b, g = make_inputs(w, dev, seed=rank)
    ops = fd.NativeOps()
    group = None        # default group; with one rank no process group exists and the gather is the identity

    def step():
        h, saved = fd.seqpar_forward(a, b, group, ops)
        fd.seqpar_backward(a, h, g, saved, group, ops)

    for _ in range(max(3, args.warmup)):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    pkg.check_status()
    peak, kind = peaks()
    total = w.elems * world
    gbs = w.elems * 16 / (ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": total / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"c5: sequence-parallel fwd+bwd scan, B1 T{w.seq * world} D{w.d_model}, "
                                   f"{w.seq} rows per GPU, a~U(0.9,0.9999)",
                       "parallelism": f"sequence split x{world}: local scan, all-gather of (prod, carry), fix-up",
                       "l2": "per-rank working set 1.6 GB >> L2"},
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                         "traffic": None, "peak_kind": f"of {kind}", "per": "GPU, fwd+bwd 16 B/elem, fix-up traffic not counted"},
            "gpu_launches": None}), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------ gated forward mode
def run_gated(args, dev):
    """Forward scan with the gates computed in the kernel (fss_scan_forward_gated) on the workload's
    shape, beside the unfused route (torch gate formulas, then the plain forward scan).  One GPU."""
    import torch
    import fast_sequential_scan_b200 as pkg
    from fast_sequential_scan_b200 import sequential_scan_cuda as native
    from fast_sequential_scan_b200.workloads import CONFIGS, make_gate_inputs
    w = CONFIGS[args.workload if args.workload != "c2" else "c4_bf16"]
    esize = 2 if w.dtype == "bf16" else 4
    sets = min(16, max(3, -(-3 * L2_BYTES // (4 * w.elems * esize))))
    bufs = []
    for s in range(sets):
        r, i, x, lam = make_gate_inputs(w, dev, seed=s)
        bufs.append((r, i, x, lam, torch.empty_like(r)))

    def fused(s):
        r, i, x, lam, h = bufs[s % sets]
        native.forward_gated_into(r, i, x, lam, h)

    def unfused(s):
        r, i, x, lam, h = bufs[s % sets]
        a, b = native.gates_reference(r, i, x, lam)
        native.forward_into(a, b, h)

    def timed(fn):
        for s in range(max(3, args.warmup)):
            fn(s)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(args.steps):
            fn(s)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.steps

    ms, ms_unfused = timed(fused), timed(unfused)
    pkg.check_status()
    peak, kind = peaks()
    gbs = w.elems * 4 * esize / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "gated scan fwd elems/s", "value": w.elems / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": f"{w.name}: gated forward scan, B{w.batch} T{w.seq} D{w.d_model}, r,i,x~N(0,1), "
                               "lambda~U(-4.3,-0.5)",
                   "l2": f"rotating {sets} disjoint buffer sets", "launch": "one C-ABI launch per step from Python"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                     "traffic": None, "peak_kind": f"of {kind}",
                     "algorithmic_bytes": w.elems * 4 * esize, "per": "read r, i, x; write h"},
        "unfused": {"ms_per_step": ms_unfused, "what": "torch gate formulas (fp32 math, rounded once) + plain forward scan",
                    "speedup": ms_unfused / ms},
        "gpu_launches": args.steps}), flush=True)


# ------------------------------------------------------------------ GPU arm
def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch
    import torch.distributed as dist
    import fast_sequential_scan_b200 as pkg
    from fast_sequential_scan_b200 import _lib, sequential_scan_cuda as native
    from fast_sequential_scan_b200.workloads import CONFIGS, make_inputs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.mode == "seqpar":
        run_seqpar(args, world, rank, dev)
        return
    if args.mode == "gated":
        if rank == 0:
            run_gated(args, dev)
        return

    w = CONFIGS[args.workload]
    if args.shape:
        import dataclasses
        bb, tt, dd = (int(x) for x in args.shape.split(","))
        w = dataclasses.replace(w, name=f"{w.name}[{bb}x{tt}x{dd}]", batch=bb, seq=tt, d_model=dd)
    algo = _lib.ALGO_BY_NAME[args.algo]
    dt = w.torch_dtype
    esize = 2 if w.dtype == "bf16" else 4
    tensor_bytes = w.elems * esize
    # rotate enough disjoint buffer sets that no step finds its inputs in L2
    sets = max(3, -(-3 * L2_BYTES // (6 * tensor_bytes)))
    sets = min(sets, 16)
    bufs = []
    for s in range(sets):
        a, b, g = make_inputs(w, dev, seed=1000 * rank + s)
        bufs.append(dict(a=a, b=b, g=g, h=torch.empty_like(a), da=torch.empty_like(a), db=torch.empty_like(a)))

    def fwd(s):
        x = bufs[s % sets]
        native.forward_into(x["a"], x["b"], x["h"], algo=algo)

    def bwd(s):
        x = bufs[s % sets]
        native.backward_into(x["a"], x["h"], x["g"], x["da"], x["db"], algo=algo)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    side = torch.cuda.Stream(dev)

    def capture(fn, first, count):
        """CUDA graph of `count` consecutive steps starting at buffer set `first` (the launches
        themselves are the library's own C-ABI calls, recorded on the capture stream)."""
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(count):
                fn(first + i)
        return g

    def timed(fn, steps, warmup, graphs=True):
        """Device time per step of exactly `steps` steps, max over ranks.  With graphs the steps
        are replayed from CUDA graphs of `sets` steps each (plus one shorter graph for the
        remainder) so that host launch cost does not gate a ~50 us step."""
        with torch.cuda.stream(side):
            for i in range(max(warmup, 3)):
                fn(i)
        side.synchronize()
        if graphs:
            full, rem = divmod(steps, sets)
            g_full = capture(fn, 0, sets) if full else None
            g_rem = capture(fn, 0, rem) if rem else None
            with torch.cuda.stream(side):
                for g in (g_full, g_rem):
                    if g is not None:
                        g.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(side):
            e0.record()
            if graphs:
                for _ in range(full):
                    g_full.replay()
                if rem:
                    g_rem.replay()
            else:
                for i in range(steps):
                    fn(warmup + i)
            e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # which kernels a step launches (for gpu_launches): probe the algorithm actually taken
    took_lookback = True
    try:
        native.forward_into(bufs[0]["a"], bufs[0]["b"], bufs[0]["h"], algo=_lib.ALGO_LOOKBACK)
    except _lib.FssError:
        took_lookback = False
    if args.algo == "chunked":
        took_lookback = False
    launches_per_step = 2 if took_lookback else 6

    use_graphs = not args.no_graphs
    sampler = ClockSampler(local) if rank == 0 else None
    t_begin = time.perf_counter()
    ms_step = timed(lambda i: (fwd(i), bwd(i)), args.steps, args.warmup, use_graphs)
    ms_fwd = timed(fwd, args.steps, max(3, args.warmup // 4), use_graphs)
    ms_bwd = timed(bwd, args.steps, max(3, args.warmup // 4), use_graphs)
    # keep the same step loop running until the clock sampler (100 ms period) has a few samples
    # under load; these extra steps are not part of any reported time
    soak_steps = 0
    while not args.no_soak and time.perf_counter() - t_begin < 1.5:
        with torch.cuda.stream(side):
            for i in range(200):
                fwd(i); bwd(i)
        side.synchronize()
        soak_steps += 200
    clocks = sampler.stop() if sampler else None
    if clocks is not None:
        clocks["window"] = f"warm-up + timed region + {soak_steps} further steps of the same loop"
    pkg.check_status()

    total_elems = w.elems * world
    value = total_elems / (ms_step * 1e-3)
    peak, peak_kind = peaks()
    bwd_bytes = w.elems * w.bytes_per_elem(backward=True, forward=False)
    fwd_bytes = w.elems * w.bytes_per_elem(backward=False, forward=True)
    ach_bwd = bwd_bytes / (ms_bwd * 1e-3) / 1e9
    ach_fwd = fwd_bytes / (ms_fwd * 1e-3) / 1e9
    ach_step = (bwd_bytes + fwd_bytes) / (ms_step * 1e-3) / 1e9
    kernel_bwd = "fss::lookback::scan_kernel<bf16, backward> (single pass)" if took_lookback else "fss::chunked::chunk_scan_backward (+summary, compose)"
    roofline = {"bound": "hbm", "kernel": kernel_bwd, "achieved": ach_bwd, "peak": peak, "unit": "GB/s",
                "frac": ach_bwd / peak,
                "traffic": NCU_TRAFFIC.get((args.workload if not args.shape else "", "lookback" if took_lookback else "chunked")),
                "algorithmic_bytes": bwd_bytes, "peak_kind": f"of {peak_kind}",
                "ms_per_launch": ms_bwd,
                "forward": {"achieved": ach_fwd, "frac": ach_fwd / peak, "ms_per_launch": ms_fwd},
                "step": {"achieved": ach_step, "frac": ach_step / peak}}

    # ---- end to end through the public autograd API, from pinned host memory ----
    e2e = None
    if not args.no_e2e:
        ha, hb, hg = (x.cpu().pin_memory() for x in (bufs[0]["a"], bufs[0]["b"], bufs[0]["g"]))
        out_da = torch.empty(ha.shape, dtype=dt).pin_memory()
        out_db = torch.empty(ha.shape, dtype=dt).pin_memory()
        out_h = torch.empty(ha.shape, dtype=dt).pin_memory()

        # Three streams, two device buffer sets: the host-to-device copies of step i+1 and the
        # device-to-host copies of step i-1 run while step i computes (PCIe is full duplex).  Every
        # copy and every launch of a step is inside the timed region; the timing stream waits for
        # the last device-to-host copy of every step.
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        dsets = [tuple(torch.empty(ha.shape, dtype=dt, device=dev) for _ in range(3)) for _ in range(2)]
        computed = [None, None]          # event: the compute that last read buffer set k is done
        scan_fn = pkg.scan_cu if w.dtype == "bf16" else pkg.scan_cu_single

        def e2e_step(i):
            k = i % 2
            da_, db_, dg_ = dsets[k]
            with torch.cuda.stream(s_in):
                if computed[k] is not None:
                    s_in.wait_event(computed[k])
                da_.copy_(ha, non_blocking=True)
                db_.copy_(hb, non_blocking=True)
                dg_.copy_(hg, non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(arrived)
                a = da_.detach().requires_grad_(True)
                b = db_.detach().requires_grad_(True)
                h = scan_fn(a, b)
                h.backward(dg_)
                done = torch.cuda.Event()
                done.record(s_cmp)
                computed[k] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for t in (h, a.grad, b.grad):
                    t.record_stream(s_out)
                out_h.copy_(h.detach(), non_blocking=True)
                out_da.copy_(a.grad, non_blocking=True)
                out_db.copy_(b.grad, non_blocking=True)
                left = torch.cuda.Event()
                left.record(s_out)
            torch.cuda.current_stream().wait_event(left)

        e_steps = max(3, min(args.steps, 20))
        ms_e2e = timed(e2e_step, e_steps, 3, graphs=False)
        e2e = {"value": total_elems / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e, "steps": e_steps,
               "h2d_bytes_per_step": 3 * tensor_bytes, "d2h_bytes_per_step": 3 * tensor_bytes,
               "api": "scan_cu(alpha, beta); h.backward(grad) on tensors copied from pinned host memory; "
                      "h, dalpha, dbeta copied back; copies of neighbouring steps overlap the compute "
                      "(3 streams, 2 device buffer sets)"}
        pkg.check_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        v, kind, cores, sample, _ = cpu_reference_leg(w, args.cpu_seconds, os.cpu_count() or 1)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample,
               "host_cpus": os.cpu_count()}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
            "config": {"workload": f"{w.name}: fwd+bwd scan, B{w.batch} T{w.seq} D{w.d_model} per GPU, {w.gates} gates",
                       "algo": "lookback" if took_lookback else "chunked",
                       "parallelism": f"channel-sharded x{world} (d_model {w.d_model * world} total), no collective",
                       "launch": "CUDA-graph replay of the C-ABI launches" if use_graphs else "one C-ABI call per kernel from Python",
                       "l2": f"rotating {sets} disjoint buffer sets ({sets * 6 * tensor_bytes / 1e6:.0f} MB > 126 MB L2)"},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches_per_step * args.steps,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
