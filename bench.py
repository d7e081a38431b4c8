#!/usr/bin/env python
"""Benchmark of the FlashMask hot path: forward + backward of
``flashmask_attention`` on a causal-document mask.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  ``value`` is fwd+bwd effective TFLOP/s counting
only unmasked (query, key) pairs, summed over all GPUs, with inputs resident in
HBM; ``e2e`` is the same metric through the public operator with pinned HOST
buffers (host->device and device->host copies of every step inside the timed
region, pipelined over three streams and two buffer sets);
``roofline`` describes the dominant kernel; ``cpu_baseline`` is the CPU
restatement of the reference's dense-mask attention timed on a bounded sample.
``--impl reference`` times that CPU implementation alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC = "fwd_bwd_effective_tflops_unmasked"
UNIT = "TFLOP/s"


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks / throttle reasons while running: NVML polled every few ms from a thread (read-only
    queries), or `nvidia-smi -lms 100` when the NVML binding is not importable."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    # bits of the NVML clocks-event (throttle) reasons word
    BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.nv = None
        self._stop = False

    def _start_nvml(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        self.reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
            pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
        self.mx = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        pynvml.nvmlDeviceGetClockInfo(self.h, pynvml.NVML_CLOCK_SM)       # fails here rather than in the thread
        self.nv = pynvml
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def _poll(self):
        nv = self.nv
        while not self._stop:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                word = int(self.reasons_fn(self.h))
                f = [str(mhz), str(self.mx)] + ["Active" if word & bit else "Not Active" for _, bit in self.BITS]
                self.samples.append((time.perf_counter(), ", ".join(f)))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            self._start_nvml()
            return
        except Exception:
            self.nv = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def mark(self):
        """Start of the timed region (the sampler itself is started before the warm-up: nvidia-smi
        takes a few hundred ms to deliver its first sample)."""
        self.t_mark = time.perf_counter()

    def stop(self):
        if self.proc is None and self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        t_end = time.perf_counter()
        if self.nv is not None:
            self._stop = True
            self.thread.join(timeout=1)
        else:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
        t_mark = getattr(self, "t_mark", 0.0)
        inside = [l for t, l in self.samples if t_mark <= t <= t_end + (0.0 if self.nv is not None else 0.1)]
        window = "timed region"
        if not inside:      # a timed region shorter than the sampling period: the warm-up ran the same load
            inside, window = [l for _, l in self.samples], "warm-up + timed region"
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in inside:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm),
                "window": window, "source": "nvml" if self.nv is not None else "nvidia-smi"}


# ---------------------------------------------------------------------------
# CPU baseline (the checker's dense-mask attention, fp32, all host threads)
# ---------------------------------------------------------------------------
def cpu_sample(w, heads: int = 4):
    """Bounded sample of the workload for the CPU arm: batch 0, one kv head and
    the first ``heads`` q heads of its group; the full sequence up to 16K tokens, a
    sample of 1024 query rows (forward, dQ and their share of dK / dV) beyond."""
    import oracle  # CPU-baseline leg only
    g = torch.Generator().manual_seed(w.seed)
    heads = min(heads, w.Hq // w.Hkv)
    if w.Sq > 16384:
        q = torch.randn(w.Sq, heads, w.d, generator=g)
        k = torch.randn(w.Sk, w.d, generator=g)
        v = torch.randn(w.Sk, w.dv, generator=g)
        do = torch.randn(w.Sq, heads, w.dv, generator=g)
        bounds = None if w.idx is None else w.idx[0, 0]
        rows = np.sort(np.random.default_rng(w.seed).choice(w.Sq, 1024, replace=False))
        nvis = 0
        for c0 in range(0, rows.size, 512):
            nvis += int(oracle.visible_block(bounds, w.Sq, w.Sk, w.causal, rows[c0:c0 + 512],
                                             np.arange(w.Sk)).sum())
        flops = 2 * nvis * heads * (4 * w.d + 3 * w.dv)

        def step_rows():
            return [oracle.attention_rows(q[:, h], k, v, do[:, h], bounds, w.causal, rows=rows)
                    for h in range(heads)]
        desc = (f"batch 0, 1 kv head x {heads} q heads, 1024 sampled query rows of S={w.Sq} against all keys "
                f"({nvis * heads / max(1, w.n_visible()):.2e} of the workload's unmasked pairs), fp32")
        return step_rows, flops, desc
    q = torch.randn(1, w.Sq, heads, w.d, generator=g)
    k = torch.randn(1, w.Sk, 1, w.d, generator=g)
    v = torch.randn(1, w.Sk, 1, w.dv, generator=g)
    do = torch.randn(1, w.Sq, heads, w.dv, generator=g)
    idx = None if w.idx is None else w.idx[:1]
    from flashmask_b200 import workloads as W
    nvis = int(W.count_visible(idx, 1, w.Sq, w.Sk, w.causal).sum()) * heads
    flops = 2 * nvis * (4 * w.d + 3 * w.dv)

    def step():
        return oracle.attention_forward_backward(q, k, v, do, idx, w.causal)
    desc = f"batch 0, 1 kv head x {heads} q heads, S={w.Sq} (1/{w.B * w.Hq // heads} of the workload), fp32"
    return step, flops, desc


def time_cpu(step, flops, steps, warmup):
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return flops / dt / 1e12, dt * 1e3


# ---------------------------------------------------------------------------
# end-to-end leg: host buffers in, host buffers out
# ---------------------------------------------------------------------------
def e2e_pipelined(compute, host_in, n_steps, dev, sync):
    """Time `n_steps` steps of `compute` with host buffers on both sides, every copy inside the timed region.

    Each step copies ALL its inputs from pinned host memory into device buffers, runs the public operator
    (`compute(dict of device tensors) -> tuple of device results`) and copies ALL its results into pinned
    host memory.  The three phases run on three streams over two buffer sets, the way a caller with host
    data would drive the operator: the upload of step i+1 and the download of step i-1 overlap the
    kernels of step i (PCIe carries both directions at once).  Returns (ms per step, d2h bytes per step)."""
    main = torch.cuda.current_stream(dev)
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev = lambda: torch.cuda.Event()
    slots = [{"inp": {n_: torch.empty_like(t_, device=dev) for n_, t_ in host_in.items()}, "host": None,
              "keep": None, "up": ev(), "done": ev(), "down": ev()} for _ in range(2)]

    def run(n):
        for i in range(n):
            sl = slots[i % 2]
            if sl["keep"] is not None:
                up.wait_event(sl["done"])          # the step that read these input buffers has finished
            with torch.cuda.stream(up):
                for n_, t_ in host_in.items():
                    sl["inp"][n_].copy_(t_, non_blocking=True)
                sl["up"].record(up)
            main.wait_event(sl["up"])
            if sl["keep"] is not None:
                main.wait_event(sl["down"])        # its results have left before their memory is reused
            outs = compute(sl["inp"])
            sl["done"].record(main)
            sl["keep"] = outs
            if sl["host"] is None:
                sl["host"] = [torch.empty(o_.shape, dtype=o_.dtype).pin_memory() for o_ in outs]
            down.wait_event(sl["done"])
            with torch.cuda.stream(down):
                for h_, o_ in zip(sl["host"], outs):
                    h_.copy_(o_, non_blocking=True)
                sl["down"].record(down)
        for sl in slots:
            if sl["keep"] is not None:
                main.wait_event(sl["down"])

    run(2)
    sync()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(main)
    up.wait_event(a)
    run(n_steps)
    b.record(main)
    sync()
    d2h = sum(h_.numel() * h_.element_size() for h_ in slots[0]["host"])
    return a.elapsed_time(b) / n_steps, d2h


# ---------------------------------------------------------------------------
# context-parallel leg (N > 1): 128K-token causal-document mask, sequence sharded
# ---------------------------------------------------------------------------
def run_cp(args, rank, local_rank, world):
    import torch.distributed as dist
    import flashmask_b200 as fm
    from flashmask_b200 import cp_balance, workloads as W
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # NCCL's internal stream at high priority: its send/recv blocks get SM slots
    # ahead of the queued attention CTAs, so the transfers really overlap
    from torch.distributed import ProcessGroupNCCL
    opts = ProcessGroupNCCL.Options(is_high_priority_stream=True)
    dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    name = args.workload or "cp_causal_doc_128k"
    w = W.make_workload(name)
    chunk = 2048
    from flashmask_b200 import _lib
    parity = cp_parity_check(name, rank, world, dev, chunk)
    if not parity["ok"]:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "n_gpus": world, "cp_parity": parity, "error": "cp parity failed"}))
        dist.destroy_process_group()
        sys.exit(1)
    idx = torch.from_numpy(w.idx).to(dev)
    t0 = time.perf_counter()
    local_mask, buckets = cp_balance.balance_flashmask_input(idx, world, rank, balance_chunk_size=chunk)
    torch.cuda.synchronize()
    partition_ms = (time.perf_counter() - t0) * 1e3
    loads = [sum(x for x, _ in b) for b in buckets]
    S_local = w.Sq // world
    g = torch.Generator().manual_seed(w.seed + rank)
    host = {n_: torch.randn(w.B, S_local, h, dd, generator=g).to(torch.bfloat16).pin_memory()
            for n_, h, dd in (("q", w.Hq, w.d), ("k", w.Hkv, w.d), ("v", w.Hkv, w.dv), ("do", w.Hq, w.dv))}
    q, k, v, do = (host[n_].to(dev) for n_ in ("q", "k", "v", "do"))
    fwd_flops, bwd_flops = w.flops()
    group = dist.group.WORLD

    def step(qd, kd, vd, dod):
        qd.requires_grad_(True); kd.requires_grad_(True); vd.requires_grad_(True)
        o = fm.flashmask_attention(qd, kd, vd, local_mask, causal=False, group=group)
        o.backward(dod)
        return o, qd.grad, kd.grad, vd.grad

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def fresh():
        return q.detach().clone(), k.detach().clone(), v.detach().clone(), do

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        step(*fresh())
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ins = [fresh() for _ in range(args.steps)]
    barrier()
    sampler.mark()
    n0 = _lib.load().fm_launch_count()
    t_host = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        step(*ins[i])
    e1.record()
    host_ms = (time.perf_counter() - t_host) * 1e3 / args.steps     # host time to ENQUEUE a step
    launches = torch.tensor([_lib.load().fm_launch_count() - n0], device=dev, dtype=torch.int64)
    barrier()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(launches, op=dist.ReduceOp.SUM)
    ms_step = t.item() / args.steps
    value = (fwd_flops + bwd_flops) / (ms_step * 1e-3) / 1e12
    phases = None
    if args.cp_phases:
        from flashmask_b200 import cp as cpm
        cpm.profile_phases(True)
        for _ in range(3):
            step(*fresh())
        rep = cpm.phase_report()
        cpm.profile_phases(False)
        names = sorted(rep)
        vals = torch.tensor([rep[n_] / 3 for n_ in names], device=dev)
        allv = [torch.empty_like(vals) for _ in range(world)]
        dist.all_gather(allv, vals)
        phases = {n_: [round(float(a_[i]), 3) for a_ in allv] for i, n_ in enumerate(names)}

    e2e = None
    if not args.no_e2e:
        def compute(inp):
            o, dq, dk, dv = step(inp["q"].detach(), inp["k"].detach(), inp["v"].detach(), inp["do"])
            return o.detach(), dq, dk, dv
        n_e = max(3, args.steps)
        ms_e, d2h = e2e_pipelined(compute, host, n_e, dev, barrier)
        te = torch.tensor([ms_e], device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        nbytes = sum(x.numel() * x.element_size() for x in host.values())
        e2e = {"value": (fwd_flops + bwd_flops) / (te.item() * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": d2h * world,
               "ms_per_step": te.item(), "steps": n_e,
               "pipeline": "upload / operator / download on three streams, two buffer sets; every step copies "
                           "all its inputs and all its results"}
    from flashmask_b200 import cp as cpmod
    n_needed = int(cpmod.shard_need_row(local_mask, S_local, False, world).sum().item())
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_tf = peaks.get("bf16_tflops_sustained") or 1400.0
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{name}: B={w.B} Hq={w.Hq} Hkv={w.Hkv} S={w.Sq} d={w.d} causal-document mask "
                                   f"(heavy-tailed lognormal docs) in the non-causal 2-column form, sequence sharded "
                                   f"over {world} ranks by the mask-aware partitioner ({chunk}-row chunks)",
                       "l2": "per-rank tensors exceed the 126 MB L2; no flush between steps",
                       "mask_sparsity": round(w.sparsity(), 4), "parallelism": f"cp{world}",
                       "partition_ms": partition_ms, "rank_loads": loads},
            "clocks": clocks, "e2e": e2e, "cp_parity": parity, "host_enqueue_ms_per_step": round(host_ms, 3),
            "gpu_launches": int(launches.item()), "tokens_per_s": w.B * w.Sq / (ms_step * 1e-3),
            "roofline": {"bound": "tensor", "kernel": "fwd + bwd tcgen05 kernels over all ring steps (aggregate)",
                         "achieved": value / world, "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": value / world / peak_tf, "peak_source": "measured (sustained cuBLAS bf16)",
                         "traffic": None}}
    if phases is not None:
        line["cp_phases_ms_per_rank"] = phases
    if rank == 0:
        print(json.dumps(line))
    dist.destroy_process_group()


def cp_parity_check(name, rank, world, dev, chunk, S=16384):
    """Before anything is timed: the context-parallel operator on a reduced copy of the workload
    (same generator, S tokens) against the single-GPU operator, on this rank's rows and keys.
    Returns {"ok", "max_err", "tol", "S"} with the maximum over ranks and over out / dq / dk / dv
    (tolerance: every element is a sum of at most `world` bf16-rounded partials)."""
    import torch.distributed as dist
    import flashmask_b200 as fm
    from flashmask_b200 import cp_balance, workloads as W
    w = W.make_workload(name, S=S)
    idx = torch.from_numpy(w.idx).to(dev)
    g = torch.Generator().manual_seed(w.seed)
    q, k, v, do = (torch.randn(w.B, S, h, dd, generator=g).to(torch.bfloat16).to(dev)
                   for h, dd in ((w.Hq, w.d), (w.Hkv, w.d), (w.Hkv, w.dv), (w.Hq, w.dv)))
    local, buckets = cp_balance.balance_flashmask_input(idx, world, rank, balance_chunk_size=chunk)
    ql, kl, vl, dol = (cp_balance.scatter_by_buckets(t, buckets, rank) for t in (q, k, v, do))
    ql, kl, vl = (t.requires_grad_(True) for t in (ql, kl, vl))
    out = fm.flashmask_attention(ql, kl, vl, local, causal=False, group=dist.group.WORLD, deterministic=True)
    out.backward(dol)
    qg, kg, vg = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref = fm.flashmask_attention(qg, kg, vg, idx, causal=False, deterministic=True)
    ref.backward(do)
    worst, ok = 0.0, True
    for a, b in ((out, ref), (ql.grad, qg.grad), (kl.grad, kg.grad), (vl.grad, vg.grad)):
        bl = cp_balance.scatter_by_buckets(b.detach(), buckets, rank).float()
        err = (a.detach().float() - bl).abs().max().item()
        tol = 2 ** -7 * world * max(1.0, bl.abs().max().item())
        worst = max(worst, err / tol)
        ok = ok and err <= tol and not torch.isnan(a.float()).any().item()
    t = torch.tensor([worst, 0.0 if ok else 1.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"ok": t[1].item() == 0.0, "max_err_over_tol": round(t[0].item(), 4), "S": S,
            "checked": "out, dq, dk, dv of every rank vs the single-GPU operator, bf16"}


# ---------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--cp-phases", action="store_true", help="N > 1: per-phase device times of every rank")
    ap.add_argument("--sustained", type=float, default=2.0,
                    help="N = 1: seconds of back-to-back steps for the sustained-clock figure (0: skip)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    from flashmask_b200 import workloads as W
    name = args.workload or ("cp_causal_doc_128k" if args.gpus > 1 else "causal_doc_8k_gqa")
    w = W.make_workload(name)
    kind = ("causal mask, per-head sink logit, deterministic backward" if w.idx is None else
            "mask from the column bounds of the named workload")
    config = {"workload": f"{name}: B={w.B} Hq={w.Hq} Hkv={w.Hkv} S={w.Sq} d={w.d} dv={w.dv} "
                          f"{kind}, bf16, fwd+bwd",
              "l2": "inputs+outputs (>500 MB) exceed the 126 MB L2; no flush between steps",
              "mask_sparsity": round(w.sparsity(), 4),
              "parallelism": "1 GPU" if args.gpus == 1 else f"cp{args.gpus}"}

    if args.impl == "reference":
        if rank != 0:
            return
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        step, flops, desc = cpu_sample(w)
        val, ms = time_cpu(step, flops, max(1, args.steps), max(1, args.warmup))
        line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc},
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if world > 1:
        return run_cp(args, rank, local_rank, world)

    import flashmask_b200 as fm
    from flashmask_b200 import _lib
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    launch_count = _lib.load().fm_launch_count

    g = torch.Generator().manual_seed(w.seed + rank)
    host = {
        "q": torch.randn(w.B, w.Sq, w.Hq, w.d, generator=g).to(torch.bfloat16).pin_memory(),
        "k": torch.randn(w.B, w.Sk, w.Hkv, w.d, generator=g).to(torch.bfloat16).pin_memory(),
        "v": torch.randn(w.B, w.Sk, w.Hkv, w.dv, generator=g).to(torch.bfloat16).pin_memory(),
        "do": torch.randn(w.B, w.Sq, w.Hq, w.dv, generator=g).to(torch.bfloat16).pin_memory(),
    }
    idx_host = torch.from_numpy(w.idx).pin_memory() if w.idx is not None else None
    q, k, v, do = (host[n].to(dev) for n in ("q", "k", "v", "do"))
    idx = idx_host.to(dev) if idx_host is not None else None
    fwd_flops, bwd_flops = w.flops()
    sink = torch.randn(w.Hq, generator=g).to(dev) if w.sink else None
    det = bool(w.deterministic)

    ftm, ftn = fm.fwd_tile_shape(w.d, w.dv)
    btm, btn = fm.bwd_tile_shape(w.d, w.dv)

    def step_device():
        # mask preprocessing and the launch tables are part of every step
        info_f = fm.prepare_mask(idx, w.Sq, w.causal, ftm, ftn) if idx is not None else None
        info_b = info_f if (info_f is None or btn == ftn) else fm.prepare_mask(idx, w.Sq, w.causal, btm, btn)
        out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=w.causal, learnable_sink=sink, mask_info=info_f)
        return fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=w.causal, learnable_sink=sink,
                                  deterministic=det, mask_info=info_b)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(max(3, args.warmup)):
        step_device()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.mark()
    n0 = launch_count()
    e0.record()
    for _ in range(args.steps):
        step_device()
    e1.record()
    gpu_launches = launch_count() - n0
    barrier()
    ms_total = e0.elapsed_time(e1)
    clocks = sampler.stop()
    # per-kernel-group timing on the launching stream (roofline of the dominant one), under the conditions of the
    # timed region above: a short loop at full clocks
    info_f = fm.prepare_mask(idx, w.Sq, w.causal, ftm, ftn) if idx is not None else None
    info_b = info_f if (info_f is None or btn == ftn) else fm.prepare_mask(idx, w.Sq, w.causal, btm, btn)
    out, lse = fm._flash_attn_fwd(q, k, v, idx, causal=w.causal, learnable_sink=sink, mask_info=info_f)

    def timed(fn, reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()                          # one untimed call: allocator growth and first-use costs stay outside
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps
    reps = max(3, args.steps // 2)
    ms_fwd = timed(lambda: fm._flash_attn_fwd(q, k, v, idx, causal=w.causal, learnable_sink=sink,
                                              mask_info=info_f), reps)
    ms_bwd = timed(lambda: fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=w.causal, learnable_sink=sink,
                                              deterministic=det, mask_info=info_b), reps)
    ms_prep = timed(lambda: fm.prepare_mask(idx, w.Sq, w.causal, ftm, ftn), reps) if idx is not None else 0.0

    # the same step back to back for a few seconds: the clocks a long training run sees (power cap)
    sustained = None
    if args.sustained > 0 and world == 1:
        n_s = max(args.steps, int(args.sustained * 1e3 / max(ms_total / args.steps, 1e-3)))
        smp = ClockSampler(local_rank)
        smp.start()
        time.sleep(0.3)
        torch.cuda.synchronize()
        smp.mark()
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_.record()
        for _ in range(n_s):
            step_device()
        b_.record()
        torch.cuda.synchronize()
        ck = smp.stop()
        ms_s = a_.elapsed_time(b_) / n_s
        ms_bwd_s = timed(lambda: fm._flash_attn_bwd(q, k, v, out, do, lse, idx, causal=w.causal, learnable_sink=sink,
                                                    deterministic=det, mask_info=info_b), reps)
        sustained = {"steps": n_s, "ms_per_step": ms_s,
                     "value": (fwd_flops + bwd_flops) / (ms_s * 1e-3) / 1e12, "unit": UNIT, "clocks": ck,
                     "bwd_ms_after": ms_bwd_s}
    t = torch.tensor([ms_total], device=dev)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = world * (fwd_flops + bwd_flops) / (ms_step * 1e-3) / 1e12

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    # the group is timed alone in a short loop at full clocks: the burst figure is its denominator; the long loop
    # of the `sustained` leg is read against the sustained figure
    peak_tf = peaks.get("bf16_tflops") or 1590.0
    peak_sus = peaks.get("bf16_tflops_sustained") or 1400.0
    peak_src = "measured (burst cuBLAS bf16; sustained figure for the sustained leg)" if peaks else "fallback"
    dom = "bwd" if ms_bwd >= ms_fwd else "fwd"
    # DRAM bytes per launch of this workload from one ncu capture: forward kernel; backward = preprocess (with
    # the accumulator clear) + one-kernel backward + dQ rounding (the two-kernel backward measured 1771 MB)
    NCU_DRAM_BYTES = {"fwd": 389.9e6, "bwd": 3495.0e6 if not det else 1771.0e6}
    dom_flops, dom_ms = (bwd_flops, ms_bwd) if dom == "bwd" else (fwd_flops, ms_fwd)
    ach = dom_flops / (dom_ms * 1e-3) / 1e12
    bwd_kind = ("preprocess + dK/dV + dQ kernels" if det or w.d != w.dv or w.d not in (64, 128) else
                "preprocess + one-kernel backward + dQ rounding")
    roofline = {"bound": "tensor", "kernel": f"fm_bwd ({bwd_kind})" if dom == "bwd" else "fm_fwd kernel",
                "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
                "peak_source": peak_src,
                "sustained": None if sustained is None else {
                    "achieved": bwd_flops / (sustained["bwd_ms_after"] * 1e-3) / 1e12, "peak": peak_sus,
                    "frac": bwd_flops / (sustained["bwd_ms_after"] * 1e-3) / 1e12 / peak_sus,
                    "what": "the backward group timed right after the sustained loop, at the clocks it left"},
                "traffic": NCU_DRAM_BYTES[dom] if name == "causal_doc_8k_gqa" else None,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, "
                "one capture of this workload (constants copied from the ncu summaries committed with this file)"
                if name == "causal_doc_8k_gqa" else "no capture of this workload",
                "fwd_ms": ms_fwd, "bwd_ms": ms_bwd, "mask_prep_ms": ms_prep,
                "fwd_tflops": fwd_flops / (ms_fwd * 1e-3) / 1e12,
                "bwd_tflops": bwd_flops / (ms_bwd * 1e-3) / 1e12}

    # end to end through the public operator with host buffers
    host_in = dict(host)
    if idx_host is not None:
        host_in["idx"] = idx_host

    def compute(inp):
        qd = inp["q"].detach().requires_grad_(True)
        kd = inp["k"].detach().requires_grad_(True)
        vd = inp["v"].detach().requires_grad_(True)
        o = fm.flashmask_attention(qd, kd, vd, inp.get("idx"), causal=w.causal, sink=sink, deterministic=det)
        o.backward(inp["do"])
        return o.detach(), qd.grad, kd.grad, vd.grad
    h2d = sum(t_.numel() * t_.element_size() for t_ in host_in.values())
    e2e = None
    if not args.no_e2e:
        e_steps = max(6, 2 * args.steps)      # the two-step ramp of the pipeline weighs less over more steps
        ms_e, d2h = e2e_pipelined(compute, host_in, e_steps, dev, barrier)
        te = torch.tensor([ms_e], device=dev)
        if world > 1:
            torch.distributed.all_reduce(te, op=torch.distributed.ReduceOp.MAX)
        e2e_val = world * (fwd_flops + bwd_flops) / (te.item() * 1e-3) / 1e12
        e2e = {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": te.item(), "steps": e_steps,
               "pipeline": "upload / operator / download on three streams, two buffer sets; every step copies "
                           "all its inputs (q, k, v, dO, mask) and all its results (O, dQ, dK, dV)"}

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config, "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": int(gpu_launches), "roofline": roofline, "sustained": sustained,
            "frac_of_peak_fwd_bwd": value / world / peak_tf,
            "frac_of_sustained_peak_fwd_bwd": None if sustained is None else sustained["value"] / peak_sus,
            "tokens_per_s": world * w.B * w.Sq / (ms_step * 1e-3)}
    if w.Sq <= 16384:
        # the reference benchmark's accounting: every 128x128 block with one unmasked element counts in full
        dens = W.block_density(w.idx, w.B, w.Sq, w.Sk, w.causal)
        blk_flops = 2.0 * w.B * w.Hq * w.Sq * w.Sk * dens * (4 * w.d + 3 * w.dv)
        line["block_density_convention"] = {"density": dens, "value": world * blk_flops / (ms_step * 1e-3) / 1e12,
                                            "unit": UNIT}
    if world == 1 and not args.no_e2e and args.workload is None:
        # the context-parallel workload on this one GPU: the N=1 point of the 128K scaling series
        wc = W.make_workload("cp_causal_doc_128k")
        gc = torch.Generator().manual_seed(wc.seed)
        qc, kc, vc, doc = (torch.randn(wc.B, wc.Sq, h, wc.d, generator=gc).to(torch.bfloat16).to(dev)
                           for h in (wc.Hq, wc.Hkv, wc.Hkv, wc.Hq))
        idc = torch.from_numpy(wc.idx).to(dev)

        def step_c():
            o_, l_ = fm._flash_attn_fwd(qc, kc, vc, idc, causal=wc.causal)
            return fm._flash_attn_bwd(qc, kc, vc, o_, doc, l_, idc, causal=wc.causal)
        ms_c = timed(step_c, 5) if (step_c(), step_c(), step_c()) else 0.0
        fc, bc = wc.flops()
        line["cp_128k_single_gpu"] = {"ms_per_step": ms_c, "tokens_per_s": wc.B * wc.Sq / (ms_c * 1e-3),
                                      "mask_form": "non-causal 2-column [LTS, UTE], as in the N > 1 runs",
                                      "value": (fc + bc) / (ms_c * 1e-3) / 1e12, "unit": UNIT,
                                      "mask_sparsity": round(wc.sparsity(), 4)}
        del qc, kc, vc, doc
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        step, flops, desc = cpu_sample(w)
        val, ms = time_cpu(step, flops, 3, 1)
        line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                                "sample": desc + f"; {ms:.0f} ms per fwd+bwd"}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
