#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg4] [--impl ours|reference]

Headline: one layer, forward + dgrad + wgrad per step, over one synthetic voxel cloud
(``fgms_b200.workloads``; default ``cfg4``: LiDAR-like sweep, 3x3x3 submanifold, fp16 128->128 — the
configuration the 60 %-of-roofline target is stated on).  The metric is effective TFLOPS =
6 * pairs * c_in * c_out / time; ``ms_per_step`` is ms per layer.

* ``value``      device-resident inputs, CUDA events around each step on the launching stream, L2
                 flushed (a 512 MB buffer is overwritten) and outputs re-zeroed before every step,
                 outside the timed interval.
* ``e2e``        the same step through the public binding with HOST buffers: pinned host -> device
                 copies of features, weights, output gradient and maps, the three operator calls,
                 and device -> host copies of all three results, all inside the timed interval.
* ``roofline``   for the slowest of the three kernels of the step: algorithmic bytes of that pass
                 divided by its mean launch duration (events around the kernel call alone, no
                 collective inside), against max(bytes / measured HBM bandwidth, flops / tensor peak).
* ``cpu_baseline`` / ``--impl reference``  the reference's CPU definition (cpu-check.py /
                 cpu-check-back.py) restated per offset as index_select -> matmul -> index_add_ in
                 fp32 on all host threads (``oracle/spconv_oracle.py``), on the same workload.
* ``cfg5``       beside the headline: one training step of the MinkUNet-style stack
                 (``fgms_b200.unet``, 25 layers, fp16), one ~120 k-voxel scene per rank, with the
                 bucketed weight-gradient all-reduce overlapped with the backward when N > 1.

* ``output_stationary``  (N = 1) the forward that writes every output row once, beside the scatter form.

With N > 1 (torchrun, one rank per GPU) every rank holds its own scene of the same kind (weak
scaling, data parallel); the weight-gradient partial sums are exchanged inside the timed step — by
the library's peer-memory kernel beside the input-gradient kernel, the whole step replayed from one
CUDA graph (``--transport nccl``: one NCCL all-reduce, eager launches) — and the exchanged result
is checked on the GPUs after the timed loop (``multi_gpu_check``).  A rendezvous kernel after the
untimed L2 flush starts every rank's timed step together.  Beside it ONE scene is cut over the ranks
by output-row range (forward) / input-row range (dgrad) and that step is reported as
``strong_scaling`` (``--shard scenes`` skips it).  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "spconv fwd+bwd effective TFLOPS (6*pairs*c_in*c_out / time), one layer"
UNIT = "TFLOPS"

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the named pass on the named workload, from
# ncu captures of this benchmark's own command; reported only for exactly that pass and workload.
NCU_TRAFFIC = {
    ("fwd", "cfg4"): 79.5e6, ("dgrad", "cfg4"): 79.3e6, ("wgrad", "cfg4"): 81.7e6,
    ("fwd", "cfg2"): 33.5e6, ("dgrad", "cfg2"): 33.5e6, ("wgrad", "cfg2"): 33.5e6,
    ("fwd", "cfg5l0"): 24.6e6, ("dgrad", "cfg5l0"): 24.6e6, ("wgrad", "cfg5l0"): 24.6e6,
}


def load_peaks():
    """(HBM GB/s, dense 16-bit tensor TFLOPS, source).  tf32 runs at half the 16-bit tensor rate."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


def tensor_peak_tflops(mode: str, f16_peak: float):
    """Peak of the arithmetic a mode runs on: fp16 = the measured dense 16-bit figure, tf32 = half of it (the
    tensor cores' tf32 rate), fp32 = the CUDA cores' FFMA rate (148 SMs x 128 lanes x 2 flop x 1.965 GHz)."""
    return {"fp16": f16_peak, "tf32": f16_peak / 2, "fp32": 148 * 128 * 2 * 1.965e9 / 1e12}[mode]


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU (NVML, read-only) while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index, self.mhz, self.mask, self.max_mhz = index, [], 0, None
        self._stop, self._thread, self._nvml, self._h = threading.Event(), None, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.mhz.append(float(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                self.mask |= int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
            except Exception:
                pass
            self._stop.wait(0.005)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        reasons = [n for n, bit in self.REASONS.items() if self.mask & bit]
        return {"sm_mhz": statistics.median(self.mhz) if self.mhz else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.mhz)}


def cpu_step(wl, threads: int):
    """One forward + backward of the workload on the host (fp32, all threads); returns seconds."""
    import numpy as np
    import torch
    from fgms_b200 import clouds
    from oracle import spconv_oracle as orc
    torch.set_num_threads(threads)
    km = wl.kmap
    f, w, g = clouds.make_tensors(km.n_in, km.n_out, wl.c_in, wl.c_out, km.k_vol, wl.seed, np.float32)
    t0 = time.perf_counter()
    orc.fwd(f, w, km.n_out, km.kpos, km.imap, km.omap, acc=torch.float32)
    orc.dgrad(g, w, km.n_in, km.kpos, km.imap, km.omap, acc=torch.float32)
    orc.wgrad(f, g, km.k_vol, km.kpos, km.imap, km.omap, acc=torch.float32)
    return time.perf_counter() - t0


def cpu_literal_cfg1():
    """The reference's own nested loops (cpu-check.py:16-44, cpu-check-back.py:16-44) timed on cfg1, the one
    configuration they can finish: the C restatement of the loops on the whole layer, and the Python form on
    the first 300 pairs scaled to the layer's pair count."""
    import numpy as np
    from fgms_b200 import clouds, workloads
    from oracle import c_oracle
    from oracle import spconv_oracle as orc
    wl = workloads.get("cfg1")
    km = wl.kmap
    f, w, g = clouds.make_tensors(km.n_in, km.n_out, wl.c_in, wl.c_out, km.k_vol, wl.seed, np.float32)
    c_oracle.fwd(f, w, km.n_out, km.knnz, km.imap, km.omap, acc="f32")
    t0 = time.perf_counter()
    c_oracle.fwd(f, w, km.n_out, km.knnz, km.imap, km.omap, acc="f32")
    c_oracle.bwd(g, w, f, km.n_in, km.knnz, km.imap, km.omap, acc="f32")
    c_ms = (time.perf_counter() - t0) * 1e3
    sample = 300
    knnz = np.zeros_like(km.knnz)
    knnz[0] = sample  # the loops only count pairs per offset; which offset they sit in does not change the work
    t0 = time.perf_counter()
    orc.fwd_literal(f, w, km.n_out, knnz, km.imap, km.omap, False)
    orc.bwd_literal(g, w, f, km.n_in, knnz, km.imap, km.omap)
    py_ms = (time.perf_counter() - t0) * 1e3 * km.pairs / sample
    return {"workload": "cfg1 (8000 voxels, 14040 pairs, fp32 16->16), fwd + dgrad + wgrad", "cores": 1,
            "c_loops_ms": c_ms, "python_loops_ms_extrapolated": py_ms,
            "sample": f"C: whole layer; Python: first {sample} pairs, scaled by pairs / {sample}"}


def workload_config(wl, gpus, shard):
    """Identical in both arms for one command line: what is computed, not how it is timed."""
    km = wl.kmap
    if gpus == 1:
        par = "single GPU"
    else:
        par = f"dp{gpus} (one scene per GPU, wgrad all-reduce)"
    return {"workload": f"{wl.name}: {wl.description}", "n_in": km.n_in, "n_out": km.n_out, "pairs": km.pairs,
            "k_vol": km.k_vol, "c_in": wl.c_in, "c_out": wl.c_out, "math": wl.mode, "seed": wl.seed, "parallelism": par}


def run_reference(args):
    """The reference's CPU path timed on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from fgms_b200 import workloads
    wl = workloads.get(args.workload)
    threads = os.cpu_count() or 1
    flops = workloads.flops(wl)
    for _ in range(args.warmup):
        cpu_step(wl, threads)
    times = [cpu_step(wl, threads) for _ in range(args.steps)]
    t = statistics.mean(times)
    val = flops / t / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(wl, args.gpus, args.shard),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"whole {wl.name} layer, fwd+dgrad+wgrad, per step; mean of {len(times)} steps"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "timing": "host wall clock around each step, inputs in host memory",
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# cfg5: the encoder-decoder stack
# ---------------------------------------------------------------------------------------------
def run_cfg5(args, dev, rank, world, flush):
    """One training step of the stack per timed step; one scene per rank.  Returns rank 0's report (None elsewhere)."""
    import torch
    import torch.distributed as dist
    from fgms_b200 import backend, unet, workloads

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def build(scenes, first):
        wl = workloads.unet_workload(scenes=scenes, first_scene=first)
        spec = unet.minkunet_spec(wl.c_in, wl.widths)
        umaps = unet.build_unet_maps(torch.from_numpy(wl.coords).to(dev))
        weights = unet.unet_weights(spec, umaps, wl.seed)
        feats, grad_out = torch.from_numpy(wl.feats).to(dev), torch.from_numpy(wl.grad_out).to(dev)
        return wl, spec, umaps, weights, feats, grad_out

    def time_steps(run, steps, warm):
        for _ in range(warm):
            flush(); run()
        barrier()
        evs = []
        for _ in range(steps):
            flush()
            a, b = ev(), ev()
            a.record(); run(); b.record()
            evs.append((a, b))
        barrier()
        return sum(a.elapsed_time(b) for a, b in evs)

    steps = max(3, min(args.steps, args.cfg5_steps))
    wl, spec, umaps, weights, feats, grad_out = build(1, rank)
    stack_transport = "nccl" if args.transport == "auto" else args.transport
    step = unet.UNetStep(spec, umaps, weights, feats, grad_out, transport=stack_transport)
    flops_local = unet.step_flops(spec, umaps)
    run = step.run
    graph = None
    if world == 1 and args.graph:
        # no collective in the single-rank step: capture its launches once, replay them
        for _ in range(2):
            step.run()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step.run()
            graph, run = g, g.replay
        except Exception as exc:
            sys.stderr.write(f"bench: cfg5 CUDA graph capture failed ({exc!r}); timing eager launches\n")
            torch.cuda.synchronize()
    # Several ranks: the step with NCCL buckets is launched eagerly (74 kernels + the collectives from Python).  The
    # same step with the library's own exchange kernel on the buckets can be replayed from one CUDA graph, which
    # takes the host out of it; a short trial (max over ranks) decides which form is timed.
    trial_ms = None
    if world > 1 and args.graph and args.transport == "auto":
        peer_step = None
        try:
            peer_step = unet.UNetStep(spec, umaps, weights, feats, grad_out, transport="peer")
            for _ in range(2):
                peer_step.run()
        except Exception as exc:
            sys.stderr.write(f"bench: rank {rank}: cfg5 with peer-mapped buckets unavailable ({exc!r})\n")
            peer_step = None
        barrier()
        agreed = torch.tensor([1.0 if peer_step is not None else 0.0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        g = None
        if agreed.item() >= 1:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    peer_step.run()
            except Exception as exc:
                sys.stderr.write(f"bench: rank {rank}: cfg5 graph capture failed ({exc!r})\n")
                g = None
                torch.cuda.synchronize()
            agreed = torch.tensor([1.0 if g is not None else 0.0], device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if agreed.item() >= 1:
                def trial(fn):
                    t = torch.tensor([time_steps(fn, 5, 2) / 5], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                    return float(t.item())
                trial_ms = {"nccl_buckets_eager": trial(step.run), "peer_buckets_graph_replay": trial(g.replay)}
                if trial_ms["peer_buckets_graph_replay"] < 0.98 * trial_ms["nccl_buckets_eager"]:
                    step, run, graph, stack_transport = peer_step, g.replay, g, "peer"
        if graph is None:
            del peer_step, g
    total_ms = time_steps(run, steps, 3)
    report = {"what": wl.description, "layers": len(spec), "steps": steps,
              "launch": "CUDA-graph replay" if graph is not None else "eager launches",
              "kernels_per_step": step.launches_per_step}

    check = None
    exposed_ms = None
    if world > 1:
        # the same step without the collectives: what the all-reduces add to the step is their exposed time
        alone = unet.UNetStep(spec, umaps, weights, feats, grad_out, exchange=False)
        alone_ms = time_steps(alone.run, steps, 2)
        # result check: the all-reduced gradient equals the sum of the ranks' own gradients
        step.run(); alone.run()
        torch.cuda.synchronize()
        mine = alone.w_grad.float()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ref = torch.stack(parts).sum(0)
        scale = float(ref.abs().max())
        werr = float((step.w_grad.float() - ref).abs().max()) / max(scale, 1e-30)
        oerr = float((step.val[spec[-1].dst].float() - alone.val[spec[-1].dst].float()).abs().max())
        check = {"wgrad_rel_err": werr, "out_abs_diff_vs_single_rank": oerr, "ok": bool(werr <= 1e-2)}

    stats = torch.tensor([total_ms, flops_local, (alone_ms if world > 1 else 0.0), float(umaps.voxels[0])],
                         dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, flops_all, alone_ms = float(mx[0]), float(sm[1]), float(mx[2])
        exposed_ms = (total_ms - alone_ms) / steps
        oks = torch.tensor([1.0 if check["ok"] else 0.0], device=dev)
        dist.all_reduce(oks, op=dist.ReduceOp.MIN)
        check["ok"] = bool(oks.item() > 0)
    else:
        flops_all = flops_local
    if not rank == 0:
        return None, check
    report.update({"ms_per_step": total_ms / steps, "value": flops_all * steps / (total_ms * 1e-3) / 1e12, "unit": UNIT,
                   "scaling": "weak (one scene per rank)", "voxels_per_level": umaps.voxels,
                   "flops_per_step_all_ranks": flops_all})
    if world > 1:
        report["allreduce"] = {"transport": stack_transport, "buckets": len(step.buckets), "bytes_fp32": int(step.w_grad.numel() * 4),
                               "exposed_ms_per_step": exposed_ms, "kernels_only_ms_per_step": alone_ms / steps,
                               "kernels_only": "the same step without the exchange, eager launches",
                               **({"trial_ms_per_step": trial_ms} if trial_ms else {})}
        report["multi_gpu_check"] = check
    else:
        # per-layer table and the roofline of the slowest call (eager launches with events around every call)
        hbm, f16_peak, _ = load_peaks()
        rows = step.profile(reps=5, flush=flush)
        by_name = {l.name: (l, step.run_spec[i]) for i, l in enumerate(spec)}
        table, worst = [], None
        for r in rows:
            l, run_l = by_name[r["layer"]]  # as specified (flops and bytes count the real channels) and as run
            pairs = int(umaps.of(l).pairs)
            b = workloads.layer_bytes(pairs, l.c_in, l.c_out, l.k_vol, 2, r["pass"])
            fl = 2.0 * pairs * l.c_in * l.c_out
            t_roof = max(b / (hbm * 1e9), fl / (f16_peak * 1e12)) * 1e3
            fam = backend.kernel_family(r["pass"], run_l.c_in, run_l.c_out, torch.float16, True, l.k_vol)
            row = {"layer": l.name, "pass": r["pass"], "shape": f"{l.c_in}->{l.c_out} k{l.k_vol}", "pairs": pairs,
                   "ms": round(r["ms"], 5), "frac": round(t_roof / r["ms"], 4), "family": fam}
            table.append(row)
            if worst is None or r["ms"] > worst[0]["ms"]:
                worst = (row, b)
        report["per_call"] = table
        report["sum_of_calls_ms"] = sum(r["ms"] for r in rows)
        w, b = worst
        report["slowest_call"] = {"layer": w["layer"], "pass": w["pass"], "shape": w["shape"], "ms": w["ms"],
                                  "achieved_gbs": b / (w["ms"] * 1e-3) / 1e9, "peak_gbs": hbm, "frac": w["frac"]}
        del step, graph
        # the whole batch of 8 scenes on this one GPU (what the single-GPU case of the configuration is)
        try:
            wl8, spec8, umaps8, weights8, feats8, grad8 = build(8, 0)
            step8 = unet.UNetStep(spec8, umaps8, weights8, feats8, grad8)
            run8 = step8.run
            if args.graph:
                for _ in range(2):
                    step8.run()
                torch.cuda.synchronize()
                g8 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g8):
                    step8.run()
                run8 = g8.replay
            n8 = max(3, steps // 2)
            ms8 = time_steps(run8, n8, 2)
            report["batch8_one_gpu"] = {"voxels_per_level": umaps8.voxels, "ms_per_step": ms8 / n8,
                                        "value": unet.step_flops(spec8, umaps8) * n8 / (ms8 * 1e-3) / 1e12, "unit": UNIT}
        except Exception as exc:  # reported, not fatal: the headline does not depend on it
            report["batch8_one_gpu"] = {"error": repr(exc)}
    return report, check


# ---------------------------------------------------------------------------------------------
# one scene cut over the ranks by row range
# ---------------------------------------------------------------------------------------------
def run_row_shard(args, dev, rank, world, wl, p, flush):
    """Forward on this rank's output-row range, dgrad on its input-row range, wgrad on the forward cut's pairs with
    the partial sums all-reduced.  The maps are cut on the device (``dist.shard_map_device``).  Checks that rows
    outside the rank's range stay exactly zero and that the gathered result matches the uncut run."""
    import torch
    import torch.distributed as dist
    from fgms_b200 import backend
    from fgms_b200 import dist as fdist

    ev = lambda: torch.cuda.Event(enable_timing=True)
    km = wl.kmap
    out_cut = fdist.shard_map_device(p.kpos, p.imap, p.omap, km.n_out, rank, world, by="out")
    in_cut = fdist.shard_map_device(p.kpos, p.imap, p.omap, km.n_in, rank, world, by="in")
    out = torch.zeros((km.n_out, wl.c_out), dtype=p.dtype, device=dev)
    in_grad = torch.zeros((km.n_in, wl.c_in), dtype=p.dtype, device=dev)
    w_grad = torch.zeros_like(p.weights)
    part = torch.zeros(p.weights.numel(), dtype=torch.float32, device=dev)

    def step():
        backend.fgms_fusion_fwd_cuda(p.feats, p.weights, 0, out, out_cut.kpos, None, out_cut.imap, out_cut.omap, False, p.arch80)
        if p.dtype == torch.float16:
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, out_cut.kpos, out_cut.imap, out_cut.omap, p.arch80,
                                    workspace=part, accumulate=False)
        else:
            part.zero_()
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, part.view_as(w_grad), out_cut.kpos, out_cut.imap, out_cut.omap, p.arch80)
        work = dist.all_reduce(part, async_op=True)
        backend.fgms_dgrad_cuda(p.grad_out, p.weights, in_grad, in_cut.kpos, in_cut.imap, in_cut.omap, p.arch80)
        work.wait()
        if p.dtype == torch.float16:
            backend.wgrad_finalize(w_grad, part)
        else:
            w_grad.add_(part.view_as(w_grad))

    def prepare():
        out.zero_(); in_grad.zero_(); w_grad.zero_(); flush()

    for _ in range(args.warmup):
        prepare(); step()
    dist.barrier(); torch.cuda.synchronize()
    evs = []
    steps = min(args.steps, 100)
    for _ in range(steps):
        prepare()
        a, b = ev(), ev()
        a.record(); step(); b.record()
        evs.append((a, b))
    dist.barrier(); torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in evs) / steps
    # ---- checks
    prepare(); step(); torch.cuda.synchronize()
    lo, hi = out_cut.row_range
    outside_zero = bool((out[:lo] == 0).all() and (out[hi:] == 0).all())
    ilo, ihi = in_cut.row_range
    outside_zero = outside_zero and bool((in_grad[:ilo] == 0).all() and (in_grad[ihi:] == 0).all())
    full_out = out.clone(); dist.all_reduce(full_out)          # the ranges are disjoint: the sum is the concatenation
    full_in = in_grad.clone(); dist.all_reduce(full_in)
    ref_out = torch.zeros_like(out); ref_in = torch.zeros_like(in_grad); ref_w = torch.zeros_like(w_grad)
    backend.fgms_fusion_fwd_cuda(p.feats, p.weights, 0, ref_out, p.kpos, None, p.imap, p.omap, False, p.arch80)
    backend.fgms_bwd_cuda(p.grad_out, p.feats, p.weights, 0, ref_in, ref_w, p.kpos, None, p.imap, p.omap, False, p.arch80)
    rel = lambda a, b: float((a.float() - b.float()).abs().max()) / max(float(b.float().abs().max()), 1e-30)
    errs = {"out": rel(full_out, ref_out), "in_grad": rel(full_in, ref_in), "w_grad": rel(w_grad, ref_w)}
    pairs_local = torch.tensor([float(out_cut.imap.numel()), float(in_cut.imap.numel()), ms], dtype=torch.float64, device=dev)
    gathered = [torch.empty_like(pairs_local) for _ in range(world)]
    dist.all_gather(gathered, pairs_local)
    ok = outside_zero and max(errs.values()) <= 1e-2
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ms_max = max(float(g[2]) for g in gathered)
    return {"mode": "one scene, forward by output-row range, dgrad by input-row range, wgrad partial sums all-reduced",
            "ms_per_step": ms_max, "value": 6.0 * km.pairs * wl.c_in * wl.c_out / (ms_max * 1e-3) / 1e12, "unit": UNIT,
            "pairs_per_rank_fwd": [int(g[0]) for g in gathered], "pairs_per_rank_dgrad": [int(g[1]) for g in gathered],
            "rows_outside_own_range_zero": outside_zero, "rel_err_vs_uncut": errs, "ok": bool(flag.item() > 0)}


def run_reference_cuda(wl, p, prepare, ev):
    """The reference's CUDA extension (built from its two source files for sm_100a by ``oracle/build_ref.py``) timed on
    this workload's tensors with the same events and L2 flush.  Only fp16 layers whose channel counts are multiples of
    32 and whose output width is not 64 are run: the reference's other kernels for the benchmark shapes read or write
    out of range (see the header of tests/test_gpu_reference_cuda.py)."""
    import torch
    from oracle import build_ref
    if not build_ref.available():
        return {"unavailable": "the reference extension is not built (python -m oracle.build_ref needs a checkout of the reference)"}
    if not (wl.mode == "fp16" and wl.c_in % 32 == 0 and wl.c_out % 32 == 0 and wl.c_out != 64 and wl.c_in > 16):
        return {"unavailable": f"the reference's kernels for {wl.mode} {wl.c_in}->{wl.c_out} are not sound; not launched"}
    ref = build_ref.load()
    km = wl.kmap
    out = torch.zeros((km.n_out, wl.c_out), dtype=p.dtype, device=p.feats.device)
    in_grad = torch.zeros((km.n_in, wl.c_in), dtype=p.dtype, device=p.feats.device)
    w_grad = torch.zeros_like(p.weights)

    def step():
        ref.fgms_fusion_fwd_cuda(p.feats, p.weights, p.qsum, out, p.kpos, p.qkpos, p.imap, p.omap, False, True)
        ref.fgms_bwd_cuda(p.grad_out, p.feats, p.weights, p.qsum, in_grad, w_grad, p.kpos, p.qkpos, p.imap, p.omap, False, True)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    fwd_ms, step_ms = [], []
    for _ in range(20):
        prepare(); out.zero_(); in_grad.zero_(); w_grad.zero_()
        a, b, c = ev(), ev(), ev()
        a.record()
        ref.fgms_fusion_fwd_cuda(p.feats, p.weights, p.qsum, out, p.kpos, p.qkpos, p.imap, p.omap, False, True)
        b.record()
        ref.fgms_bwd_cuda(p.grad_out, p.feats, p.weights, p.qsum, in_grad, w_grad, p.kpos, p.qkpos, p.imap, p.omap, False, True)
        c.record()
        torch.cuda.synchronize()
        fwd_ms.append(a.elapsed_time(b)); step_ms.append(a.elapsed_time(c))
    fm, sm = statistics.mean(fwd_ms), statistics.mean(step_ms)
    from fgms_b200 import workloads
    return {"what": "hkeee21/FGMS CUDA extension compiled for sm_100a (wmma kernels), same tensors, events and L2 flush; "
                    "fused forward + backward (dgrad + wgrad) through its own Python functions",
            "fwd_ms": fm, "bwd_ms": sm - fm, "step_ms": sm, "value": workloads.flops(wl) / (sm * 1e-3) / 1e12, "unit": UNIT}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from fgms_b200 import backend, workloads
    from fgms_b200.dist import BoundSceneLayer, SceneParallelLayer

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # the weight-gradient all-reduces are small and latency-bound; on 8-GPU B200 boxes they were measured
        # faster without NVLink-switch reductions (30.8 vs 46.0 us back to back for 1.8 MB)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    shard_rows = args.shard != "scenes" and world > 1
    wl = workloads.get(args.workload, seed_offset=1000 * rank)
    km = wl.kmap
    p = workloads.LayerTensors(km, wl.c_in, wl.c_out, wl.seed, wl.mode, device=dev)
    layer = SceneParallelLayer(p.kpos, p.imap, p.omap, p.qsum, p.arch80)
    out = torch.zeros((km.n_out, wl.c_out), dtype=p.dtype, device=dev)
    in_grad = torch.zeros((km.n_in, wl.c_in), dtype=p.dtype, device=dev)
    w_grad = torch.zeros_like(p.weights)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    flush = lambda: flush_buf.fill_(1)  # evict L2 (126 MB) so that every step starts cold

    # With several ranks and peer-mapped buffers, a rendezvous kernel (the exchange kernel with nothing to sum)
    # follows the untimed L2 flush, so that every rank's timed step starts together: without it a rank whose
    # flush ends early spends the difference waiting in its exchange, inside its timed interval.
    aligner = [None]

    def prepare():
        out.zero_(); in_grad.zero_(); w_grad.zero_()
        flush()
        if aligner[0] is not None:
            aligner[0].run()

    ev = lambda: torch.cuda.Event(enable_timing=True)
    pass_ms = {"fwd": [], "dgrad": [], "wgrad": []}

    layer_transport = "peer" if args.transport == "auto" else args.transport
    bound = None
    if world > 1:
        make = lambda tr: BoundSceneLayer(p.feats, p.weights, p.grad_out, out, in_grad, w_grad, p.kpos, p.imap, p.omap,
                                          p.arch80, transport=tr)
        if layer_transport == "peer":
            # peer-mapped buffers need the symmetric-memory allocator and peer access between the GPUs; where a rank
            # cannot get them, all ranks agree to use NCCL instead
            try:
                bound = make("peer")
            except Exception as exc:
                sys.stderr.write(f"bench: rank {rank}: peer-mapped buffers unavailable ({exc!r})\n")
            agreed = torch.tensor([1.0 if bound is not None else 0.0], device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if agreed.item() < 1:
                layer_transport, bound = "nccl", None
        if bound is None:
            bound = make(layer_transport)
    if world > 1 and layer_transport == "peer" and args.align:
        from fgms_b200.dist import PeerExchange
        aligner[0] = PeerExchange(0, dev, ctas=1)
    bound_alone = BoundSceneLayer(p.feats, p.weights, p.grad_out, out, in_grad, w_grad, p.kpos, p.imap, p.omap, p.arch80,
                                  exchange=False) if world > 1 else None
    ws = backend.wgrad_workspace(wl.c_in, wl.c_out, km.k_vol, dev) if p.dtype == torch.float16 else None
    part32 = torch.zeros_like(w_grad) if p.dtype != torch.float16 else None

    def wgrad_kernel_only():
        """The weight-gradient kernel of this step's form, without the collective (for the per-pass times)."""
        if p.dtype == torch.float16 and world == 1:
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, p.kpos, p.imap, p.omap, p.arch80)
        elif p.dtype == torch.float16:
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, p.kpos, p.imap, p.omap, p.arch80, workspace=ws, accumulate=False)
        else:
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, part32 if world > 1 else w_grad, p.kpos, p.imap, p.omap, p.arch80)

    def step(record, which=bound):
        """One fwd + dgrad + wgrad; nothing between the launches.  record: events around the step."""
        e = [ev(), ev()] if record else None
        if record: e[0].record()
        if world > 1:
            # data parallel: the step bound to its buffers (no per-call argument checks on the host); wgrad first,
            # its all-reduce runs beside dgrad
            which.forward()
            which.backward()
        else:
            layer.forward(p.feats, p.weights, out)
            backend.fgms_dgrad_cuda(p.grad_out, p.weights, in_grad, p.kpos, p.imap, p.omap, p.arch80)
            wgrad_kernel_only()
        if record: e[1].record()
        return e

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------------------
    for _ in range(args.warmup):
        prepare(); step(False)
    barrier()
    # The launches are captured once into a CUDA graph and replayed, which takes the host out of the step; the
    # kernels, their order and their arguments are those of the eager step.  --no-graph times the eager step.
    # With several ranks this holds for the peer-memory exchange (the library's own kernel, which numbers its
    # calls on the device); a step with an NCCL collective in it stays eager.  Nothing is outstanding on the
    # process group when the capture starts (barrier + synchronize above), and the capture is thread-local, so
    # that a CUDA call of another thread of the process cannot invalidate it.
    graph = None
    launches_per_step = None
    if args.graph and (world == 1 or layer_transport == "peer"):
        try:
            c0 = backend.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                step(False)
            launches_per_step = backend.launch_count() - c0
            graph = g
            for _ in range(3):
                prepare(); graph.replay()
            barrier()
        except Exception as exc:  # capture not possible: time the eager step
            sys.stderr.write(f"bench: CUDA graph capture failed ({exc!r}); timing the eager step\n")
            graph = None
            torch.cuda.synchronize()

    # Several ranks: a short trial of both forms (max over ranks, so every rank decides alike); the timed region
    # below uses the faster one.  Replayed graphs take the host out of the step but give the device no say in
    # when the exchange's side branch starts; which form wins depends on the number of ranks.
    trial_ms = None
    if world > 1 and args.graph and layer_transport == "peer":
        captured = torch.tensor([1.0 if graph is not None else 0.0], device=dev)
        dist.all_reduce(captured, op=dist.ReduceOp.MIN)
        if captured.item() < 1:
            graph = None
    if graph is not None and world > 1:
        def trial(use_graph, n=10):
            evs = []
            for _ in range(n):
                prepare()
                e = [ev(), ev()]
                e[0].record()
                graph.replay() if use_graph else step(False)
                e[1].record()
                evs.append(e)
            barrier()
            t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs) / n], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        trial_ms = {"graph_replay": trial(True), "eager": trial(False)}
        if trial_ms["eager"] < 0.98 * trial_ms["graph_replay"]:
            graph = None

    def timed_step():
        if graph is None:
            return step(True)
        e = [ev(), ev()]
        e[0].record(); graph.replay(); e[1].record()
        return e

    launches0 = backend.launch_count()
    fallbacks0 = backend.fallback_count()
    events = []
    with ClockSampler(local) as clocks:
        for _ in range(args.steps):
            prepare()
            events.append(timed_step())
        barrier()
    launches = (backend.launch_count() - launches0) if graph is None else launches_per_step * args.steps
    total_ms = sum(e[0].elapsed_time(e[1]) for e in events)

    # the same step without the collective (N > 1): the difference is the all-reduce's exposed time
    alone_ms = 0.0
    if world > 1:
        evs = []
        for _ in range(min(args.steps, 50)):
            prepare()
            evs.append(step(True, bound_alone))
        barrier()
        alone_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)

    # per-pass durations (for the roofline of the slowest pass): the step's three kernels in the step's order with an
    # event between them.  The host enqueues the three calls while the untimed flush (about 140 us of device time)
    # still runs, so no launch gap falls between the events.
    pe = []
    for _ in range(min(args.steps, 50)):
        prepare()
        e = [ev() for _ in range(4)]
        e[0].record()
        layer.forward(p.feats, p.weights, out)
        e[1].record()
        backend.fgms_dgrad_cuda(p.grad_out, p.weights, in_grad, p.kpos, p.imap, p.omap, p.arch80)
        e[2].record()
        wgrad_kernel_only()
        e[3].record()
        pe.append(e)
    barrier()
    for e in pe:
        pass_ms["fwd"].append(e[0].elapsed_time(e[1]))
        pass_ms["dgrad"].append(e[1].elapsed_time(e[2]))
        pass_ms["wgrad"].append(e[2].elapsed_time(e[3]))

    # ---- the output-stationary forward beside the scatter form (one rank, tensor-core shapes) ----------------
    out_stationary = None
    if world == 1 and backend.kernel_family("fwd", wl.c_in, wl.c_out, p.dtype, p.arch80, km.k_vol) == "tcgen05":
        tb = [ev(), ev()]
        tb[0].record()
        nbr = backend.build_neighbor_table(p.kpos, p.imap, p.omap, km.n_in, km.n_out)
        tb[1].record()
        os_out = torch.empty_like(out)
        for _ in range(3):
            backend.fgms_fwd_os_cuda(p.feats, p.weights, os_out, nbr, p.arch80)
        oe = []
        for _ in range(min(args.steps, 20)):
            flush()
            e = [ev(), ev()]
            e[0].record()
            backend.fgms_fwd_os_cuda(p.feats, p.weights, os_out, nbr, p.arch80)
            e[1].record()
            oe.append(e)
        torch.cuda.synchronize()
        first = os_out.clone()
        backend.fgms_fwd_os_cuda(p.feats, p.weights, os_out, nbr, p.arch80)
        out.zero_()
        layer.forward(p.feats, p.weights, out)
        torch.cuda.synchronize()
        n_tiles = (km.n_out + 127) // 128
        out_stationary = {
            "what": "forward with one accumulator per output row over all offsets, each row written once (no atomics, "
                    "bias / ReLU fusable); one 128-row stage per (128 output rows, offset) whatever the number of pairs in it",
            "fwd_ms": statistics.mean(a.elapsed_time(b) for a, b in oe),
            "scatter_fwd_ms": statistics.mean(pass_ms["fwd"]),
            "stages": n_tiles * km.k_vol, "scatter_stages": (km.pairs + 127) // 128,
            "table_build_ms": tb[0].elapsed_time(tb[1]),
            "same_bits_on_a_second_run": bool(torch.equal(first, os_out)),
            "max_abs_diff_vs_scatter_form": float((os_out.float() - out.float()).abs().max()),
        }
        del nbr, os_out, first

    # warm-L2 variant (no flush), reported beside the headline
    for _ in range(2):
        out.zero_(); in_grad.zero_(); w_grad.zero_(); step(False)
    barrier()
    warm = []
    for _ in range(args.steps):
        out.zero_(); in_grad.zero_(); w_grad.zero_()
        warm.append(timed_step())
    barrier()
    warm_ms = sum(e[0].elapsed_time(e[1]) for e in warm)

    # ---- multi-GPU result check: the exchanged weight gradient is the sum of the ranks' own sums ----------
    check = None
    if world > 1:
        out.zero_(); in_grad.zero_(); w_grad.zero_()
        if graph is not None:
            graph.replay()   # the timed form of the step is the one that is checked
        else:
            bound.forward(); bound.backward()
        torch.cuda.synchronize()
        got_w, got_out, got_in = w_grad.clone(), out.clone(), in_grad.clone()
        if p.dtype == torch.float16:
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, p.kpos, p.imap, p.omap, p.arch80, workspace=ws, accumulate=False)
            mine = ws[: w_grad.numel()].clone()
        else:
            mine = torch.zeros_like(w_grad)
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, mine, p.kpos, p.imap, p.omap, p.arch80)
            mine = mine.flatten()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ref_w = torch.stack(parts).sum(0)
        ref_out = torch.zeros_like(out); ref_in = torch.zeros_like(in_grad)
        layer.forward(p.feats, p.weights, ref_out)
        backend.fgms_dgrad_cuda(p.grad_out, p.weights, ref_in, p.kpos, p.imap, p.omap, p.arch80)
        rel = lambda a, b: float((a.float().flatten() - b.float().flatten()).abs().max()) / max(float(b.float().abs().max()), 1e-30)
        check = {"wgrad_rel_err": rel(got_w, ref_w), "out_rel_err": rel(got_out, ref_out), "in_grad_rel_err": rel(got_in, ref_in)}
        # waits that ran out, map entries skipped, kpos entries clamped since the process started (this rank's count;
        # `ok` below covers every rank's)
        check["device_problems"] = int(backend.device_status(reset=False))
        ok = max(check["wgrad_rel_err"], check["out_rel_err"], check["in_grad_rel_err"]) <= 1e-2 and check["device_problems"] == 0
        flag = torch.tensor([1.0 if ok else 0.0], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        check["ok"] = bool(flag.item() > 0)
        check["what"] = "all-reduced w_grad vs the sum of every rank's own fp32 sums (all_gather); out / in_grad vs the single-rank entry points"

    # ---- where the peer exchange sits in the step (eager steps, events on both streams) -----------------------
    timeline = None
    if world > 1 and bound.px is not None:
        rows = []
        inner = bound.px.run
        for it in range(15):
            prepare()
            t0, t1, x0, x1 = ev(), ev(), ev(), ev()

            def timed_run(stream=None, *a, _x0=x0, _x1=x1):
                _x0.record(stream); inner(stream, *a); _x1.record(stream)

            bound.px.run = timed_run
            t0.record(); bound.forward(); bound.backward(); t1.record()
            bound.px.run = inner
            barrier()
            if it >= 5:
                rows.append((t0.elapsed_time(x0), t0.elapsed_time(x1), t0.elapsed_time(t1)))
        m = [statistics.mean(c) * 1e3 for c in zip(*rows)]
        timeline = {"what": "eager step of this rank, microseconds after the step's first kernel starts; the exchange is enqueued on "
                            "its side stream when the weight-gradient kernel has finished, the input-gradient kernel runs beside it",
                    "exchange_starts_us": m[0], "exchange_ends_us": m[1], "step_ends_us": m[2]}

    # ---- end to end with host buffers ----------------------------------------------------------
    # Three streams and two sets of device / host buffers: the upload of step i + 1 and the download of
    # step i - 1 run beside the kernels of step i.  Every step still uploads all its inputs from pinned
    # host memory and downloads all three results inside the timed region.
    pin = lambda t: t.cpu().pin_memory()
    h_in = {k: pin(v) for k, v in dict(feats=p.feats, weights=p.weights, grad_out=p.grad_out, kpos=p.kpos,
                                       imap=p.imap, omap=p.omap).items()}
    d_in = [{k: torch.empty_like(v, device=dev) for k, v in h_in.items()} for _ in range(2)]
    d_out = [dict(out=torch.empty_like(out), in_grad=torch.empty_like(in_grad), w_grad=torch.empty_like(w_grad)) for _ in range(2)]
    h_out = [{k: torch.empty_like(v, device="cpu").pin_memory() for k, v in d_out[0].items()} for _ in range(2)]
    h2d = sum(v.numel() * v.element_size() for v in h_in.values())
    d2h = sum(v.numel() * v.element_size() for v in h_out[0].values())
    s_up, s_run, s_down = (torch.cuda.Stream(device=dev) for _ in range(3))
    ev_up = [ev() for _ in range(2)]; ev_run = [ev() for _ in range(2)]; ev_down = [ev() for _ in range(2)]

    def e2e_step(i):
        b = i & 1
        with torch.cuda.stream(s_up):
            if i >= 2: s_up.wait_event(ev_run[b])        # the kernels of step i - 2 have read these inputs
            for k in h_in:
                d_in[b][k].copy_(h_in[k], non_blocking=True)
            ev_up[b].record(s_up)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_up[b])
            if i >= 2: s_run.wait_event(ev_down[b])      # the results of step i - 2 have left the device
            di, do = d_in[b], d_out[b]
            do["out"].zero_(); do["in_grad"].zero_(); do["w_grad"].zero_()
            backend.fgms_fusion_fwd_cuda(di["feats"], di["weights"], p.qsum, do["out"], di["kpos"], None, di["imap"],
                                         di["omap"], False, p.arch80)
            lay = SceneParallelLayer(di["kpos"], di["imap"], di["omap"], p.qsum, p.arch80)
            lay.backward(di["grad_out"], di["feats"], di["weights"], do["in_grad"], do["w_grad"])
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_down):
            s_down.wait_event(ev_run[b])
            for k in h_out[b]:
                h_out[b][k].copy_(d_out[b][k], non_blocking=True)
            ev_down[b].record(s_down)

    e2e_steps = min(args.steps, 100)
    for i in range(max(2, args.warmup // 2) * 2):
        e2e_step(i)
    barrier()
    e2e_t0, e2e_t1 = ev(), [ev() for _ in range(3)]
    e2e_t0.record(s_up)
    s_run.wait_event(e2e_t0); s_down.wait_event(e2e_t0)
    for i in range(e2e_steps):
        e2e_step(i)
    for e, st in zip(e2e_t1, (s_up, s_run, s_down)):
        e.record(st)
    barrier()
    e2e_ms = max(e2e_t0.elapsed_time(e) for e in e2e_t1) / e2e_steps
    # the last step's results, downloaded through the same path, must match the device-resident run
    # (fp16 reds arrive in a different order every run, so the comparison allows rounding differences)
    out.zero_(); layer.forward(p.feats, p.weights, out); torch.cuda.synchronize()
    if not torch.allclose(h_out[(e2e_steps - 1) & 1]["out"].float(), out.cpu().float(), rtol=2e-2, atol=2e-2):
        raise SystemExit("end-to-end forward output differs from the device-resident run")

    # ---- the step before the path: this scene's kernel map built on the device (reported beside the headline)
    map_builder = None
    if rank == 0 and km.out_coords is not None and km.n_in == km.n_out and km.k_vol == 27:
        from fgms_b200 import gpu_maps
        coords_d = torch.from_numpy(np.ascontiguousarray(km.out_coords, dtype=np.int32)).to(dev)
        for _ in range(3):
            dk = gpu_maps.build_submanifold_map(coords_d, 3)
        torch.cuda.synchronize()
        evs = []
        for _ in range(10):
            flush()
            a, b = ev(), ev()
            a.record(); dk = gpu_maps.build_submanifold_map(coords_d, 3); b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
        same = bool(torch.equal(dk.imap, p.imap) and torch.equal(dk.omap, p.omap) and torch.equal(dk.kpos, p.kpos))
        map_builder = {"what": "submanifold 3x3x3 kernel map of this scene, hash table + 27 queries per voxel + scan",
                       "ms": ms, "voxels": km.n_in, "pairs": dk.pairs, "Mqueries_per_s": 27 * km.n_in / ms / 1e3,
                       "identical_to_host_builder": same,
                       "note": "includes the allocation of its outputs and one stream synchronisation (pair count)"}

    # ---- the reference's own CUDA kernels on the same tensors (only where they are sound, only when built) ------
    reference_cuda = None
    if rank == 0 and args.reference_cuda:
        try:
            reference_cuda = run_reference_cuda(wl, p, prepare, ev)
        except Exception as exc:  # a checker that cannot load or run must not take the benchmark down
            reference_cuda = {"unavailable": f"the reference extension could not be used: {exc!r}"}

    fallbacks = backend.fallback_count() - fallbacks0
    strong = None
    if shard_rows:
        # every rank holds the SAME scene here (rank 0's) and works on its own row ranges of it
        wl0 = workloads.get(args.workload, seed_offset=0)
        p0 = p if rank == 0 else workloads.LayerTensors(wl0.kmap, wl0.c_in, wl0.c_out, wl0.seed, wl0.mode, device=dev)
        strong = run_row_shard(args, dev, rank, world, wl0, p0, flush)
        del p0
    cfg5, cfg5_check = (None, None)
    if args.cfg5:
        del d_in, d_out
        cfg5, cfg5_check = run_cfg5(args, dev, rank, world, flush)

    # ---- reduce over ranks ---------------------------------------------------------------------
    flops_local = workloads.flops(wl)
    stats = torch.tensor([total_ms, warm_ms, e2e_ms, flops_local, float(km.pairs), alone_ms], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, warm_ms, e2e_ms, alone_ms = float(mx[0]), float(mx[1]), float(mx[2]), float(mx[5])
        flops_all, pairs_all = float(sm[3]), float(sm[4])
    else:
        flops_all, pairs_all = flops_local, float(km.pairs)

    failed = [n for n, c in (("multi_gpu_check", check), ("cfg5.multi_gpu_check", cfg5_check), ("strong_scaling", strong))
              if c is not None and not c["ok"]]
    if rank == 0:
        k = args.steps
        value = flops_all * k / (total_ms * 1e-3) / 1e12
        hbm, f16_peak, peak_src = load_peaks()
        t_peak = tensor_peak_tflops(wl.mode, f16_peak)
        pass_flops = 2.0 * km.pairs * wl.c_in * wl.c_out
        dom = max(pass_ms, key=lambda n: statistics.mean(pass_ms[n]))
        dom_ms = statistics.mean(pass_ms[dom])
        dom_bytes = workloads.algorithmic_bytes(wl, dom)
        t_hbm, t_tensor = dom_bytes / (hbm * 1e9), pass_flops / (t_peak * 1e12)
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        all_bytes = workloads.algorithmic_bytes(wl, "all")
        t_roof_step = max(all_bytes / (hbm * 1e9), 3 * pass_flops / (t_peak * 1e12)) * 1e3
        family = backend.kernel_family(dom, wl.c_in, wl.c_out, p.dtype, p.arch80, km.k_vol)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": k, "warmup": args.warmup,
            "ms_per_step": total_ms / k, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"fp16": "f16 (fp32 accumulate)", "tf32": "tf32 (fp32 accumulate)", "fp32": "f32"}[wl.mode],
            "data": "synthetic",
            "config": workload_config(wl, world, args.shard),
            "timing": {"l2": "flushed before every step (512 MB overwrite), outputs re-zeroed, both untimed",
                       "launch": "CUDA-graph replay of the step's launches" if graph is not None else "eager launches",
                       **({"trial_ms_per_step": trial_ms} if trial_ms else {}),
                       **({"ranks": "a rendezvous kernel after the untimed flush starts every rank's step together"}
                          if aligner[0] is not None else {})},
            "e2e": {"value": flops_all / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": int(launches),
            "tensor_core_fallbacks": int(fallbacks),
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm" if t_hbm >= t_tensor else "tensor", "kernel": f"{dom} ({family})",
                         "achieved": achieved, "peak": hbm, "peak_source": peak_src, "unit": "GB/s",
                         "frac": max(t_hbm, t_tensor) / (dom_ms * 1e-3), "traffic": NCU_TRAFFIC.get((dom, wl.name)),
                         "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms,
                         "t_hbm_ms": t_hbm * 1e3, "t_tensor_ms": t_tensor * 1e3, "tensor_peak_tflops": t_peak},
            "step_roofline": {"algorithmic_bytes": all_bytes, "t_roof_ms": t_roof_step, "frac": t_roof_step / (total_ms / k)},
            "pass_ms": {n: statistics.mean(v) for n, v in pass_ms.items()},
            "value_l2_warm": flops_all * k / (warm_ms * 1e-3) / 1e12,
            "ms_per_step_l2_warm": warm_ms / k,
            "pairs_all_ranks": pairs_all,
            "map_builder": map_builder,
            **({"output_stationary": out_stationary} if out_stationary else {}),
        }
        if world > 1:
            line["pass_ms"]["wgrad_kernel"] = line["pass_ms"]["wgrad"]
            line["pass_ms"]["step_kernels_only"] = alone_ms
            line["pass_ms"]["allreduce_exposed"] = total_ms / k - alone_ms
            line["multi_gpu_check"] = check
            if timeline is not None:
                line["exchange_timeline"] = timeline
            line["exchange"] = {"peer": "fgms_b200_peer_exchange: one kernel per rank over peer-mapped memory (plain loads and stores), on a "
                                        "side stream beside the input-gradient kernel",
                                "nccl": "NCCL all-reduce of the fp32 sums (async, beside the input-gradient kernel)"}[layer_transport]
        if reference_cuda is not None:
            if "step_ms" in reference_cuda:
                reference_cuda["speedup_of_this_library"] = reference_cuda["step_ms"] / (total_ms / k)
            line["reference_cuda"] = reference_cuda
        if strong is not None:
            line["strong_scaling"] = strong
        if cfg5 is not None:
            line["cfg5"] = cfg5
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            cpu_step(wl, threads)
            ts = [cpu_step(wl, threads) for _ in range(3)]
            line["cpu_baseline"] = {"value": flops_local / min(ts) / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"whole {wl.name} layer (fwd+dgrad+wgrad) on the host, best of 3",
                                    "ms_per_step": min(ts) * 1e3}
            line["cpu_literal_cfg1"] = cpu_literal_cfg1()
        if failed:
            line["failed_checks"] = failed
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if failed:
        raise SystemExit(f"result check failed: {failed}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg4")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shard", default="both", choices=["both", "scenes"],
                    help="N > 1: the headline is always one scene per rank (weak scaling); 'both' also cuts ONE scene over the "
                         "ranks by row range and reports that step as strong_scaling, 'scenes' skips it")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time the eager step instead of a CUDA-graph replay of it")
    ap.add_argument("--no-align", dest="align", action="store_false",
                    help="N > 1, peer transport: no rendezvous kernel between the untimed L2 flush and the timed step")
    ap.add_argument("--no-cfg5", dest="cfg5", action="store_false", help="skip the encoder-decoder stack")
    ap.add_argument("--cfg5-steps", type=int, default=20)
    ap.add_argument("--transport", default="auto", choices=["auto", "peer", "nccl"],
                    help="N > 1: how the weight-gradient sums are exchanged: the library's kernel over peer memory, an NCCL "
                         "all-reduce, or (auto) the former for the single layer's 1.8 MB and, for the stack's buckets, whichever of "
                         "NCCL launched eagerly and the library's kernel replayed from a graph a short trial finds faster")
    ap.add_argument("--no-reference-cuda", dest="reference_cuda", action="store_false",
                    help="do not time the reference's CUDA kernels beside this library (they run only when built and sound)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.steps < 1:
        args.steps = 1
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
