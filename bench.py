#!/usr/bin/env python
"""Benchmark of the sparse-convolution hot path: one layer, forward + dgrad + wgrad per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg4] [--impl ours|reference]

A *step* is one forward and one backward (input gradient + weight gradient) of one layer over one
synthetic voxel cloud (``fgms_b200.workloads``; default ``cfg4``: LiDAR-like sweep, 3x3x3
submanifold, fp16 128->128 — the configuration the 60 %-of-roofline target is stated on).  The metric
is effective TFLOPS = 6 * pairs * c_in * c_out / time; ``ms_per_step`` is ms per layer.

* ``value``      device-resident inputs, CUDA events around each step on the launching stream, L2
                 flushed (a 512 MB buffer is overwritten) and outputs re-zeroed before every step,
                 outside the timed interval.
* ``e2e``        the same step through the public binding with HOST buffers: pinned host -> device
                 copies of features, weights, output gradient and maps, the three operator calls,
                 and device -> host copies of all three results, all inside the timed interval.
* ``roofline``   for the slowest of the three kernels of the step: algorithmic bytes of that pass
                 divided by its mean launch duration (events recorded around the call, in the same
                 timed steps), against the measured HBM copy bandwidth.
* ``cpu_baseline`` / ``--impl reference``  the reference's CPU definition (cpu-check.py /
                 cpu-check-back.py) restated per offset as index_select -> matmul -> index_add_ in
                 fp32 on all host threads (``oracle/spconv_oracle.py``), on the same workload.

With N > 1 (torchrun, one rank per GPU) every rank holds its own scene of the same kind (weak
scaling, data parallel); the weight-gradient partial sums are combined with one NCCL all-reduce
inside the timed step.  Rank 0 prints ONE JSON line.
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (kernel -> workload -> bytes); None where no capture exists yet.
NCU_TRAFFIC = {  # profiles/cfg4_fp16_c128_umma_kernels.md
    ("fwd", "cfg4"): 79.8e6, ("dgrad", "cfg4"): 79.4e6, ("wgrad", "cfg4"): 83.7e6,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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


def run_reference(args):
    """The reference's CPU path timed on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from fgms_b200 import workloads
    wl = workloads.get(args.workload)
    threads = os.cpu_count() or 1
    flops = workloads.flops(wl)
    for _ in range(max(1, min(args.warmup, 1))):
        cpu_step(wl, threads)
    times = [cpu_step(wl, threads) for _ in range(max(1, min(args.steps, 5)))]
    t = statistics.mean(times)
    val = flops / t / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": len(times),
        "warmup": 1, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(wl, args.gpus, "host memory"),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": f"whole {wl.name} layer, fwd+dgrad+wgrad, mean of {len(times)} runs"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(wl, gpus, l2):
    km = wl.kmap
    return {"workload": f"{wl.name}: {wl.description}", "n_in": km.n_in, "n_out": km.n_out, "pairs": km.pairs,
            "k_vol": km.k_vol, "c_in": wl.c_in, "c_out": wl.c_out, "math": wl.mode, "seed": wl.seed,
            "parallelism": f"dp{gpus} (one scene per GPU, wgrad all-reduce)" if gpus > 1 else "single GPU",
            "l2": l2}


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
        # the 1.8 MB weight-gradient all-reduce is latency-bound; on 8-GPU B200 boxes it was measured
        # faster without NVLink-switch reductions (30.8 vs 46.0 us back to back, 213 vs 228 us per step)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    wl = workloads.get(args.workload, seed_offset=1000 * rank)
    km = wl.kmap
    p = workloads.LayerTensors(km, wl.c_in, wl.c_out, wl.seed, wl.mode, device=dev)
    layer = SceneParallelLayer(p.kpos, p.imap, p.omap, p.qsum, p.arch80)
    out = torch.zeros((km.n_out, wl.c_out), dtype=p.dtype, device=dev)
    in_grad = torch.zeros((km.n_in, wl.c_in), dtype=p.dtype, device=dev)
    w_grad = torch.zeros_like(p.weights)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def prepare():
        out.zero_(); in_grad.zero_(); w_grad.zero_()
        flush_buf.fill_(1)  # evict L2 (126 MB) so that every step starts cold

    ev = lambda: torch.cuda.Event(enable_timing=True)
    pass_ms = {"fwd": [], "dgrad": [], "wgrad": []}

    bound = BoundSceneLayer(p.feats, p.weights, p.grad_out, out, in_grad, w_grad, p.kpos, p.imap, p.omap, p.arch80) if world > 1 else None

    def layer_wgrad():
        if p.dtype == torch.float16 and world == 1:
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, p.kpos, p.imap, p.omap, p.arch80)
        elif p.dtype == torch.float16:
            ws = backend.fgms_wgrad_cuda(p.feats, p.grad_out, w_grad, p.kpos, p.imap, p.omap, p.arch80,
                                         workspace=backend.wgrad_workspace(wl.c_in, wl.c_out, km.k_vol, dev), accumulate=False)
            part = ws[: w_grad.numel()]
            dist.all_reduce(part)
            backend.wgrad_finalize(w_grad, part)
        else:
            part = torch.zeros_like(w_grad)
            backend.fgms_wgrad_cuda(p.feats, p.grad_out, part, p.kpos, p.imap, p.omap, p.arch80)
            if world > 1:
                dist.all_reduce(part)
            w_grad.add_(part)

    def step(record, passes=False):
        """One fwd + dgrad + wgrad.  record: events around the step; passes: also between the passes (used in a
        separate loop only, so that the headline step has nothing between its kernels)."""
        e = [ev() for _ in range(4)] if record else None
        if record: e[0].record()
        if world > 1 and not passes:
            # data parallel: the step bound to its buffers (no per-call argument checks on the host); wgrad first,
            # its all-reduce runs beside dgrad
            bound.forward()
            bound.backward()
            if record: e[3].record()
            return e
        layer.forward(p.feats, p.weights, out)
        if passes: e[1].record()
        backend.fgms_dgrad_cuda(p.grad_out, p.weights, in_grad, p.kpos, p.imap, p.omap, p.arch80)
        if passes: e[2].record()
        layer_wgrad()
        if record: e[3].record()
        return e

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing --------------------------------------------------------------
    for _ in range(args.warmup):
        prepare(); step(False)
    barrier()
    # The same launches are captured once into a CUDA graph and replayed, which takes the host out of the step;
    # the kernels, their order and their arguments are those of the eager step.  --no-graph times the eager step.
    graph = None
    launches_per_step = None
    if args.graph and world == 1:  # with a collective in the step the capture hung when it was tried with 2 ranks: N > 1 runs the bound step eagerly
        try:
            c0 = backend.launch_count()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
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

    def timed_step():
        if graph is None:
            return step(True)
        e = [ev() for _ in range(4)]
        e[0].record(); graph.replay(); e[3].record()
        return e

    launches0 = backend.launch_count()
    events = []
    with ClockSampler(local) as clocks:
        for _ in range(args.steps):
            prepare()
            events.append(timed_step())
        barrier()
    launches = (backend.launch_count() - launches0) if graph is None else launches_per_step * args.steps
    step_ms = [e[0].elapsed_time(e[3]) for e in events]
    total_ms = sum(step_ms)

    # per-pass durations (for the roofline of the slowest pass): same steps with events between the passes
    pass_events = []
    for _ in range(min(args.steps, 50)):
        prepare()
        pass_events.append(step(True, passes=True))
    barrier()
    for e in pass_events:
        pass_ms["fwd"].append(e[0].elapsed_time(e[1]))
        pass_ms["dgrad"].append(e[1].elapsed_time(e[2]))
        pass_ms["wgrad"].append(e[2].elapsed_time(e[3]))

    # warm-L2 variant (no flush), reported beside the headline
    for _ in range(2):
        out.zero_(); in_grad.zero_(); w_grad.zero_(); step(False)
    barrier()
    warm = []
    for _ in range(args.steps):
        out.zero_(); in_grad.zero_(); w_grad.zero_()
        e = timed_step()
        warm.append(e)
    barrier()
    warm_ms = sum(e[0].elapsed_time(e[3]) for e in warm)

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

    for i in range(max(2, args.warmup // 2) * 2):
        e2e_step(i)
    barrier()
    e2e_t0, e2e_t1 = ev(), [ev() for _ in range(3)]
    e2e_t0.record(s_up)
    s_run.wait_event(e2e_t0); s_down.wait_event(e2e_t0)
    for i in range(args.steps):
        e2e_step(i)
    for e, st in zip(e2e_t1, (s_up, s_run, s_down)):
        e.record(st)
    barrier()
    e2e_ms = max(e2e_t0.elapsed_time(e) for e in e2e_t1)
    # the last step's results, downloaded through the same path, must match the device-resident run
    # (fp16 reds arrive in a different order every run, so the comparison allows rounding differences)
    if not torch.allclose(h_out[(args.steps - 1) & 1]["out"].float(), out.cpu().float(), rtol=2e-2, atol=2e-2):
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
            flush_buf.fill_(1)
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

    # ---- reduce over ranks ---------------------------------------------------------------------
    flops_local = workloads.flops(wl)
    stats = torch.tensor([total_ms, warm_ms, e2e_ms, flops_local, float(km.pairs)], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, warm_ms, e2e_ms = float(mx[0]), float(mx[1]), float(mx[2])
        flops_all, pairs_all = float(sm[3]), float(sm[4])
    else:
        flops_all, pairs_all = flops_local, float(km.pairs)

    if rank == 0:
        k = args.steps
        value = flops_all * k / (total_ms * 1e-3) / 1e12
        dom = max(pass_ms, key=lambda n: statistics.mean(pass_ms[n]))
        dom_ms = statistics.mean(pass_ms[dom])
        dom_bytes = workloads.algorithmic_bytes(wl, dom)
        peak, peak_src = load_peaks()
        achieved = dom_bytes / (dom_ms * 1e-3) / 1e9
        all_bytes = workloads.algorithmic_bytes(wl, "all")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": k, "warmup": args.warmup,
            "ms_per_step": total_ms / k, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"fp16": "f16 (fp32 accumulate)", "tf32": "tf32 (fp32 accumulate)", "fp32": "f32"}[wl.mode],
            "data": "synthetic",
            "config": dict(workload_config(wl, world, "flushed before every step (512 MB overwrite), outputs re-zeroed, both untimed"),
                           launch="CUDA-graph replay of the step's launches" if graph is not None else "eager launches"),
            "e2e": {"value": flops_all * k / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / k},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": f"{dom} ({backend.kernel_family(dom, wl.c_in, wl.c_out, p.dtype, p.arch80)})",
                         "achieved": achieved, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC.get((dom, wl.name)),
                         "algorithmic_bytes_per_launch": dom_bytes, "ms_per_launch": dom_ms},
            "step_roofline": {"algorithmic_bytes": all_bytes, "t_roof_ms": all_bytes / (peak * 1e9) * 1e3,
                              "frac": all_bytes / (peak * 1e9) * 1e3 / (total_ms / k)},
            "pass_ms": {n: statistics.mean(v) for n, v in pass_ms.items()},
            "value_l2_warm": flops_all * k / (warm_ms * 1e-3) / 1e12,
            "ms_per_step_l2_warm": warm_ms / k,
            "pairs_all_ranks": pairs_all,
            "map_builder": map_builder,
        }
        if world == 1 and not args.no_cpu:
            threads = os.cpu_count() or 1
            cpu_step(wl, threads)
            ts = [cpu_step(wl, threads) for _ in range(3)]
            line["cpu_baseline"] = {"value": flops_local / min(ts) / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"whole {wl.name} layer (fwd+dgrad+wgrad) on the host, best of 3",
                                    "ms_per_step": min(ts) * 1e3}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="cfg4")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time the eager step instead of a CUDA-graph replay of it")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
