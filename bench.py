#!/usr/bin/env python
"""Benchmark of the sparse-DNN inference path: edges/s = batch * N * 32 * L / time.

    python bench.py --gpus N --steps K --warmup W            # the CUDA path of this repository
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path, host cores

One step = one inference pass (all L layers) over one batch of seeded synthetic images.
Default workload: N=1024 neurons, L=1920 layers, 60000 images per GPU (weak scaling: every
rank runs its own 60000-image shard, weights replicated, no collective in the layer loop, one
final gather of the surviving image numbers).  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = [
    {"neurons": 1024, "layers": 120, "batch": 6000},
    {"neurons": 1024, "layers": 1920, "batch": 60000},
    {"neurons": 4096, "layers": 480, "batch": 60000},
    {"neurons": 16384, "layers": 1920, "batch": 60000},
    {"neurons": 65536, "layers": 1920, "batch": 60000},
]
METRIC = "inference edges/sec (batch*N*32*L/time)"
UNIT = "edges/s"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--config", type=int, default=1, help="index into BASELINE.json configs")
    p.add_argument("--pattern", default="radix16", choices=["radix16", "random"])
    p.add_argument("--neurons", type=int)
    p.add_argument("--layers", type=int)
    p.add_argument("--batch", type=int, help="images per GPU")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the cpu_baseline sample")
    return p.parse_args()


def workload(args):
    cfg = dict(CONFIGS[args.config])
    for k in ("neurons", "layers", "batch"):
        if getattr(args, k) is not None:
            cfg[k] = getattr(args, k)
    return cfg


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def ncu_traffic(cfg, pattern):
    """DRAM bytes (read + write) per launch of the layer kernel on this workload, from the
    committed summary of an ncu capture (profiles/); None when no capture covers it."""
    path = os.path.join(ROOT, "profiles", "layer_kernel_traffic.json")
    if not os.path.exists(path):
        return None
    try:
        for rec in json.load(open(path)):
            if rec.get("neurons") == cfg["neurons"] and rec.get("pattern") == pattern:
                return rec.get("dram_bytes_per_launch")
    except Exception:
        return None
    return None


class ClockSampler:
    """nvidia-smi samples of the SM clock and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for nm, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(nm)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), samples=len(sm))
        out["reasons"] = sorted(reasons)
        return out


# ---- CPU arm: the reference's own CPU loop (or the oracle port) on the host cores ------------

def cpu_sample_case(cfg, pattern, batch, layers, path):
    from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images
    from oracle import make_case
    net = SyntheticNetwork(cfg["neurons"], layers, pattern)
    y0 = synthetic_images(cfg["neurons"], batch)
    make_case.write_case(path, y0, [net.layer_rows(l) for l in range(layers)], float(net.bias))
    return net, y0


def run_cpu_reference(cfg, pattern, seconds, threads=None):
    """Times CpuSpmm::run_and_cmp (the reference's CPU implementation of one layer's product,
    src/utils/cpu_spmm.h:11-55) over all layers of a bounded sample of the workload, image slices
    spread over all host threads.  Falls back to the oracle port when the compiled reference
    harness is not present.  Returns a cpu_baseline dict."""
    from oracle import build as ob
    threads = threads or os.cpu_count() or 1
    harness = ob.build_ref()
    n = cfg["neurons"]
    batch = min(cfg["batch"], 64 * max(threads, 8))
    layers = min(cfg["layers"], 8)
    sample = f"first {batch} images x first {layers} layers of the workload, repeated to fill ~{seconds:.0f} s"
    if harness is not None:
        with tempfile.TemporaryDirectory() as d:
            case = os.path.join(d, "case.bin")
            cpu_sample_case(cfg, pattern, batch, layers, case)
            r = json.loads(subprocess.run([harness, "time", case, str(threads), "1"], capture_output=True, text=True,
                                          check=True).stdout.strip().splitlines()[-1])
            reps = max(1, int(seconds / max(r["seconds"], 1e-3)))
            r = json.loads(subprocess.run([harness, "time", case, str(threads), str(reps)], capture_output=True,
                                          text=True, check=True).stdout.strip().splitlines()[-1])
        return {"value": r["edges_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "reference",
                "sample": sample + f" ({r['repetitions']} repetitions, {r['seconds']:.1f} s; no pruning of dead images, "
                "as the reference's CPU loop)", "seconds": r["seconds"]}
    from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images
    from oracle import c_oracle
    net = SyntheticNetwork(n, layers, pattern)
    y0 = synthetic_images(n, batch)
    lay = [(net.layer_rows(l), None) for l in range(layers)]
    t0 = time.perf_counter(); c_oracle.infer(y0, lay, float(net.bias), prune=False, want_activations=False)
    one = time.perf_counter() - t0
    reps = max(1, int(seconds / max(one, 1e-3)))
    t0 = time.perf_counter()
    for _ in range(reps):
        c_oracle.infer(y0, lay, float(net.bias), prune=False, want_activations=False)
    dt = time.perf_counter() - t0
    return {"value": batch * n * 32.0 * layers * reps / dt, "unit": UNIT, "cores": c_oracle.max_threads(), "kind": "port",
            "sample": sample + f" ({reps} repetitions, {dt:.1f} s)", "seconds": dt}


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cfg = workload(args)
    per_step = max(2.0, min(20.0, 90.0 / max(args.steps + args.warmup, 1)))
    for _ in range(args.warmup):
        run_cpu_reference(cfg, args.pattern, min(per_step, 2.0))
    vals, secs, last = [], 0.0, None
    for _ in range(args.steps):
        last = run_cpu_reference(cfg, args.pattern, per_step)
        vals.append(last["value"]); secs += last["seconds"]
    value = len(vals) / sum(1.0 / v for v in vals)
    cb = dict(last); cb["value"] = value; cb.pop("seconds", None)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * secs / max(args.steps, 1), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"N={cfg['neurons']} L={cfg['layers']} batch={cfg['batch']} per GPU, pattern {args.pattern}",
                   "note": "reference CPU loop on the host cores; each step is a bounded sample of the workload"},
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))
    return 0


# ---- our arm -----------------------------------------------------------------------------------

def main_ours(args):
    import torch
    import torch.distributed as dist
    from graphchallenge21_b200 import SpDNN, SyntheticNetwork, synthetic_images
    from graphchallenge21_b200.network import gather_categories

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = workload(args)
    n, L, B = cfg["neurons"], cfg["layers"], cfg["batch"]
    net = SyntheticNetwork(n, L, args.pattern)
    g = SpDNN(n, L, float(net.bias), device=local)
    for l in range(L):
        g.set_layer_csc(l, *net.layer_csc(l))
    info = g.layer_info(min(1, L - 1))
    y_host = torch.from_numpy(synthetic_images(n, B, first_image=rank * B)).pin_memory()
    y_dev = y_host.cuda()
    stream = torch.cuda.current_stream()
    g.set_stream(stream.cuda_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        g.set_input_dense(y_dev, rank * B)
        g.infer_async()

    def step_e2e():
        g.set_input_dense(y_host, rank * B)      # H2D inside
        g.infer_async()
        return g.categories()                    # D2H of the result (waits for the step)

    for _ in range(args.warmup):
        step_resident()
        g.sync()
    # -- value: inputs resident in HBM, device-timed
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    infer_ms, prep_ms, algo_bytes, launches, loop_launches, group = [], [], 0.0, 0, 0, 0
    ev0.record(stream)
    for _ in range(args.steps):
        step_resident()
        r = g.sync()             # waits for this step: the statistics come from the device
        infer_ms.append(r.infer_ms); prep_ms.append(r.prepare_ms)
        algo_bytes, launches = r.algorithmic_bytes, r.kernel_launches
        loop_launches, group = r.loop_launches, r.resident_group
    ev1.record(stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = ev0.elapsed_time(ev1)
    survivors = r.survivors
    live = g.layer_live().copy()
    # -- e2e: host buffers in, category list out, copies inside the timed region
    step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        cats = step_e2e()
    e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    d2h = int(len(cats) * 4 + (L + 1) * 16 + 4)
    all_cats = gather_categories(np.asarray(cats).copy())
    t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e = float(t[0]), float(t[1])
    edges_step = float(world) * B * n * 32.0 * L
    out = None
    if rank == 0:
        peak, peak_kind = peaks()
        loop_ms = sum(infer_ms) / len(infer_ms)
        achieved = algo_bytes / (loop_ms * 1e-3) / 1e9
        out = {
            "metric": METRIC, "value": edges_step * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"N={n} L={L} batch={B} per GPU, pattern {args.pattern}", "neurons": n, "layers": L,
                       "batch_per_gpu": B, "pattern": args.pattern, "bias": float(net.bias),
                       "parallelism": f"batch-sharded x{world}, weights replicated",
                       "l2": "inputs larger than L2 (%.0f MB per step), no flush" % (B * n * 4 / 1e6),
                       "survivors_rank0": int(survivors), "survivors_total": int(len(all_cats)),
                       "live_after_layer": {str(i): int(live[i]) for i in sorted({0, 1, 2, 4, 8, 16, 32, L - 1}) if i < L},
                       "classes_per_layer": info["classes"]},
            "e2e": {"value": edges_step * args.steps / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": B * n * 4,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches * args.steps),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json hbm_gbs)", "traffic": None,
                         "kernel": "resident_kernel<%d>" % group if group else "layer_kernel",
                         "launches_per_step": loop_launches, "avg_launch_us": loop_ms * 1e3 / max(loop_launches, 1),
                         "algorithmic_bytes_per_launch": algo_bytes / max(loop_launches, 1),
                         "us_per_layer": loop_ms * 1e3 / L, "layer_loop_ms": loop_ms,
                         "input_layout_ms": sum(prep_ms) / len(prep_ms),
                         "note": ("activations stay in shared memory across the layers of a launch, so DRAM traffic is far "
                                  "below the algorithmic bytes and frac can exceed 1" if group else "one launch per layer")},
            "clocks": clocks,
        }
        tr = ncu_traffic(cfg, args.pattern)
        if tr is not None:
            out["roofline"]["traffic"] = tr
    g.close()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb = run_cpu_reference(cfg, args.pattern, args.cpu_seconds)
        cb.pop("seconds", None)
        out["cpu_baseline"] = cb
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    a = parse()
    sys.exit(main_reference(a) if a.impl == "reference" else main_ours(a))
