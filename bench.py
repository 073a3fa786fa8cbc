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
    p.add_argument("--config", type=int, default=1, help="index into CONFIGS above (the five network sizes of the Graph Challenge)")
    p.add_argument("--pattern", default="radix16", choices=["radix16", "random"])
    p.add_argument("--neurons", type=int)
    p.add_argument("--layers", type=int)
    p.add_argument("--batch", type=int, help="images per GPU")
    p.add_argument("--inputs", default="blobs", choices=["blobs", "mixed"],
                   help="blobs: ~15%% dense discs on the pixel grid; mixed: unstructured, density 5-60%% per image")
    p.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                   help="weak: every GPU runs --batch images; strong: --batch images are split over the GPUs")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-two-contexts", action="store_true", help="skip the end-to-end loop that alternates two contexts")
    p.add_argument("--no-per-layer-line", action="store_true",
                   help="skip the extra line that times the per-layer kernel alone (SPDNN_RESIDENT=0) against the HBM roofline")
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
    """DRAM bytes (read + write) per LAYER of the dominant kernel on this workload, from the
    committed summary of an ncu capture (profiles/); None when no capture covers it."""
    path = os.path.join(ROOT, "profiles", "layer_kernel_traffic.json")
    if not os.path.exists(path):
        return None
    try:
        for rec in json.load(open(path)):
            if rec.get("neurons") == cfg["neurons"] and rec.get("pattern") == pattern:
                return rec.get("dram_bytes_per_layer")
    except Exception:
        return None
    return None


class ClockSampler:
    """SM clock and throttle reasons DURING the timed region: an NVML polling thread (the
    region lasts tens of milliseconds, shorter than one nvidia-smi interval)."""
    REASONS = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}

    def __init__(self, index):
        self.index, self.samples, self.bits, self.max_mhz, self.thread, self.stop_flag = index, [], 0, None, None, False
        self.power, self.stamps, self.windows = [], [], []

    def _run(self, nv, h):
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                self.stamps.append(time.perf_counter())
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                if len(self.samples) % 32 == 16:      # the power query can take milliseconds: rarely, and not first
                    self.power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
            except Exception:
                pass
            time.sleep(0)            # yield; the region may last only a few milliseconds

    def prepare(self):
        """NVML set-up (milliseconds): done before the timed region, so that start() only spawns the thread."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            idx = self.index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                try:
                    idx = int(vis.split(",")[self.index])
                except Exception:
                    pass
            h = nv.nvmlDeviceGetHandleByIndex(idx)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)          # first calls pay for lazy set-up inside NVML
            nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            self.nv, self.handle = nv, h
        except Exception:
            self.nv = self.handle = None

    def start(self):
        if getattr(self, "nv", None) is None:
            self.prepare()
        if self.nv is None:
            return
        import threading
        self.thread = threading.Thread(target=self._run, args=(self.nv, self.handle), daemon=True)
        self.thread.start()

    def window(self, t0, t1):
        """A timed region (host clock, bracketed by synchronisations): only samples inside count."""
        self.windows.append((t0, t1))

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)
        inside = [m for m, t in zip(self.samples, self.stamps) if any(a <= t <= b for a, b in self.windows)] if self.windows \
            else list(self.samples)
        first = self.windows[0] if self.windows else None
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": len(inside),
               "samples_in_value_region": sum(1 for t in self.stamps if first and first[0] <= t <= first[1]),
               "regions": "value + e2e timed regions"}
        if inside:
            out["sm_mhz"] = statistics.median(inside)
            out["power_w_max"] = max(self.power) if self.power else None
        out["reasons"] = sorted(k for k, bit in self.REASONS.items() if self.bits & bit)
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

def per_layer_line(net, y_dev, cfg, device, stream, first_id, want_survivors, passes=3):
    """The same workload with ONE launch per layer (SPDNN_RESIDENT=0): the formulation whose bytes
    the roofline counts -- every layer reads and writes every live image's N activations in HBM.
    Reported beside the headline so that the hand-written gather kernel can be read against the
    measured copy bandwidth; it is not the path `value` times."""
    from graphchallenge21_b200 import SpDNN
    n, L = cfg["neurons"], cfg["layers"]
    old = os.environ.get("SPDNN_RESIDENT")
    os.environ["SPDNN_RESIDENT"] = "0"
    try:
        g = SpDNN(n, L, float(net.bias), device=device)
    finally:
        if old is None:
            del os.environ["SPDNN_RESIDENT"]
        else:
            os.environ["SPDNN_RESIDENT"] = old
    try:
        g.set_network(net)
        g.set_stream(stream.cuda_stream)
        ms, r = [], None
        for i in range(passes + 1):                   # the first pass builds the launch graph and warms up
            g.set_input_dense(y_dev, first_id)
            r = g.infer()
            if i:
                ms.append(r.infer_ms)
        assert r.survivors == want_survivors, (r.survivors, want_survivors)
        peak, peak_kind = peaks()
        loop_ms = sum(ms) / len(ms)
        achieved = r.algorithmic_bytes / (loop_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json hbm_gbs)", "kernel": "layer_kernel",
                "launches_per_pass": int(r.loop_launches), "layer_loop_ms": loop_ms, "us_per_layer": loop_ms * 1e3 / L,
                "passes": passes, "traffic": None,
                "note": "one launch per layer, activations in HBM between layers; layers after the first few work on the "
                        "survivors only, whose two activation buffers (%.0f MB) can partly stay in the 126 MB L2"
                        % (2.0 * r.survivors * n * 4 / 1e6)}
    finally:
        g.close()


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
    if args.scaling == "strong":
        B = (B + world - 1) // world              # contiguous slices of one batch, as src/multi_gpu.cpp:146-151
    net = SyntheticNetwork(n, L, args.pattern)
    g = SpDNN(n, L, float(net.bias), device=local)
    g.set_network(net)
    info = g.layer_info(min(1, L - 1))
    if args.inputs == "mixed":
        from graphchallenge21_b200.generator import mixed_density_images
        y_np = mixed_density_images(n, B, first_image=rank * B)
    else:
        y_np = synthetic_images(n, B, first_image=rank * B)
    y_host = torch.from_numpy(y_np).pin_memory()
    y_dev = y_host.cuda()
    # everything the library enqueues goes to ONE explicit stream, and the timing events are
    # recorded on that same stream (the legacy default stream has handle 0, which the library
    # reads as "use your own stream")
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    g.set_stream(stream.cuda_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step_resident():
        g.set_input_dense(y_dev, rank * B)
        g.infer_async()

    # the same images as the reference's input file holds them: (img, neuron) triplets, value 1
    img_np, neu_np = np.nonzero(y_host.numpy())
    coo_img = torch.from_numpy(img_np.astype(np.int32)).pin_memory()
    coo_neu = torch.from_numpy(neu_np.astype(np.int32)).pin_memory()

    def step_e2e(kind="coo"):
        if kind == "dense":
            g.set_input_dense(y_host, rank * B)                                  # H2D of batch x N floats inside
        else:
            g.set_input_coo(coo_img.numpy(), coo_neu.numpy(), None, B, rank * B, index_base=0)   # H2D of the triplets inside
        g.infer_async()
        return g.categories()                    # D2H of the result (waits for the step)

    for _ in range(args.warmup):
        step_resident()
        g.sync()
    # -- value: inputs resident in HBM, device-timed
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.prepare()
        # the timed loop is a few milliseconds of Python that enqueues work: let the polling thread
        # preempt it (the default switch interval of the interpreter is 5 ms)
        sys.setswitchinterval(1e-4)
    barrier()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    infer_ms, prep_ms, algo_bytes, launches, loop_launches, group = [], [], 0.0, 0, 0, 0
    t_host0 = time.perf_counter()
    ev0.record(stream)
    for _ in range(args.steps):
        step_resident()          # queued back to back on the stream; only the last pass is synchronised
    ev1.record(stream)
    while not ev1.query():       # wait without holding the interpreter lock, so that the clock sampler runs
        time.sleep(0)
    barrier()
    sampler.window(t_host0, time.perf_counter())
    ms = ev0.elapsed_time(ev1)
    r = g.sync()                 # statistics of the last timed pass (every pass does the same work)
    infer_ms.append(r.infer_ms); prep_ms.append(r.prepare_ms)
    algo_bytes, launches = r.algorithmic_bytes, r.kernel_launches
    loop_launches, group = r.loop_launches, r.resident_group
    survivors = r.survivors
    live = g.layer_live().copy()
    # -- e2e: host buffers in, category list out, copies inside the timed region
    def time_e2e(kind):
        step_e2e(kind)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        for _ in range(args.steps):
            c_ = step_e2e(kind)
        e1.record(stream)
        barrier()
        sampler.window(t0, time.perf_counter())
        return e0.elapsed_time(e1), c_
    ms_e2e_dense, _ = time_e2e("dense")
    ms_e2e, cats = time_e2e("coo")

    # -- the same end-to-end step with TWO contexts taking turns (each with its own stream and buffers, the
    #    weights held twice): the host->device copy of step k+1's input runs while step k's pass computes
    def time_e2e_two_contexts():
        g2 = SpDNN(n, L, float(net.bias), device=local)
        try:
            g2.set_network(net)
            stream2 = torch.cuda.Stream()
            g2.set_stream(stream2.cuda_stream)
            ctx = [g, g2]

            def enqueue(c):
                c.set_input_coo(coo_img.numpy(), coo_neu.numpy(), None, B, rank * B, index_base=0)
                c.infer_async()

            for c in ctx:                      # graph build and warm-up of both
                enqueue(c)
                c.categories()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record(stream)
            enqueue(ctx[0])
            c_ = None
            for k in range(args.steps):
                if k + 1 < args.steps:
                    enqueue(ctx[(k + 1) % 2])
                c_ = ctx[k % 2].categories()   # D2H of step k's result (waits for step k only)
            stream.wait_stream(stream2)
            e1.record(stream)
            barrier()
            sampler.window(t0, time.perf_counter())
            return e0.elapsed_time(e1), np.asarray(c_).copy()
        finally:
            g2.close()
    ms_e2e_two, cats_two = (None, None) if args.no_two_contexts else time_e2e_two_contexts()
    if cats_two is not None:
        assert np.array_equal(cats_two, np.asarray(cats)), "the two-context loop returned other categories"
    clocks = sampler.stop() if rank == 0 else None
    e2e_prepare_ms = g.sync().prepare_ms          # H2D + layout conversion of the last end-to-end step
    d2h = int(len(cats) * 4 + (L + 1) * 16 + 4)
    all_cats = gather_categories(np.asarray(cats).copy())
    t = torch.tensor([ms, ms_e2e, ms_e2e_dense, ms_e2e_two or 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_e2e_dense = float(t[0]), float(t[1]), float(t[2])
    ms_e2e_two = float(t[3]) if ms_e2e_two is not None else None
    edges_step = float(world) * B * n * 32.0 * L
    out = None
    if rank == 0:
        peak, peak_kind = peaks()
        loop_ms = sum(infer_ms) / len(infer_ms)
        achieved = algo_bytes / (loop_ms * 1e-3) / 1e9
        out = {
            "metric": METRIC, "value": edges_step * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"N={n} L={L} batch={B} per GPU, pattern {args.pattern}", "neurons": n, "layers": L,
                       "batch_per_gpu": B, "pattern": args.pattern, "inputs": args.inputs, "bias": float(net.bias),
                       "parallelism": f"batch-sharded x{world}, weights replicated",
                       "l2": ("inputs larger than L2 (%.0f MB per step), no flush" % (B * n * 4 / 1e6)) if B * n * 4 > 126e6
                             else ("input %.0f MB per step, smaller than L2: the timed passes run back to back, each overwriting "
                                   "both activation buffers; no flush" % (B * n * 4 / 1e6)),
                       "survivors_rank0": int(survivors), "survivors_total": int(len(all_cats)),
                       "live_after_layer": {str(i): int(live[i]) for i in sorted({0, 1, 2, 4, 8, 16, 32, L - 1}) if i < L},
                       "classes_per_layer": info["classes"]},
            "e2e": {"value": edges_step * args.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": int(coo_img.numel() * 8), "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps, "input_ms": e2e_prepare_ms,
                    "call": "spdnn_set_input_coo (the input file's img/neuron triplets, pinned host memory) + spdnn_infer "
                            "+ spdnn_get_categories",
                    "two_contexts": None if ms_e2e_two is None else {
                        "value": edges_step * args.steps / (ms_e2e_two * 1e-3), "ms_per_step": ms_e2e_two / args.steps,
                        "call": "the same three calls on two contexts in turn (own stream and buffers each): the copy of "
                                "step k+1's input overlaps step k's pass; every step's H2D and D2H are inside the region"},
                    "dense_input": {"value": edges_step * args.steps / (ms_e2e_dense * 1e-3), "h2d_bytes_per_step": B * n * 4,
                                    "ms_per_step": ms_e2e_dense / args.steps,
                                    "call": "spdnn_set_input_dense (batch x N fp32, pinned host memory)"}},
            "gpu_launches": int(launches * args.steps),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json hbm_gbs)", "traffic": None,
                         "kernel": (("alt2_kernel<%d>" if args.pattern == "radix16" else "resident_kernel<%d>") % group) if group else "layer_kernel",
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
            # per launch, like `achieved`: the capture's per-layer figure times the layers of an average launch
            out["roofline"]["traffic"] = tr * L / max(loop_launches, 1)
    g.close()
    if rank == 0 and world == 1 and not args.no_per_layer_line:
        out["roofline_per_layer_kernel"] = per_layer_line(net, y_dev, cfg, local, stream, rank * B, survivors)
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
