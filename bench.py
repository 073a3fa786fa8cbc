#!/usr/bin/env python
"""Benchmark of the sparse-DNN inference path: edges/s = batch * N * 32 * L / time.

    python bench.py --gpus N --steps K --warmup W            # the CUDA path of this repository
    python bench.py --impl reference --steps K --warmup W    # the reference's CPU path, host cores

One step = one inference pass (all L layers) over one batch of seeded synthetic images.
Default workload = the largest Graph Challenge configuration listed for the GPU count: N=16384 neurons,
L=1920 layers, 60000 images on 1, 2 or 4 GPUs, and N=65536, L=1920, 60000 images on 8 GPUs (with the
N=16384 network beside it).  The ONE batch is split over the ranks in contiguous slices (strong
scaling, as src/microbenchmark/multi_gpu/multi_gpu.cu:251-258 slices it), weights replicated, no
collective in the layer loop, one final gather of the surviving image numbers.  Prints ONE JSON line on
rank 0.
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
    p.add_argument("--config", type=int, help="index into CONFIGS above (the five network sizes of the Graph Challenge); "
                   "default: 3 (N=16384) on 1, 2 or 4 GPUs, 4 (N=65536) on 8")
    p.add_argument("--pattern", default="radix16", choices=["radix16", "random"])
    p.add_argument("--neurons", type=int)
    p.add_argument("--layers", type=int)
    p.add_argument("--batch", type=int, help="images of the whole job (strong scaling) or per GPU (weak scaling)")
    p.add_argument("--inputs", default="blobs", choices=["blobs", "mixed"],
                   help="blobs: ~15%% dense discs on the pixel grid; mixed: unstructured, density 5-60%% per image")
    p.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                   help="strong: --batch images are split over the GPUs; weak: every GPU runs --batch images")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-also", action="store_true", help="skip the extra workloads reported beside the headline")
    p.add_argument("--no-two-contexts", action="store_true", help="skip the end-to-end loop that alternates two contexts")
    p.add_argument("--no-per-layer-line", action="store_true",
                   help="skip the extra line that times the per-layer kernel alone (SPDNN_RESIDENT=0) against the HBM roofline")
    p.add_argument("--cpu-seconds", type=float, default=None,
                   help="target CPU time of each cpu_baseline sample (default 10) and, when given, of each step of --impl reference")
    p.add_argument("--only-value", action="store_true",
                   help="time the HBM-resident passes only (no end-to-end loops, no extra lines): the short run a profiler capture wraps")
    return p.parse_args()


def default_config(world):
    return 4 if world >= 8 else 3


def workload(args, world=1, index=None):
    cfg = dict(CONFIGS[index if index is not None else (args.config if args.config is not None else default_config(world))])
    if index is None:
        for k in ("neurons", "layers", "batch"):
            if getattr(args, k) is not None:
                cfg[k] = getattr(args, k)
    return cfg


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def profile_figures(neurons, pattern, kernel=None):
    """Counters of this workload's kernels from the committed summaries of ncu captures (profiles/ncu_figures.json:
    one record per kernel and network size, each naming the summary file it was read from); the record marked
    dominant first, or the one of `kernel`.  They are constants of the repository, not measured in this run -- a
    profiler cannot run inside a timed benchmark."""
    path = os.path.join(ROOT, "profiles", "ncu_figures.json")
    if not os.path.exists(path):
        return []
    try:
        recs = [r for r in json.load(open(path)) if r.get("neurons") == neurons and r.get("pattern") == pattern
                and (kernel is None or r.get("kernel") == kernel)]
    except Exception:
        return []
    return sorted(recs, key=lambda r: not r.get("dominant", False))


class ClockSampler:
    """SM clock and throttle reasons DURING the timed regions: an NVML polling thread."""
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
            time.sleep(0)            # yield; a region may last only a few milliseconds

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
               "regions": "value + e2e timed regions of the headline workload"}
        if inside:
            out["sm_mhz"] = statistics.median(inside)
            out["power_w_max"] = max(self.power) if self.power else None
        out["reasons"] = sorted(k for k, bit in self.REASONS.items() if self.bits & bit)
        return out


# ---- CPU arm: the reference's own CPU loop (or the oracle port) on the host cores ------------

_CASES = {}       # sample case files of this process: written once, removed at exit


def cpu_sample_case(cfg, pattern, batch, layers):
    """Path of the case file (inputs + layers of the sample) the reference harness reads."""
    import atexit
    import shutil
    from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images
    from oracle import make_case
    key = (cfg["neurons"], pattern, batch, layers)
    if key not in _CASES:
        d = tempfile.mkdtemp(prefix="spdnn_case_")
        atexit.register(shutil.rmtree, d, True)
        net = SyntheticNetwork(cfg["neurons"], layers, pattern)
        y0 = synthetic_images(cfg["neurons"], batch)
        path = os.path.join(d, "case.bin")
        make_case.write_case(path, y0, [net.layer_rows(l) for l in range(layers)], float(net.bias))
        _CASES[key] = path
    return _CASES[key]


def cpu_sample_shape(cfg, threads):
    """Bounded sample of the workload for the CPU arms: its first images and first layers."""
    batch = min(cfg["batch"], 64 * max(threads, 8))
    if cfg["neurons"] >= 16384:
        batch = min(batch, 16 * max(threads, 8) * 16384 // cfg["neurons"] * 2)
    return max(batch, threads), min(cfg["layers"], 8)


def run_cpu_reference(cfg, pattern, seconds, threads=None):
    """Times CpuSpmm::run_and_cmp (the reference's CPU implementation of one layer's product,
    src/utils/cpu_spmm.h:11-55) over all layers of a bounded sample of the workload, image slices
    spread over all host threads.  Falls back to the oracle port when the compiled reference
    harness is not present.  Returns a cpu_baseline dict."""
    from oracle import build as ob
    threads = threads or os.cpu_count() or 1
    harness = ob.build_ref()
    n = cfg["neurons"]
    batch, layers = cpu_sample_shape(cfg, threads)
    sample = f"first {batch} images x first {layers} layers of the workload, repeated to fill ~{seconds:.0f} s"
    if harness is not None:
        case = cpu_sample_case(cfg, pattern, batch, layers)
        r = json.loads(subprocess.run([harness, "time", case, str(threads), "1"], capture_output=True, text=True,
                                      check=True).stdout.strip().splitlines()[-1])
        reps = max(1, int(seconds / max(r["seconds"], 1e-3)))
        r = json.loads(subprocess.run([harness, "time", case, str(threads), str(reps)], capture_output=True,
                                      text=True, check=True).stdout.strip().splitlines()[-1])
        return {"value": r["edges_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "reference",
                "sample": sample + f" ({r['repetitions']} repetitions, {r['seconds']:.1f} s; no pruning of dead images, "
                "as the reference's CPU loop)", "seconds": r["seconds"]}
    return run_cpu_port(cfg, pattern, seconds, prune=False)


def run_cpu_port(cfg, pattern, seconds, prune):
    """The oracle's C restatement of the loop on all host threads (OpenMP over images), with or without
    skipping dead images, on the same bounded sample."""
    from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images
    from oracle import c_oracle
    n = cfg["neurons"]
    batch, layers = cpu_sample_shape(cfg, c_oracle.max_threads())
    if prune:
        layers = min(cfg["layers"], 24)          # long enough for the dead images to be gone
    net = SyntheticNetwork(n, layers, pattern)
    y0 = synthetic_images(n, batch)
    lay = [(net.layer_rows(l), None) for l in range(layers)]
    t0 = time.perf_counter(); c_oracle.infer(y0, lay, float(net.bias), prune=prune, want_activations=False)
    one = time.perf_counter() - t0
    reps = max(1, int(seconds / max(one, 1e-3)))
    t0 = time.perf_counter()
    for _ in range(reps):
        _, _, live = c_oracle.infer(y0, lay, float(net.bias), prune=prune, want_activations=False)
    dt = time.perf_counter() - t0
    return {"value": batch * n * 32.0 * layers * reps / dt, "unit": UNIT, "cores": c_oracle.max_threads(), "kind": "port",
            "sample": f"first {batch} images x first {layers} layers of the workload ({reps} repetitions, {dt:.1f} s; "
                      + ("dead images skipped, OpenMP over images; %d of %d alive after the sample's last layer)" % (int(live[-1]), batch)
                         if prune else "no pruning)"),
            "seconds": dt}


def run_reference_gpu_loop(cfg, pattern, _unused=None):
    """The reference's own structure-agnostic GPU inference loop (src/microbenchmark/snig.cu, built as
    oracle/_ref/ref_snig from the reference's sources) on a bounded sample of the workload, on this GPU:
    its summed kernel time as it prints it, and this library's time on the same sample."""
    from graphchallenge21_b200 import SpDNN
    from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images
    from oracle import ref_snig
    if pattern != "radix16" or ref_snig.available() is None:
        return None
    n = cfg["neurons"]
    batch = min(cfg["batch"], max(256, (1 << 25) // n))          # 32768 images at N=1024 ... 512 at N=65536
    layers = min(cfg["layers"], 60)
    net = SyntheticNetwork(n, layers, pattern)
    y0 = synthetic_images(n, batch)
    try:
        ref = ref_snig.run(net, layers, y0, timeout=300.0)
    except Exception as e:              # the baseline is a courtesy line; say why it is missing
        return {"unavailable": str(e)[:200]}
    with SpDNN(n, layers, float(net.bias)) as g:
        g.set_network(net)
        ms = []
        for _ in range(3):
            g.set_input_dense(y0)
            ms.append(g.infer().infer_ms)
        ours_live = g.layer_live().copy()
        same = bool(np.array_equal(ours_live, ref["live"]))
    edges = batch * n * 32.0 * layers
    return {"kernel": "snig_inference (src/microbenchmark/snig.cu:19-120), host loop :211-255", "value": edges / (ref["kernel_ms"] * 1e-3),
            "unit": UNIT, "kernel_ms": ref["kernel_ms"], "sec_size": ref["sec_size"],
            "sample": f"first {batch} images x first {layers} layers of the workload; sum of the per-layer kernel times it prints",
            "ours_same_sample": {"value": edges / (min(ms) * 1e-3), "layer_loop_ms": min(ms)},
            "survivor_counts_equal_ours": same, "survivors_after_last_layer_equal_ours": bool(ours_live[-1] == ref["live"][-1]),
            "layers_with_other_counts": int(np.count_nonzero(ours_live != ref["live"])),
            "why_counts_can_differ": "snig_inference starts every sum from the bias and accumulates with unordered shared-memory atomics "
                                     "(snig.cu:72-74, 98); the reference's CPU loop and its all_network.cu kernels, which this library follows "
                                     "bit for bit, sum from 0.0 and add the bias last (cpu_spmm_fuse.h:46, all_network.cu:57). An activation that "
                                     "is an exact zero in one order can be a rounding residue below 1e-5 in the other, so an image whose only "
                                     "non-zero activations are such residues is counted one layer longer by one of the two",
            "survivors_after_layer": {str(i): [int(ref["live"][i]), int(ours_live[i])] for i in sorted({0, 1, 2, 4, 8, 16, 32, layers - 1}) if i < layers},
            "first_layer_that_differs": None if same else int(np.nonzero(ours_live != ref["live"])[0][0]),
            "note": "all_network.cu's pattern-specific kernels read their work list past its end and are not run on shared GPUs"}


def main_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if rank != 0:
        return 0
    cfg = workload(args, world)
    per_step = args.cpu_seconds or max(2.0, min(20.0, 90.0 / max(args.steps + args.warmup, 1)))
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
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg, args, world, None),
        "note": "reference CPU loop on the host cores; each step is a bounded sample of the workload",
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))
    return 0


def workload_config(cfg, args, world, extra):
    n, L, B = cfg["neurons"], cfg["layers"], cfg["batch"]
    total = B if args.scaling == "strong" else B * world
    out = {"workload": f"N={n} L={L} batch={total}, pattern {args.pattern}", "neurons": n, "layers": L, "batch_total": total,
           "pattern": args.pattern, "inputs": args.inputs,
           "parallelism": f"batch split over {world} GPU(s) in contiguous slices, weights replicated"}
    if extra:
        out.update(extra)
    return out


# ---- our arm -----------------------------------------------------------------------------------

def per_layer_line(net, y_dev, cfg, device, stream, first_id, want_survivors, pattern, passes=2):
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
        fig = (profile_figures(n, pattern, "layer_kernel") or [{}])[0]
        per_launch = r.algorithmic_bytes / max(int(r.loop_launches), 1)
        # DRAM bytes per launch from the committed capture: as captured where the capture is this workload's steady state,
        # else the captured launch's ratio of traffic to algorithmic bytes applied to this run's average launch
        traffic = fig.get("dram_bytes_per_launch")
        if traffic is None and fig.get("traffic_over_algorithmic") is not None:
            traffic = fig["traffic_over_algorithmic"] * per_launch
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json hbm_gbs)", "kernel": "layer_kernel",
                "launches_per_pass": int(r.loop_launches), "layer_loop_ms": loop_ms, "us_per_layer": loop_ms * 1e3 / L,
                "passes": passes, "traffic": traffic, "traffic_source": fig.get("source"),
                "traffic_over_algorithmic": fig.get("traffic_over_algorithmic"),
                "algorithmic_bytes_per_launch": per_launch,
                "note": "one launch per layer, activations in HBM between layers; layers after the first few work on the "
                        "survivors only, whose two activation buffers (%.0f MB) can partly stay in the 126 MB L2"
                        % (2.0 * r.survivors * n * 4 / 1e6)}
    finally:
        g.close()


def run_workload(args, cfg, world, rank, local, stream, sampler, headline):
    """Times one workload on this rank's slice; returns the per-rank measurements (times in ms)."""
    import torch
    import torch.distributed as dist
    from graphchallenge21_b200 import SpDNN, SyntheticNetwork, synthetic_images
    from graphchallenge21_b200.network import gather_categories, pack_bits, shard_bounds

    n, L, B = cfg["neurons"], cfg["layers"], cfg["batch"]
    if args.scaling == "strong":
        lo, hi = shard_bounds(B, world, rank)     # contiguous slices of one batch, as src/multi_gpu.cpp:146-151
    else:
        lo, hi = rank * B, (rank + 1) * B
    b = hi - lo
    net = SyntheticNetwork(n, L, args.pattern)
    g = SpDNN(n, L, float(net.bias), device=local)
    g.set_network(net)
    info = g.layer_info(min(1, L - 1))
    if args.inputs == "mixed":
        from graphchallenge21_b200.generator import mixed_density_images
        y_np = mixed_density_images(n, b, first_image=lo)
    else:
        y_np = synthetic_images(n, b, first_image=lo, threads=max(1, min(8, (os.cpu_count() or 8) // max(world, 1))))
    bits_host = torch.from_numpy(pack_bits(y_np)).pin_memory()
    y_dev = torch.from_numpy(y_np).cuda()
    bits_dev = bits_host.cuda()
    # the same images as the reference's input file holds them: (img, neuron) triplets, value 1
    coo_img = coo_neu = None
    nnz = int(np.count_nonzero(y_np))
    if nnz * 8 <= (3 << 29):
        img_np, neu_np = np.nonzero(y_np)
        coo_img = torch.from_numpy(img_np.astype(np.int32)).pin_memory()
        coo_neu = torch.from_numpy(neu_np.astype(np.int32)).pin_memory()
        del img_np, neu_np
    y_host = torch.from_numpy(y_np).pin_memory() if b * n * 4 <= (1 << 30) else None
    del y_np
    g.set_stream(stream.cuda_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(enqueue, steps, before_end=None):
        """`steps` calls of enqueue() bracketed by barrier + synchronize; device time by events on the stream
        (before_end: called before the closing event is recorded, e.g. to make the stream wait for another one)."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record(stream)
        out = None
        for _ in range(steps):
            out = enqueue()
        if before_end is not None:
            before_end()
        e1.record(stream)
        while not e1.query():        # wait without holding the interpreter lock, so that the clock sampler runs
            time.sleep(0)
        barrier()
        if headline and sampler is not None:
            sampler.window(t0, time.perf_counter())
        return e0.elapsed_time(e1), out

    def step_dense_resident():
        g.set_input_dense(y_dev, lo)
        g.infer_async()

    def step_bits_resident():
        g.set_input_bits(bits_dev, lo)
        g.infer_async()

    gather_s = [0.0]
    cap = (B + world - 1) // world if args.scaling == "strong" else B        # the largest shard: every rank knows it

    def step_e2e(kind):
        if kind == "bits":
            g.set_input_bits(bits_host, lo)                                       # H2D of batch x N/8 bytes inside
        elif kind == "dense":
            g.set_input_dense(y_host, lo)                                         # H2D of batch x N floats inside
        else:
            g.set_input_coo(coo_img.numpy(), coo_neu.numpy(), None, b, lo, index_base=0)   # H2D of the triplets inside
        g.infer_async()
        mine = g.categories()                     # D2H of this rank's result (waits for the step)
        t0 = time.perf_counter()
        everyone = gather_categories(np.asarray(mine).copy(), capacity=cap)      # the one exchange step: all-gather of the survivors
        gather_s[0] += time.perf_counter() - t0
        return everyone

    for _ in range(max(args.warmup, 1)):
        step_dense_resident()
        g.sync()
    # -- value: inputs resident in HBM as the reference keeps them (dense fp32), device-timed
    ms, _ = timed(step_dense_resident, args.steps)
    r = g.sync()                 # statistics of the last timed pass (every pass does the same work)
    res = {"ms": ms, "infer_ms": r.infer_ms, "prep_ms": r.prepare_ms, "algo_bytes": r.algorithmic_bytes,
           "launches": int(r.kernel_launches), "loop_launches": int(r.loop_launches), "group": int(r.resident_group),
           "survivors": int(r.survivors), "live": g.layer_live().copy(), "b": b, "lo": lo, "classes": info["classes"]}
    cats_dense = np.asarray(g.categories()).copy()
    # -- the same with the input resident as a bit matrix
    step_bits_resident(); g.sync()
    res["ms_bits"], _ = timed(step_bits_resident, args.steps)
    rb = g.sync()
    res["prep_ms_bits"] = rb.prepare_ms
    assert np.array_equal(np.asarray(g.categories()), cats_dense), "bit-matrix input gave other categories"
    if args.only_value:
        res.update({"ms_e2e": res["ms_bits"], "gather_ms": 0.0, "e2e_prep_ms": rb.prepare_ms, "h2d_bits": 0, "d2h": 0,
                    "all_cats": cats_dense, "net": net, "y_dev": y_dev})
        g.close()
        return res
    # -- e2e: host buffers in, category list of the whole job out; copies and the gather inside the timed region
    step_e2e("bits")
    gather_s[0] = 0.0
    res["ms_e2e"], all_cats = timed(lambda: step_e2e("bits"), args.steps)
    res["gather_ms"] = gather_s[0] * 1e3
    res["e2e_prep_ms"] = g.sync().prepare_ms
    res["h2d_bits"] = int(bits_host.numel())
    res["d2h"] = int(len(cats_dense) * 4 + (L + 1) * 16 + L * 4 + 4)
    res["all_cats"] = np.asarray(all_cats).copy()
    if coo_img is not None:
        step_e2e("coo")
        res["ms_e2e_coo"], c2 = timed(lambda: step_e2e("coo"), args.steps)
        res["h2d_coo"] = int(coo_img.numel() * 8)
        assert np.array_equal(c2, res["all_cats"]), "triplet input gave other categories"
    if headline and not args.no_two_contexts:
        # the same end-to-end step with TWO contexts taking turns (own stream and buffers each, the weights held twice):
        # the host->device copy of step k+1's input runs while step k's pass computes
        g2 = SpDNN(n, L, float(net.bias), device=local)
        try:
            g2.set_network(net)
            stream2 = torch.cuda.Stream()
            g2.set_stream(stream2.cuda_stream)
            ctx = [g, g2]

            def enqueue(c):
                c.set_input_bits(bits_host, lo)
                c.infer_async()

            for c in ctx:                      # graph build and warm-up of both
                enqueue(c)
                c.categories()
            state = {"k": 0}

            def step_two():
                k = state["k"]
                if k == 0:
                    enqueue(ctx[0])
                if k + 1 < args.steps:
                    enqueue(ctx[(k + 1) % 2])                  # step k+1's copy and pass are queued before step k is waited for
                mine = ctx[k % 2].categories()                 # D2H of step k's result (waits for step k only)
                state["k"] = k + 1
                return gather_categories(np.asarray(mine).copy(), capacity=cap)

            ms2, c4 = timed(step_two, args.steps, before_end=lambda: stream.wait_stream(stream2))
            res["ms_e2e_two"] = ms2
            assert np.array_equal(c4, res["all_cats"]), "the two-context loop returned other categories"
        finally:
            g2.close()
    if y_host is not None:
        step_e2e("dense")
        res["ms_e2e_dense"], c3 = timed(lambda: step_e2e("dense"), args.steps)
        res["h2d_dense"] = int(b * n * 4)
        assert np.array_equal(c3, res["all_cats"]), "dense host input gave other categories"
    res["net"], res["y_dev"] = net, y_dev
    g.close()
    return res


def reduce_max(vals, world):
    import torch
    import torch.distributed as dist
    t = torch.tensor([v if v is not None else 0.0 for v in vals], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) if v is not None else None for x, v in zip(t.tolist(), vals)]


def gather_ints(v, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return [int(v)]
    t = torch.tensor([int(v)], dtype=torch.int64, device="cuda")
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [int(x.item()) for x in out]


def gather_floats(v, world):
    import torch
    import torch.distributed as dist
    if world == 1:
        return [float(v)]
    t = torch.tensor([float(v)], dtype=torch.float64, device="cuda")
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [float(x.item()) for x in out]


def summarize(args, cfg, world, res, headline):
    """Whole-job figures of one workload (rank 0 uses them); every rank must call it (collectives inside)."""
    n, L = cfg["neurons"], cfg["layers"]
    keys = ["ms", "ms_bits", "ms_e2e", "ms_e2e_coo", "ms_e2e_dense", "gather_ms", "infer_ms", "prep_ms", "ms_e2e_two"]
    mx = dict(zip(keys, reduce_max([res.get(k) for k in keys], world)))
    per_rank_b = gather_ints(res["b"], world)
    per_rank_surv = gather_ints(res["survivors"], world)
    per_rank_ms = gather_floats(res["ms"] / max(args.steps, 1), world)          # the slowest rank sets `value`
    per_rank_loop = gather_floats(res["infer_ms"], world)
    total = sum(per_rank_b)
    edges_step = float(total) * n * 32.0 * L
    steps = args.steps
    peak, peak_kind = peaks()
    loop_ms = res["infer_ms"]
    achieved = res["algo_bytes"] / (loop_ms * 1e-3) / 1e9
    live = res["live"]
    out = {
        "value": edges_step * steps / (mx["ms"] * 1e-3), "ms_per_step": mx["ms"] / steps,
        "config": workload_config(cfg, args, world, {
            "images_per_gpu": per_rank_b, "survivors_per_gpu": per_rank_surv, "survivors_total": int(len(res["all_cats"])),
            "ms_per_step_per_gpu": [round(x, 4) for x in per_rank_ms], "layer_loop_ms_per_gpu": [round(x, 4) for x in per_rank_loop],
            "live_after_layer_rank0": {str(i): int(live[i]) for i in sorted({0, 1, 2, 4, 8, 16, 32, 64, 128, L - 1}) if i < L},
            "classes_per_layer": res["classes"], "resident_input": "dense fp32 batch x N in HBM (the reference's A_d)",
            "l2": ("inputs larger than L2 (%.0f MB per GPU and step), no flush" % (res["b"] * n * 4 / 1e6)) if res["b"] * n * 4 > 126e6
                  else ("input %.0f MB per GPU and step, smaller than L2: the timed passes run back to back, each overwriting "
                        "both activation buffers; no flush" % (res["b"] * n * 4 / 1e6))}),
        "value_bit_matrix_input": {"value": edges_step * steps / (mx["ms_bits"] * 1e-3), "ms_per_step": mx["ms_bits"] / steps,
                                   "note": "the same pass with the input resident in HBM as a bit matrix (N/8 bytes per image)"},
        "e2e": {"value": edges_step * steps / (mx["ms_e2e"] * 1e-3), "unit": UNIT, "h2d_bytes_per_step": res["h2d_bits"],
                "d2h_bytes_per_step": res["d2h"], "ms_per_step": mx["ms_e2e"] / steps, "input_ms": res["e2e_prep_ms"],
                "gather_ms_per_step": mx["gather_ms"] / steps,
                "call": "spdnn_set_input_bits (bit matrix in pinned host memory) + spdnn_infer + spdnn_get_categories + the "
                        "all-gather of every rank's surviving image numbers, all inside the timed region; bytes are per GPU",
                "two_contexts": None if mx["ms_e2e_two"] is None else {
                    "value": edges_step * steps / (mx["ms_e2e_two"] * 1e-3), "ms_per_step": mx["ms_e2e_two"] / steps,
                    "call": "the same calls on two contexts in turn (own stream and buffers each): the copy of step k+1's input "
                            "overlaps step k's pass; every step's H2D, D2H and gather are inside the region"},
                "triplet_input": None if mx["ms_e2e_coo"] is None else {
                    "value": edges_step * steps / (mx["ms_e2e_coo"] * 1e-3), "ms_per_step": mx["ms_e2e_coo"] / steps,
                    "h2d_bytes_per_step": res.get("h2d_coo"),
                    "call": "spdnn_set_input_coo (the input file's img/neuron triplets, pinned host memory)"},
                "dense_input": None if mx["ms_e2e_dense"] is None else {
                    "value": edges_step * steps / (mx["ms_e2e_dense"] * 1e-3), "ms_per_step": mx["ms_e2e_dense"] / steps,
                    "h2d_bytes_per_step": res.get("h2d_dense"),
                    "call": "spdnn_set_input_dense (batch x N fp32, pinned host memory)"}},
        "roofline_input_conversion": {
            "bound": "hbm", "kernel": "dense_to_words_kernel", "achieved": res["b"] * n * (4.0 + 0.125) / (res["prep_ms"] * 1e-3) / 1e9,
            "peak": peak, "unit": "GB/s", "frac": res["b"] * n * (4.0 + 0.125) / (res["prep_ms"] * 1e-3) / 1e9 / peak,
            "ms": res["prep_ms"],
            "note": "the one kernel of the timed pass that streams HBM: the dense fp32 input read once (4 bytes per activation) and "
                    "written as one bit per activation; time by CUDA events around the whole input set-up (it also holds two "
                    "small memsets and three launches that exit at entry for a binary input), rank 0"},
        "gpu_launches": int(res["launches"] * steps),
        "layer_loop_ms": loop_ms, "input_layout_ms": res["prep_ms"], "us_per_layer": loop_ms * 1e3 / L,
    }
    kernel = ("alt2_kernel" if args.pattern == "radix16" else "resident_kernel") if res["group"] else "layer_kernel"
    figs = profile_figures(n, args.pattern)
    fig = figs[0] if figs else {}
    out["roofline"] = {
        "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
        "peak_kind": peak_kind + " copy bandwidth (MEASURED_PEAKS.json hbm_gbs)",
        "kernel": fig.get("kernel", kernel), "kernel_form": fig.get("form"), "launches_per_step": res["loop_launches"],
        "avg_launch_us": loop_ms * 1e3 / max(res["loop_launches"], 1),
        "algorithmic_bytes_per_launch": res["algo_bytes"] / max(res["loop_launches"], 1),
        "traffic": fig.get("dram_bytes_per_launch"),
        "bound_actual": "the FP32 pipe (float form: 32 dependent adds per output, see fp32_pipe) and the latency of a dependent chain per layer "
                        "(bit form): activations stay in shared memory across the layers of a launch, one bit per activation once "
                        "saturated, so the HBM roofline of the per-layer formulation does not bind and frac exceeds 1; the kernels "
                        "that do stream HBM are in roofline_input_conversion and roofline_per_layer_kernel"
                        if res["group"] else "hbm",
        "issue_slots_busy_pct": fig.get("issue_slots_busy_pct"), "sm_active_cycles_per_layer": fig.get("sm_active_cycles_per_layer"),
        "ncu_source": fig.get("source"),
        # the resource that does bind the dominant kernel's float form: additions per second against the FP32 pipe's peak
        # and against what the same inner loop reaches alone (graphchallenge21_b200/bin/add_chain_ceiling)
        "fp32_pipe": fig.get("fp32_pipe"),
        "ncu_kernels": [{k: r.get(k) for k in ("kernel", "form", "issue_slots_busy_pct", "sm_active_cycles_per_layer",
                                                "dram_bytes_per_launch", "scale", "source")} for r in figs],
        "ncu_note": "figures from committed ncu captures of a smaller case of the same kernels, scaled as each record says; "
                    "not measured in this run",
    }
    return out


def main_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = workload(args, world)
    # everything the library enqueues goes to ONE explicit stream, and the timing events are
    # recorded on that same stream (the legacy default stream has handle 0, which the library
    # reads as "use your own stream")
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler is not None:
        sampler.prepare()
        # the timed loops are milliseconds of Python that enqueues work: let the polling thread
        # preempt them (the default switch interval of the interpreter is 5 ms)
        sys.setswitchinterval(1e-4)
        sampler.start()
    res = run_workload(args, cfg, world, rank, local, stream, sampler, True)
    clocks = sampler.stop() if sampler is not None else None
    head = summarize(args, cfg, world, res, True)
    out = None
    if rank == 0:
        out = {"metric": METRIC, "value": head.pop("value"), "unit": UNIT, "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": head.pop("ms_per_step"), "higher_is_better": True, "scaling": args.scaling,
               "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
        out.update(head)
        out["clocks"] = clocks
    if args.only_value:
        args.no_per_layer_line = args.no_also = args.no_cpu_baseline = True
        if rank == 0:
            out["e2e"] = None
    if world == 1 and not args.no_per_layer_line:
        out["roofline_per_layer_kernel"] = per_layer_line(res["net"], res["y_dev"], cfg, local, stream, res["lo"], res["survivors"],
                                                          args.pattern)
    res = None
    torch.cuda.empty_cache()
    # -- other workloads beside the headline: the N=16384 network on 8 GPUs, the N=1024 network on one
    also = []
    if not args.no_also and args.config is None and args.neurons is None:
        also = [3] if world >= 8 else ([1] if world == 1 else [])
    for idx in also:
        c2 = workload(args, world, index=idx)
        r2 = run_workload(args, c2, world, rank, local, stream, None, False)
        s2 = summarize(args, c2, world, r2, False)
        r2 = None
        torch.cuda.empty_cache()
        if rank == 0:
            out.setdefault("also", {})["config%d" % idx] = {k: s2[k] for k in ("value", "ms_per_step", "config", "e2e", "layer_loop_ms",
                                                                                "us_per_layer", "value_bit_matrix_input")}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cb = run_cpu_reference(cfg, args.pattern, args.cpu_seconds or 10.0)
        cb.pop("seconds", None)
        out["cpu_baseline"] = cb
        cp = run_cpu_port(cfg, args.pattern, args.cpu_seconds or 10.0, prune=True)
        cp.pop("seconds", None)
        out["cpu_baseline_pruned"] = cp
        out["reference_gpu_loop"] = run_reference_gpu_loop(cfg, args.pattern, None)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    a = parse()
    sys.exit(main_reference(a) if a.impl == "reference" else main_ours(a))
