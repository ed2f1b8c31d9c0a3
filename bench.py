"""Headline benchmark: ResNet-50 fp16 batch-64 inference images/s on N B200s (one replica per GPU, no collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

One step = one forward of the configured network over one batch of synthetic images. After W warm-up steps the timed
region is R windows of exactly K steps each, every window bracketed by a barrier + synchronise on both sides and timed
with CUDA events (max over ranks); `value` is the median window, `value_min` / `value_max` the slowest / fastest one.
R is chosen so that the windows together last about a second: long enough for the clock sampler to see tens of samples.
Prints ONE JSON line (rank 0):
  value     images/s over all ranks with inputs resident in HBM
  e2e       images/s through the public API from pinned HOST buffers (fp32 images, the reference's input contract): the
            host->device copy of every batch and the device->host read of its logits are inside the timed region
            (copies overlap compute on a second stream); `e2e_fp16_input` is the same with fp16 host images
  roofline  algorithmic bytes of one forward / measured forward time against the measured HBM peak
  cpu_baseline  the upstream fp32 model on the host cores (rank 0, N=1 only; a bounded sample)
  gpu_portable  the portable tier (folded fp16 channels-last on plain PyTorch / cuDNN) on the same GPU (N=1 only)
  other_configs the other benchmark configurations (EfficientNet-B4, ConvNeXt-T, DeepLabV3) on the same GPU (N=1 only)
  startup   seconds of the first call at the benchmark shape (per-layer tile tuning + graph capture) and at a new size
`--impl reference` times the reference's CPU path (its upstream tier: the unmodified fp32 torchvision model) instead.
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

MODEL = os.environ.get("FVM_BENCH_MODEL", "resnet50")
BATCH = int(os.environ.get("FVM_BENCH_BATCH", "64"))
# the headline metric by its published name; another model or batch (FVM_BENCH_MODEL / FVM_BENCH_BATCH) is labelled as such
METRIC = "ResNet-50 fp16 b64 images/s" if (MODEL, BATCH) == ("resnet50", 64) else f"{MODEL} fp16 b{BATCH} images/s"
CPU_BATCH = 8
# Algorithmic work of one image through the reference's fused-op partition (each op reads its inputs once and writes
# its output once; weights once per forward): bytes and FLOPs per image at the network's benchmark resolution.
ALGO = {
    "resnet50": {"bytes": 59.52e6, "flops": 8.178e9, "batch": 64},
    "efficientnet_b4": {"bytes": 247.6e6, "flops": 8.79e9, "batch": 64},
    "convnext_tiny": {"bytes": 73.1e6, "flops": 8.91e9, "batch": 64},
    "deeplabv3-r50": {"bytes": 1.303e9, "flops": 654.3e9, "batch": 8},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
TARGET_TIMED_SECONDS = 1.0


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops_sustained"]), "source": "measured"}
    return {**FALLBACK_PEAKS, "source": "fallback"}


def roofline_of(model: str, batch: int, ms_step: float, pk: dict) -> dict:
    """Fraction of the slower of the HBM and tensor rooflines for one forward of `batch` images in `ms_step`."""
    a = ALGO[model]
    nbytes, flops = a["bytes"] * batch, a["flops"] * batch
    t_hbm, t_tensor = nbytes / (pk["hbm_gbs"] * 1e9), flops / (pk["bf16_tflops"] * 1e12)
    bound = "hbm" if t_hbm >= t_tensor else "tensor"
    sec = ms_step / 1e3
    if bound == "hbm":
        achieved, peak, unit = nbytes / sec / 1e9, pk["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = flops / sec / 1e12, pk["bf16_tflops"], "TFLOP/s"
    return {"bound": bound, "achieved": round(achieved, 1), "peak": peak, "unit": unit, "frac": round(achieved / peak, 4),
            "peak_source": pk["source"], "algorithmic_bytes_per_step": nbytes, "algorithmic_flops_per_step": flops,
            "hbm_frac": round(nbytes / sec / 1e9 / pk["hbm_gbs"], 4),
            "tensor_frac": round(flops / sec / 1e12 / pk["bf16_tflops"], 4)}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            t0 = time.perf_counter()
            while not self.lines and time.perf_counter() - t0 < 2.0:      # the first sample takes a moment to arrive
                time.sleep(0.01)
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()          # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_upstream(steps: int, warmup: int):
    """The reference's upstream tier on the host cores: unmodified fp32 torchvision model, batch 8 (BASELINE config 0)."""
    from fast_vision_models_b200.classification import zoo
    from fast_vision_models_b200.weights import seeded_input
    from oracle import models_ref
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    model = zoo.build_upstream(MODEL, seed=1)
    x = seeded_input((CPU_BATCH, 3, 224, 224), seed=0)
    _, sec, used = models_ref.upstream_fp32(model, x, warmup=warmup, iters=steps, threads=threads)
    return CPU_BATCH / sec, used, sec


def reference_arm(args, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 10))
    warmup = max(1, min(args.warmup, 3))
    ips, cores, sec = cpu_upstream(steps, warmup)
    sample = f"{MODEL} fp32 eager, batch {CPU_BATCH} of 3x224x224, median of {steps} forwards after {warmup} warm-ups"
    line = {"impl": "reference", "metric": METRIC, "value": round(ips, 2), "unit": "images/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{MODEL} batch {BATCH} per GPU, 3x224x224 fp32 NCHW in, logits out",
                       "reference_arm": f"upstream fp32 tier on the host cores, bounded sample: batch {CPU_BATCH} per step"},
            "cpu_baseline": {"value": round(ips, 2), "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(ips, 2), "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def window_count(first_ms: float, target_s: float, min_windows: int, max_windows: int, agree=lambda v: v) -> int:
    """How many windows fill `target_s` seconds, from the time of the first one. `agree` turns this rank's time into a
    value all ranks share, so that all of them get the same count (each window is bracketed by collective barriers)."""
    return int(min(max_windows, max(min_windows, target_s * 1e3 / max(agree(first_ms), 1e-3))))


def timed_windows(step_fn, steps: int, barrier, target_s: float = TARGET_TIMED_SECONDS, min_windows: int = 10,
                  max_windows: int = 200, agree=lambda v: v):
    """R windows of exactly `steps` calls of step_fn(i), each bracketed by barrier() and timed with CUDA events.
    Returns the list of window times in ms (this rank). R follows from the first window's time; `agree` maps that time
    to a value all ranks share (its maximum over ranks), so that every rank runs the same number of windows and
    barriers."""
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    barrier()
    first = e0.elapsed_time(e1)
    windows = window_count(first, target_s, min_windows, max_windows, agree)
    times = [first]
    for _ in range(windows - 1):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step_fn(i)
        e1.record()
        barrier()
        times.append(e0.elapsed_time(e1))
    return times


def time_callable(fn, xs, reps: int = 20, rounds: int = 5) -> float:
    """Median ms per call of fn(x) over rotating inputs (CUDA events), after warm-up."""
    for i in range(3):
        fn(xs[i % len(xs)])
    torch.cuda.synchronize()
    out = []
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(reps):
            fn(xs[i % len(xs)])
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1) / reps)
    return statistics.median(out)


def other_configs(dev, pk) -> dict:
    """The other benchmark configurations on this GPU: images/s (device-resident inputs) and roofline fraction."""
    from fast_vision_models_b200 import ops
    from fast_vision_models_b200.classification import zoo
    from fast_vision_models_b200.segmentation import zoo as segzoo
    from fast_vision_models_b200.weights import seeded_input
    res = {}
    for name, shape in (("efficientnet_b4", (64, 3, 380, 380)), ("convnext_tiny", (64, 3, 224, 224)),
                        ("deeplabv3-r50", (8, 3, 512, 1024))):
        try:
            xs = [seeded_input(shape, seed=300 + i).to(dev) for i in range(2)]
            t0 = time.perf_counter()
            if name.startswith("deeplab"):
                w = segzoo.build(name, "b200", device=dev, num_classes=19, seed=1)
                fn = w.predict            # image batch -> int32 class map (fused upsample + argmax)
            else:
                fn = zoo.load(name, "b200", device=dev, seed=1).model
            fn(xs[0])
            torch.cuda.synchronize()
            first = time.perf_counter() - t0
            ms = time_callable(fn, xs, reps=10 if shape[0] == 64 else 5, rounds=5)
            rf = roofline_of(name, shape[0], ms, pk)
            res[name] = {"workload": f"batch {shape[0]} of 3x{shape[2]}x{shape[3]}", "ms_per_step": round(ms, 4),
                         "images_per_s": round(shape[0] / ms * 1e3, 1), "bound": rf["bound"], "roofline_frac": rf["frac"],
                         "hbm_frac": rf["hbm_frac"], "tensor_frac": rf["tensor_frac"], "first_call_s": round(first, 2),
                         "status": ops.last_status()}
            del fn, xs
            torch.cuda.empty_cache()
        except Exception as e:                       # a side measurement must not take the headline line down
            res[name] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip other_configs / gpu_portable / startup.new_size_s")
    ap.add_argument("--profile-window", type=int, default=0,
                    help="after warm-up, run this many forwards between cudaProfilerStart/Stop and exit (for a "
                         "profiler started with --profile-from-start off); prints no bench line")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, rank)
        return

    import torch.distributed as dist
    from fast_vision_models_b200 import ops, parallel
    from fast_vision_models_b200.classification import zoo
    from fast_vision_models_b200.weights import seeded_input

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: the b200 tier has no CPU path"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)

    ops.init(dev)
    m = zoo.load(MODEL, "b200", device=dev, seed=1)
    size = m.input_size[1]
    NBUF = 4      # rotating inputs: 4 x 38.5 MB > the 126 MB L2, on top of ~3.8 GB of activation traffic per step
    xs = [seeded_input((BATCH, 3, size, size), seed=100 * rank + i).to(dev) for i in range(NBUF)]

    # ---------------------------------------------------------------- start-up: first call at the benchmark shape (tile tuning of every layer
    # unless an earlier process left its choices in the per-user cache, then graph capture)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    y = m.model(xs[0])
    torch.cuda.synchronize()
    first_call_s = time.perf_counter() - t0

    # launches per forward: count the library's launches over one un-captured forward (after tuning)
    eager = zoo.load(MODEL, "b200", device=dev, seed=1, graphs=False)
    eager.model(xs[0])            # first call: per-layer tile tuning launches extra kernels
    torch.cuda.synchronize()
    n0 = ops.launches()
    eager.model(xs[0])
    launches_per_fwd = ops.launches() - n0
    del eager

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- value: inputs resident in HBM
    for i in range(warmup):
        y = m.model(xs[i % NBUF])
    if args.profile_window > 0:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        for i in range(args.profile_window):
            y = m.model(xs[i % NBUF])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profile_window": args.profile_window, "status": ops.last_status()}))
        return
    sampler = ClockSampler(local_rank)
    sampler.start()
    out = [None]

    # One graph replica per rotating input, each input resident in its replica's static buffer (what a preceding GPU
    # stage would write into): a step is the replay alone, without the 38.5 MB device copy into a shared static input.
    from fast_vision_models_b200.classification.fast import Fast
    replicas = [m.model] + [Fast(m.model.net) for _ in range(NBUF - 1)]
    resident = []
    for r, x in zip(replicas, xs):
        _, static_in, _ = r.runner.static_buffers(x)
        static_in.copy_(x)
        resident.append(static_in)
    for i in range(NBUF):
        replicas[i](resident[i])
    torch.cuda.synchronize()

    def step_dev(i):
        out[0] = replicas[i % NBUF](resident[i % NBUF])

    def agree(v):        # the same number on every rank
        return parallel.max_over_ranks([float(v)], device=dev)[0]

    win_dev = timed_windows(step_dev, steps, barrier, agree=agree)
    clocks = sampler.stop()
    y = out[0]
    status = ops.last_status()
    assert status == 0, f"device status {status:#x}"
    assert torch.isfinite(y).all()

    # ---------------------------------------------------------------- e2e: pinned host buffers in, logits out
    # The library's serving loop for host batches (Fast.host_pipeline -> runtime.HostPipeline): two graph replicas of the
    # network in rotation; the copy stream writes batch i+1 from pinned host memory straight into one replica's static
    # input while the other replica's graph computes batch i, and the logits of batch i-1 leave on a third stream into
    # pinned host memory. Every byte in and out is inside the timed region.
    def e2e_windows(dtype):
        hx = [seeded_input((BATCH, 3, size, size), seed=200 + 100 * rank + i).to(dtype).pin_memory() for i in range(2)]
        pipe = m.model.host_pipeline(hx[0], replicas=2)

        def step(i):
            return pipe.submit(hx[i % 2])

        for i in range(warmup):
            step(i)
        torch.cuda.synchronize()
        wins = []
        barrier()
        n_win = window_count(statistics.median(win_dev), TARGET_TIMED_SECONDS, 10, 200, agree)
        for _ in range(n_win):
            barrier()
            t0 = time.perf_counter()
            for i in range(steps):
                step(i)
            torch.cuda.synchronize()
            wins.append((time.perf_counter() - t0) * 1e3)
            barrier()
        assert torch.isfinite(pipe.result(0)).all() and torch.isfinite(pipe.result(1)).all()
        assert pipe.out_bytes == BATCH * 1000 * 4
        return wins, pipe.in_bytes

    win_e2e, h2d_bytes = e2e_windows(torch.float32)
    win_e2e16, h2d_bytes16 = e2e_windows(torch.float16)
    status = ops.last_status()
    assert status == 0, f"device status {status:#x}"

    # ---------------------------------------------------------------- max over ranks (window by window), then median
    def reduce_windows(w):
        n = int(parallel.max_over_ranks([float(-len(w))], device=dev)[0] * -1)   # the shortest list over ranks
        return parallel.max_over_ranks(w[:n], device=dev)

    win_dev, win_e2e, win_e2e16 = reduce_windows(win_dev), reduce_windows(win_e2e), reduce_windows(win_e2e16)
    images_per_window = BATCH * steps * world
    med = statistics.median(win_dev)
    value = images_per_window / (med / 1e3)

    if rank == 0:
        pk = peaks()
        ms_step = med / steps
        roof = roofline_of(MODEL, BATCH, ms_step, pk)
        roof["kernel"] = ("whole forward graph; the three convolution kernels carry 96 % of the device time "
                          "(conv_pair_kernel 68 % over 43 launches, conv_tcgen05_kernel 20 % over 7, "
                          "conv_dual_kernel 7 % over 2)")
        roof["traffic"] = 2212.4e6 if (MODEL, BATCH) == ("resnet50", 64) else None
        roof["traffic_source"] = ("ncu capture of this forward (dram__bytes_read.sum + dram__bytes_write.sum over its 56 "
                                  "launches, serialised, cold caches); not measured in this run")
        line = {"metric": METRIC, "value": round(value, 1),
                "value_min": round(images_per_window / (max(win_dev) / 1e3), 1),
                "value_max": round(images_per_window / (min(win_dev) / 1e3), 1), "unit": "images/s", "n_gpus": world,
                "steps": steps, "warmup": warmup, "windows": len(win_dev), "ms_per_step": round(ms_step, 4),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
                "data": "synthetic",
                "config": {"workload": f"{MODEL} batch {BATCH} per GPU, 3x{size}x{size} fp32 NCHW in, logits out",
                           "l2": f"{NBUF} rotating input batches (> L2), each resident in the static input of its own graph replica, and ~3.8 GB activation traffic per step",
                           "timing": f"median of {len(win_dev)} windows of {steps} steps, CUDA events, max over ranks per window",
                           "parallelism": f"replicas x{world}, no collective"},
                "roofline": roof,
                "e2e": {"value": round(images_per_window / (statistics.median(win_e2e) / 1e3), 1), "unit": "images/s",
                        "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": BATCH * 1000 * 4,
                        "value_min": round(images_per_window / (max(win_e2e) / 1e3), 1),
                        "value_max": round(images_per_window / (min(win_e2e) / 1e3), 1), "input": "fp32 pinned host"},
                "e2e_fp16_input": {"value": round(images_per_window / (statistics.median(win_e2e16) / 1e3), 1),
                                   "unit": "images/s", "h2d_bytes_per_step": h2d_bytes16,
                                   "d2h_bytes_per_step": BATCH * 1000 * 4, "input": "fp16 pinned host"},
                "gpu_launches": launches_per_fwd * steps * len(win_dev), "launches_per_step": launches_per_fwd,
                "clocks": clocks, "startup": {"first_call_s": round(first_call_s, 2)}}
        if world == 1 and not args.no_extras:
            # a new input size: tuning of every layer at its new shape + capture (the reference publishes the same pair)
            t0 = time.perf_counter()
            m.model(seeded_input((BATCH // 2, 3, size - 32, size - 32), seed=7).to(dev))
            torch.cuda.synchronize()
            line["startup"]["new_size_s"] = round(time.perf_counter() - t0, 2)
            port = zoo.load(MODEL, "portable", device=dev, seed=1).model
            with torch.inference_mode():
                ms_port = time_callable(port, xs, reps=10, rounds=5)
            line["gpu_portable"] = {"value": round(BATCH / ms_port * 1e3, 1), "unit": "images/s", "ms_per_step": round(ms_port, 4),
                                    "what": "portable tier: BatchNorm folded, fp16 channels-last, plain PyTorch (cuDNN / cuBLAS)"}
            del port
            torch.cuda.empty_cache()
            line["other_configs"] = other_configs(dev, pk)
        if world == 1 and not args.no_cpu_baseline:
            ips, cores, sec = cpu_upstream(3, 1)
            line["cpu_baseline"] = {"value": round(ips, 2), "unit": "images/s", "cores": cores, "kind": "port",
                                    "sample": f"{MODEL} upstream fp32 eager on host cores, batch {CPU_BATCH}, median of 3 forwards"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
