"""Headline benchmark: ResNet-50 fp16 batch-64 inference images/s on N B200s (one replica per GPU, no collective).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

One step = one forward of the configured network over one batch of synthetic images. Prints ONE JSON line (rank 0):
  value     images/s over all ranks with inputs resident in HBM (CUDA events, max over ranks)
  e2e       images/s through the public API from pinned HOST buffers: the host->device copy of every batch and the
            device->host read of its logits are inside the timed region (copies overlap compute on a second stream)
  roofline  algorithmic bytes of one forward / measured forward time against the measured HBM peak
  cpu_baseline  the upstream fp32 model on the host cores (rank 0, N=1 only; a bounded sample)
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
CPU_BATCH = 8
# Algorithmic work of one image through the reference's fused-op partition of ResNet-50 at 224x224 (each op reads its
# inputs once and writes its output once; weights once per forward of 64 images): 59.52 MB and 8.178 GFLOP per image.
ALGO_BYTES_PER_IMAGE = {"resnet50": 59.52e6}
ALGO_FLOPS_PER_IMAGE = {"resnet50": 8.178e9}
# DRAM traffic of one 64-image forward from an ncu capture of the replayed graph (dram__bytes_read.sum +
# dram__bytes_write.sum summed over its 59 launches; profiles/resnet50_b64_forward_launches.md).
NCU_TRAFFIC_PER_STEP = {("resnet50", 64): 2486.9e6}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops_sustained"]), "source": "measured"}
    return {**FALLBACK_PEAKS, "source": "fallback"}


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
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
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
    line = {"impl": "reference", "metric": "ResNet-50 fp16 b64 images/s", "value": round(ips, 2), "unit": "images/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{MODEL} batch {BATCH} per GPU, 3x224x224 fp32 NCHW in, logits out",
                       "reference_arm": f"upstream fp32 tier on the host cores, bounded sample: batch {CPU_BATCH} per step"},
            "cpu_baseline": {"value": round(ips, 2), "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": round(ips, 2), "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
    from fast_vision_models_b200 import ops
    from fast_vision_models_b200.classification import zoo
    from fast_vision_models_b200.weights import seeded_input

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: the b200 tier has no CPU path"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    steps = args.steps

    ops.init(dev)
    m = zoo.load(MODEL, "b200", device=dev, seed=1)
    size = m.input_size[1]
    NBUF = 4      # rotating inputs: 4 x 38.5 MB > the 126 MB L2, on top of ~3.8 GB of activation traffic per step
    xs = [seeded_input((BATCH, 3, size, size), seed=100 * rank + i).to(dev) for i in range(NBUF)]

    # launches per forward: count the library's launches over one un-captured forward
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
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        y = m.model(xs[i % NBUF])
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1)
    clocks = sampler.stop()
    status = ops.last_status()
    assert status == 0, f"device status {status:#x}"
    assert torch.isfinite(y).all()

    # ---------------------------------------------------------------- e2e: pinned host buffers in, logits out
    hx = [seeded_input((BATCH, 3, size, size), seed=200 + 100 * rank + i).pin_memory() for i in range(2)]
    hy = [torch.empty((BATCH, 1000), dtype=torch.float32).pin_memory() for _ in range(2)]
    stage = [torch.empty((BATCH, 3, size, size), dtype=torch.float32, device=dev) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream()
    ready = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def e2e_run(n):
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[b])          # the forward that last read stage[b] is done
                stage[b].copy_(hx[b], non_blocking=True)     # host -> device
                ready[b].record(copy_stream)
            main_stream.wait_event(ready[b])
            out = m.model(stage[b])                          # public API call
            consumed[b].record(main_stream)
            hy[b].copy_(out, non_blocking=True)              # device -> host
        torch.cuda.synchronize()

    for b in range(2):
        consumed[b].record(main_stream)
    e2e_run(warmup)
    barrier()
    t0 = time.perf_counter()
    e2e_run(steps)
    barrier()
    sec_e2e = time.perf_counter() - t0

    # ---------------------------------------------------------------- max over ranks
    from fast_vision_models_b200 import parallel
    ms_dev, ms_e2e = parallel.max_over_ranks([ms_dev, sec_e2e * 1e3], device=dev)
    total_images = BATCH * steps * world
    value = total_images / (ms_dev / 1e3)
    e2e_value = total_images / (ms_e2e / 1e3)

    if rank == 0:
        pk = peaks()
        ms_step = ms_dev / steps
        algo_bytes = ALGO_BYTES_PER_IMAGE.get(MODEL, 0.0) * BATCH
        algo_flops = ALGO_FLOPS_PER_IMAGE.get(MODEL, 0.0) * BATCH
        achieved = algo_bytes / (ms_step / 1e3) / 1e9 if algo_bytes else None
        roof = {"bound": "hbm", "achieved": round(achieved, 1) if achieved else None, "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4) if achieved else None,
                "traffic": NCU_TRAFFIC_PER_STEP.get((MODEL, BATCH)),
                "peak_source": pk["source"],
                "kernel": "whole forward graph; conv_tcgen05_kernel is the dominant kernel (see profiles/)",
                "algorithmic_bytes_per_step": algo_bytes, "algorithmic_flops_per_step": algo_flops,
                "tensor_frac": round(algo_flops / (ms_step / 1e3) / 1e12 / pk["bf16_tflops"], 4) if algo_flops else None}
        line = {"metric": "ResNet-50 fp16 b64 images/s", "value": round(value, 1), "unit": "images/s", "n_gpus": world,
                "steps": steps, "warmup": warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)", "data": "synthetic",
                "config": {"workload": f"{MODEL} batch {BATCH} per GPU, 3x{size}x{size} fp32 NCHW in, logits out",
                           "l2": f"{NBUF} rotating input batches (> L2) and ~3.8 GB activation traffic per step",
                           "parallelism": f"replicas x{world}, no collective"},
                "roofline": roof,
                "e2e": {"value": round(e2e_value, 1), "unit": "images/s", "h2d_bytes_per_step": BATCH * 3 * size * size * 4,
                        "d2h_bytes_per_step": BATCH * 1000 * 4},
                "gpu_launches": launches_per_fwd * steps, "launches_per_step": launches_per_fwd, "clocks": clocks}
        if world == 1 and not args.no_cpu_baseline:
            ips, cores, sec = cpu_upstream(3, 1)
            line["cpu_baseline"] = {"value": round(ips, 2), "unit": "images/s", "cores": cores, "kind": "port",
                                    "sample": f"{MODEL} upstream fp32 eager on host cores, batch {CPU_BATCH}, median of 3 forwards"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
