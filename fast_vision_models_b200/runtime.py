"""Launch path: replays a whole forward as one CUDA graph per input shape.

The reference removes per-op CPU cost with a TorchScript trace of the rewritten graph (classification/fast/__init__.py:
58-79) and, for segmentation, an LRU of CUDA graphs (segmentation/fast/ops.py:107-160). Here every op is a plain kernel
launch on the current stream, so the forward is captured once per (shape, dtype, device) and replayed: the ~60-160
launches of a network cost one graph launch. Activation memory comes from the graph's private pool of torch's caching
allocator and is reused between layers.

Image chains. Inference has no cross-image op, so a batch may be cut into `chains` equal groups of images that run
the same network as independent kernel sequences on separate streams inside the one graph. A convolution over a
14x14 or 7x7 map has fewer output tiles than the GPU has SMs, and every kernel boundary drains the machine; with
several chains in flight the tiles of one chain's layer fill the SMs another chain leaves idle. The number of chains
per shape is chosen once by timing the captured graphs (FVM_B200_CHAINS forces it).
"""
from __future__ import annotations

import os
import time
from collections import OrderedDict
from typing import Callable, Optional

import torch

from . import ops

GRAPHS = os.environ.get("FVM_B200_GRAPHS", "1") != "0"   # kill switch in the style of the reference's CLF_* variables
MAX_GRAPHS = int(os.environ.get("FVM_B200_MAX_GRAPHS", "8"))
CHAINS = int(os.environ.get("FVM_B200_CHAINS", "0"))      # 0 = choose by timing
CHAIN_CANDIDATES = (1, 2, 4)


class _Entry:
    __slots__ = ("graph", "static_in", "static_out", "chains", "capture_s", "timings")

    def __init__(self, graph, static_in, static_out, chains, capture_s, timings):
        self.graph, self.static_in, self.static_out = graph, static_in, static_out
        self.chains, self.capture_s, self.timings = chains, capture_s, timings


class GraphRunner:
    """Calls fn(x) through a per-shape CUDA graph. `fn` must be a pure function of x made of stream-ordered launches.
    With `chainable=True`, fn must also treat the images of a batch independently and return a tensor whose first
    dimension is the batch: the runner may then run groups of images as concurrent chains."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], enabled: bool = True, chainable: bool = False,
                 chains: Optional[int] = None):
        self.fn = fn
        self.enabled = enabled and GRAPHS
        self.chainable = chainable
        self.chains = CHAINS if chains is None else int(chains)
        self.cache: "OrderedDict[tuple, _Entry]" = OrderedDict()
        self.last_capture_s = 0.0      # seconds the most recent first call at a new shape spent on warm-up + capture

    # ------------------------------------------------------------------------------------------------ capture
    def _run_chained(self, x: torch.Tensor, chains: int) -> torch.Tensor:
        """fn over `chains` groups of images, group i > 0 on its own stream, joined on the current stream."""
        if chains <= 1:
            return self.fn(x)
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(cur)
        parts = x.chunk(chains, dim=0)
        outs = [None] * len(parts)
        side = [torch.cuda.Stream(device=x.device) for _ in parts[1:]]
        for i, (part, s) in enumerate(zip(parts[1:], side), start=1):
            s.wait_event(fork)
            with torch.cuda.stream(s):
                outs[i] = self.fn(part)
        outs[0] = self.fn(parts[0])
        for s in side:
            cur.wait_stream(s)
        return torch.cat(outs, dim=0)

    def _capture(self, x: torch.Tensor, chains: int):
        static_in = torch.empty_strided(tuple(x.shape), tuple(x.stride()), dtype=x.dtype, device=x.device)
        static_in.copy_(x)
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):
                self._run_chained(static_in, chains)   # warm-up outside capture (first-call set-up and tuning of every op)
        cur.wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = self._run_chained(static_in, chains)
        return graph, static_in, static_out

    @staticmethod
    def _time_graph(graph, reps: int = 8) -> float:
        for _ in range(3):
            graph.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / reps

    def _build(self, x: torch.Tensor) -> _Entry:
        ops.init(x.device)
        t0 = time.perf_counter()
        cands = [1]
        n = x.shape[0]
        if self.chainable and x.dim() >= 1:
            if self.chains > 0:
                cands = [self.chains if n % self.chains == 0 else 1]
            else:
                cands = [c for c in CHAIN_CANDIDATES if n % c == 0 and n // c >= 8] or [1]
        best, timings = None, {}
        for c in cands:
            ent = self._capture(x, c)
            if len(cands) == 1:
                best = (c, ent)
                break
            ms = self._time_graph(ent[0])
            timings[c] = ms
            if best is None or ms < timings[best[0]] * 0.98:     # more chains must be clearly faster
                best = (c, ent)
        torch.cuda.synchronize()
        code = ops.last_status()
        if code:
            raise ops.FvmError(f"device status {code:#x} after capturing the forward (a bounded wait ran out)")
        self.last_capture_s = time.perf_counter() - t0
        c, (graph, static_in, static_out) = best
        return _Entry(graph, static_in, static_out, c, self.last_capture_s, timings)

    def _entry(self, x: torch.Tensor) -> _Entry:
        key = (tuple(x.shape), x.dtype, x.device.index, tuple(x.stride()))
        ent = self.cache.get(key)
        if ent is None:
            ent = self._build(x)
            self.cache[key] = ent
            while len(self.cache) > MAX_GRAPHS:
                self.cache.popitem(last=False)
        else:
            self.cache.move_to_end(key)
        return ent

    # ------------------------------------------------------------------------------------------------ calls
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if not self.enabled or not x.is_cuda:
            return self.fn(x)
        ent = self._entry(x)
        code = ops.poll_status()          # a fault reported by an earlier replay (no synchronisation here)
        if code:
            raise ops.FvmError(f"device status {code:#x}: a bounded wait inside a kernel ran out in an earlier launch")
        ent.static_in.copy_(x, non_blocking=True)
        ent.graph.replay()
        out = ent.static_out
        return out.clone() if isinstance(out, torch.Tensor) else out

    def static_buffers(self, x: torch.Tensor):
        """(graph, static_in, static_out) for x's shape, capturing first if needed: lets a caller copy inputs into the
        static buffer itself (e.g. straight from pinned host memory) and replay without the extra device copy."""
        ent = self._entry(x)
        return ent.graph, ent.static_in, ent.static_out

    def info(self, x: torch.Tensor) -> dict:
        """What was decided for x's shape: chains in use, the candidates' replay times (ms), seconds spent capturing."""
        ent = self._entry(x)
        return {"chains": ent.chains, "chain_ms": dict(ent.timings), "capture_s": round(ent.capture_s, 3)}

    def check(self) -> None:
        """Synchronises and raises if a kernel of this device reported a fault (a bounded device-side wait ran out);
        the outputs of the affected replay are then invalid."""
        code = ops.last_status()
        if code:
            raise ops.FvmError(f"device status {code:#x}: a bounded wait inside a kernel ran out")
