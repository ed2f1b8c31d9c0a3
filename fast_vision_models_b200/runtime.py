"""Launch path: replays a whole forward as one CUDA graph per input shape.

The reference removes per-op CPU cost with a TorchScript trace of the rewritten graph (classification/fast/__init__.py:
58-79) and, for segmentation, an LRU of CUDA graphs (segmentation/fast/ops.py:107-160). Here every op is a plain kernel
launch on the current stream, so the forward is captured once per (shape, dtype, device) and replayed: the ~60-160
launches of a network cost one graph launch. Activation memory comes from the graph's private pool of torch's caching
allocator and is reused between layers.

Faults: a kernel whose bounded device-side wait ran out writes a code to the device's status word and returns; the
runner polls that word (no synchronisation) before every replay and raises, and `check()` synchronises and raises.
"""
from __future__ import annotations

import os
import time
from collections import OrderedDict
from typing import Callable

import torch

from . import ops

GRAPHS = os.environ.get("FVM_B200_GRAPHS", "1") != "0"   # kill switch in the style of the reference's CLF_* variables
MAX_GRAPHS = int(os.environ.get("FVM_B200_MAX_GRAPHS", "8"))


class _Entry:
    __slots__ = ("graph", "static_in", "static_out", "capture_s")

    def __init__(self, graph, static_in, static_out, capture_s):
        self.graph, self.static_in, self.static_out, self.capture_s = graph, static_in, static_out, capture_s


class GraphRunner:
    """Calls fn(x) through a per-shape CUDA graph. `fn` must be a pure function of x made of stream-ordered launches."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], enabled: bool = True):
        self.fn = fn
        self.enabled = enabled and GRAPHS
        self.cache: "OrderedDict[tuple, _Entry]" = OrderedDict()
        self.last_capture_s = 0.0      # seconds the most recent first call at a new shape spent on tuning + capture

    def _build(self, x: torch.Tensor) -> _Entry:
        ops.init(x.device)
        t0 = time.perf_counter()
        static_in = torch.empty_strided(tuple(x.shape), tuple(x.stride()), dtype=x.dtype, device=x.device)
        static_in.copy_(x)
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):
                self.fn(static_in)       # outside capture: first-call set-up and per-layer tile tuning of every op
        cur.wait_stream(side)
        torch.cuda.synchronize()
        from . import layers
        layers.release_tuning_buffers()      # the L2-flush buffer of the tile tuning is not needed once every layer is tuned
        layers.TileCache.flush()             # tile codes measured just now are kept for later processes
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static_out = self.fn(static_in)
        code = ops.last_status()
        if code:
            raise ops.FvmError(f"device status {code:#x} after capturing the forward (a bounded wait ran out)")
        self.last_capture_s = time.perf_counter() - t0
        return _Entry(graph, static_in, static_out, self.last_capture_s)

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

    def check(self) -> None:
        """Synchronises and raises if a kernel of this device reported a fault (a bounded device-side wait ran out);
        the outputs of the affected replay are then invalid."""
        code = ops.last_status()
        if code:
            raise ops.FvmError(f"device status {code:#x}: a bounded wait inside a kernel ran out")
