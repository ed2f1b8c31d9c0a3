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
from typing import Callable, Sequence

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
        if x.data_ptr() != ent.static_in.data_ptr():     # a caller may fill the static input itself (static_buffers)
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


class HostPipeline:
    """Batches from pinned host memory in, results in pinned host memory out, with both copies under the forwards.

    `runners` are graph runners over the same network (two or more: while one replica's graph computes batch i, the copy
    stream writes batch i+1 straight into another replica's static input, and the results of batch i-1 leave on a third
    stream). `submit(x_host)` enqueues one batch and returns its slot; `result(slot)` waits for that batch's results
    only. A slot's host buffer is rewritten when the slot comes round again, len(runners) submissions later.
    The reference serves through `Fast.__call__` on device tensors (classification/fast/__init__.py:81-95); this is the
    same call with the host <-> device copies taken off the compute stream."""

    def __init__(self, runners: Sequence[GraphRunner], example: torch.Tensor, device=None):
        if len(runners) < 2:
            raise ValueError("HostPipeline needs at least two runners (replicas of one network)")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        x0 = example.to(dev)
        self._bufs = [r.static_buffers(x0) for r in runners]          # (graph, static_in, static_out) per replica
        self._main = torch.cuda.current_stream(dev)
        self._in_stream = torch.cuda.Stream(device=dev)
        self._out_stream = torch.cuda.Stream(device=dev)
        n = len(runners)
        self._ready = [torch.cuda.Event() for _ in range(n)]
        self._consumed = [torch.cuda.Event() for _ in range(n)]
        self._drained = [torch.cuda.Event() for _ in range(n)]
        self._host_out = [torch.empty(tuple(b[2].shape), dtype=b[2].dtype).pin_memory() for b in self._bufs]
        for b in range(n):
            self._consumed[b].record(self._main)
            self._drained[b].record(self._main)
        self._next = 0
        self.in_bytes = x0.numel() * x0.element_size()
        self.out_bytes = self._host_out[0].numel() * self._host_out[0].element_size()

    def submit(self, x_host: torch.Tensor) -> int:
        b = self._next
        self._next = (b + 1) % len(self._bufs)
        graph, static_in, static_out = self._bufs[b]
        if tuple(x_host.shape) != tuple(static_in.shape) or x_host.dtype != static_in.dtype:
            raise ops.FvmError("HostPipeline.submit: batch shape / dtype differs from the example the pipeline was built for")
        with torch.cuda.stream(self._in_stream):
            self._in_stream.wait_event(self._consumed[b])      # the replay that last read this static input is done
            static_in.copy_(x_host, non_blocking=True)         # host -> device, straight into the graph's input
            self._ready[b].record(self._in_stream)
        self._main.wait_event(self._ready[b])
        self._main.wait_event(self._drained[b])                # the results this replica wrote last time have left
        with torch.cuda.stream(self._main):
            graph.replay()
        self._consumed[b].record(self._main)
        with torch.cuda.stream(self._out_stream):              # device -> host under the next forward
            self._out_stream.wait_event(self._consumed[b])
            self._host_out[b].copy_(static_out, non_blocking=True)
            self._drained[b].record(self._out_stream)
        return b

    def result(self, slot: int) -> torch.Tensor:
        self._drained[slot].synchronize()
        return self._host_out[slot]
