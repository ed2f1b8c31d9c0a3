"""Launch path: replays a whole forward as one CUDA graph per input shape.

The reference removes per-op CPU cost with a TorchScript trace of the rewritten graph (classification/fast/__init__.py:
58-79) and, for segmentation, an LRU of CUDA graphs (segmentation/fast/ops.py:107-160). Here every op is a plain kernel
launch on the current stream, so the forward is captured once per (shape, dtype, device) and replayed: the ~60-160
launches of a network cost one graph launch. Activation memory comes from the graph's private pool of torch's caching
allocator and is reused between layers.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from typing import Callable

import torch

from . import ops

GRAPHS = os.environ.get("FVM_B200_GRAPHS", "1") != "0"   # kill switch in the style of the reference's CLF_* variables
MAX_GRAPHS = int(os.environ.get("FVM_B200_MAX_GRAPHS", "8"))


class GraphRunner:
    """Calls fn(x) through a per-shape CUDA graph. `fn` must be a pure function of x made of stream-ordered launches."""

    def __init__(self, fn: Callable[[torch.Tensor], torch.Tensor], enabled: bool = True):
        self.fn = fn
        self.enabled = enabled and GRAPHS
        self.cache: "OrderedDict[tuple, tuple]" = OrderedDict()

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if not self.enabled or not x.is_cuda:
            return self.fn(x)
        key = (tuple(x.shape), x.dtype, x.device.index, tuple(x.stride()))
        ent = self.cache.get(key)
        if ent is None:
            ops.init(x.device)
            static_in = torch.empty_strided(tuple(x.shape), tuple(x.stride()), dtype=x.dtype, device=x.device)
            static_in.copy_(x)
            cur = torch.cuda.current_stream()
            side = torch.cuda.Stream()
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                for _ in range(2):
                    self.fn(static_in)       # warm-up outside capture (first-call set-up of every op)
            cur.wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = self.fn(static_in)
            ent = (graph, static_in, static_out)
            self.cache[key] = ent
            while len(self.cache) > MAX_GRAPHS:
                self.cache.popitem(last=False)
        else:
            self.cache.move_to_end(key)
        graph, static_in, static_out = ent
        static_in.copy_(x, non_blocking=True)
        graph.replay()
        return static_out.clone() if isinstance(static_out, torch.Tensor) else static_out

    def static_buffers(self, x: torch.Tensor):
        """(graph, static_in, static_out) for x's shape, capturing first if needed: lets a caller copy inputs into the
        static buffer itself (e.g. straight from pinned host memory) and replay without the extra device copy."""
        self(x)
        key = (tuple(x.shape), x.dtype, x.device.index, tuple(x.stride()))
        return self.cache[key]
