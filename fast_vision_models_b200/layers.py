"""Building blocks of the compiled networks: each holds its prepared fp16 weights as buffers and runs one library op.

They stand where the reference's fx passes insert `torch.ops.clf.*` calls (classification/fast/fused.py:163-203 for
conv + add + activation chains, :206-236 for depthwise, r3.py:188-199 for squeeze-excite).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
from torch import nn

from . import fold, ops

AUTOTUNE = os.environ.get("FVM_B200_AUTOTUNE", "1") != "0"
PAIR_STEMS = os.environ.get("FVM_B200_PAIR_STEMS", "1") != "0"   # run RGB stems over column pairs (16-channel taps)   # kill switch, in the style of the reference's CLF_* variables
GATE_IN_WEIGHTS = os.environ.get("FVM_B200_GATE_IN_WEIGHTS", "1") != "0"   # squeeze-excite scale folded into the project conv's weights
FUSED_SQUEEZE = os.environ.get("FVM_B200_FUSED_SQUEEZE", "1") != "0"   # squeeze sums from the depthwise conv's epilogue
SPLIT_STEMS = os.environ.get("FVM_B200_SPLIT_STEMS", "1") != "0"   # stride-2 RGB stems on column-parity planes

_ACT_CODES = {
    nn.ReLU: ops.ACT_RELU, nn.ReLU6: ops.ACT_RELU6, nn.SiLU: ops.ACT_SILU, nn.Hardswish: ops.ACT_HARDSWISH,
}


def act_code(m: Optional[nn.Module]) -> int:
    """Activation module -> op code; same table as the reference's `_act_of` (fused.py:22-44)."""
    if m is None or isinstance(m, nn.Identity):
        return ops.ACT_NONE
    for cls, code in _ACT_CODES.items():
        if isinstance(m, cls):
            return code
    if isinstance(m, nn.GELU):
        return ops.ACT_GELU_TANH if getattr(m, "approximate", "none") == "tanh" else ops.ACT_GELU_ERF
    raise ValueError(f"activation {type(m).__name__} has no fused code")


_FLUSH = {}


def _l2_flush_buffer(device) -> torch.Tensor:
    """A scratch buffer larger than the 126 MB L2 (one per device, allocated at the first tuning, released by
    `release_tuning_buffers`, which the graph runner calls once a forward has been tuned and captured)."""
    key = torch.device(device).index
    if key not in _FLUSH:
        _FLUSH[key] = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    return _FLUSH[key]


def release_tuning_buffers() -> None:
    _FLUSH.clear()


class TileCache:
    """Tile codes chosen by timing, kept across processes: one JSON file per (library source hash, SM count) under
    $FVM_CACHE/fvm_b200 or ~/.cache/fvm_b200. A layer whose key is in the file skips its tuning launches, so the first
    call at a known shape costs the graph capture only. Written with an atomic replace; FVM_B200_TILE_CACHE=0 turns it
    off (every process then tunes for itself)."""

    enabled = os.environ.get("FVM_B200_TILE_CACHE", "1") != "0"
    _data = {}          # device index -> {key: code}
    _dirty = set()

    @staticmethod
    def _path(device_index: int) -> str:
        from . import _lib
        base = os.environ.get("FVM_CACHE") or os.path.join(os.path.expanduser("~"), ".cache")
        sms = torch.cuda.get_device_properties(device_index).multi_processor_count
        return os.path.join(base, "fvm_b200", f"tiles-{_lib.source_hash()[:16]}-sm{sms}.json")

    @classmethod
    def table(cls, device_index: int) -> dict:
        if device_index not in cls._data:
            data = {}
            if cls.enabled:
                try:
                    import json
                    with open(cls._path(device_index)) as f:
                        data = {str(k): int(v) for k, v in json.load(f).items()}
                except (OSError, ValueError):
                    data = {}
            cls._data[device_index] = data
        return cls._data[device_index]

    @classmethod
    def put(cls, device_index: int, key: str, code: int) -> None:
        cls.table(device_index)[key] = int(code)
        cls._dirty.add(device_index)

    @classmethod
    def flush(cls) -> None:
        """Writes what was tuned since the last flush (called by the graph runner after a capture)."""
        if not cls.enabled:
            cls._dirty.clear()
            return
        import json
        for idx in list(cls._dirty):
            path = cls._path(idx)
            try:
                os.makedirs(os.path.dirname(path), exist_ok=True)
                merged = {}
                try:
                    with open(path) as f:
                        merged = json.load(f)
                except (OSError, ValueError):
                    pass
                merged.update(cls._data[idx])
                tmp = f"{path}.tmp{os.getpid()}"
                with open(tmp, "w") as f:
                    json.dump(merged, f)
                os.replace(tmp, path)
            except OSError:
                pass                      # a read-only home: the choices live for this process only
        cls._dirty.clear()


class FusedConv(nn.Module):
    """y = act((conv(x, w) + b) * scale + res): one launch of the tcgen05 implicit-GEMM kernel."""

    def __init__(self, w: torch.Tensor, b: Optional[torch.Tensor], stride=(1, 1), padding=(0, 0), dilation=(1, 1),
                 act: int = 0, scale: Optional[torch.Tensor] = None, out_channels: Optional[int] = None):
        super().__init__()
        K = w.shape[0]
        self.out_channels = K if out_channels is None else out_channels   # channels that carry data (rest is padding)
        Kp = fold.round_up(K, 8)
        w, b = fold.pad_out_channels(w, b, Kp)
        w = fold.pad_in_channels(w, fold.round_up(w.shape[1], 8))
        self.register_buffer("w", fold.to_krsc_half(w))
        self.register_buffer("b", None if b is None else b.half().contiguous())
        self.register_buffer("scale", None if scale is None else scale.float().contiguous())
        self.stride, self.padding, self.dilation, self.act = tuple(stride), tuple(padding), tuple(dilation), int(act)
        self._tiles = {}      # (input shape, has residual) -> output-channel tile chosen by timing
        self.register_buffer("w_pair", None)
        self._pair = None
        if PAIR_STEMS and self.w.shape[1] == 8 and self.stride[1] % 2 == 0 and self.dilation == (1, 1) \
                and self.w.shape[2] * self.w.shape[3] > 1:
            self._make_column_pairs(w)

    def _make_column_pairs(self, w: torch.Tensor) -> None:
        """An 8-channel (zero-padded RGB) stem with an even horizontal stride, re-expressed over pairs of input columns:
        the NHWC8 input [N,H,W,8] is the same memory as [N,H,W/2,16], a tap then covers two columns x 8 channels, the
        stride halves and the kernel has about half as many (twice as wide) taps. Same products, same sums (the added
        weights are zero); the TMA unit gathers half as many rows."""
        K, C, R, S = w.shape              # C == 8 after padding
        pw, sw = self.padding[1], self.stride[1]
        odd = pw % 2
        lo2 = (pw + 1) // 2
        S2 = (S - 1 - pw) // 2 + lo2 + 1
        w2 = torch.zeros((K, 16, R, S2), dtype=w.dtype)
        for p2 in range(S2):
            for dx in range(2):
                s = 2 * p2 + dx - odd
                if 0 <= s < S:
                    w2[:, dx * 8:(dx + 1) * 8, :, p2] = w[:, :, :, s]
        self.w_pair = fold.to_krsc_half(w2)
        self._pair = (S2, lo2, sw // 2)

    def _tile_for(self, x: torch.Tensor, res, out: torch.Tensor, act: int) -> int:
        """Output-channel tile for this layer at this input shape. The library's own rule picks from wave efficiency
        and shared-memory fit; where several tile widths are possible they are timed once (first call at a new shape,
        outside stream capture) and the fastest is kept -- the reference's `pick()` (fused_conv.cu:216-227) is a fixed
        rule tuned for another GPU, here the choice is measured on the device that runs it."""
        key = (tuple(x.shape), res is not None)
        t = self._tiles.get(key)
        if t is not None:
            return t
        if not AUTOTUNE:
            return 0
        K_, C_, R_k, S_k = self.w.shape
        ckey = (f"{tuple(x.shape)}|ld{x.stride(3) if x.shape[3] > 1 else 0}|K{K_}R{R_k}S{S_k}|s{self.stride}p{self.padding}"
                f"d{self.dilation}|act{act}|res{int(res is not None)}|scale{int(self.scale is not None)}")
        dev_idx = x.device.index if x.device.index is not None else torch.cuda.current_device()
        cached = TileCache.table(dev_idx).get(ckey)
        if cached is not None:
            self._tiles[key] = cached
            return cached
        if torch.cuda.is_current_stream_capturing() or ops.chain_active():
            return 0          # no timing while a graph is captured or while layers are recorded for a chain launch
        K = self.w.shape[0]
        # tile code: low 16 bits = output-channel tile (0 = library's choice), bits 16.. = 128-pixel sub-tiles per tile
        widths = [0] + [c for c in (64, 128, 256) if c < K or (c == 256 and K > 256)]
        if K <= 64 or self.w.shape[1] == 8:
            widths = [0]   # one tile anyway / 8-channel stems keep the library's tap-packed path (all of K in one tile)
        cands = list(widths)
        rows = x.shape[0] * out.shape[2] * out.shape[3]
        if rows >= 148 * 8 * 128 and self.w.shape[2] * self.w.shape[3] * ((self.w.shape[1] + 63) // 64) <= 9:
            cands += [c | (2 << 16) for c in widths if (c or K) <= 128]   # short reductions on large maps: 256-pixel tiles
        R_, S_ = self.w.shape[2], self.w.shape[3]
        if (R_ == 3 and S_ == 3 and tuple(self.stride) == (1, 1) and self.dilation[0] == self.dilation[1] <= 4
                and 8 < self.w.shape[1] <= 64):
            # 3x3 stride-1 over at most 64 channels: staged input patches (bits 26..27 = 1) against im2col loads (= 2),
            # per tile width. With one 64-channel chunk both modes add the taps in the same order: same bits.
            cands += [c | (1 << 26) for c in widths] + [c | (2 << 26) for c in widths]
        if self.w.shape[1] != 8:
            # weight tile resident in shared memory (bits 24..25 = 1) or streamed per k-block (= 2), per tile width
            base = list(widths)
            cands += [c | (1 << 24) for c in base] + [c | (2 << 24) for c in base]
        if rows <= 148 * 128 * 3 and self.w.shape[1] > 16:
            # few tiles per SM: stream-K (bits 28..29 = 1) spreads the k-blocks of all tiles evenly over the SMs; offered
            # per tile width against the plain schedule (= 2)
            cands += [c | (1 << 28) for c in widths] + [c | (2 << 28) for c in widths]
        if self.w.shape[1] > 16 and ops.query(4) > 0:
            # CTA pairs (bit 30): two SMs share each tile of 256 pixels and each fetches half of the weight tile; same bits
            cands += [c | (1 << 30) for c in widths]
        best = 0
        if len(cands) > 1:
            # Candidates are timed in rounds (every candidate once per round, best burst kept), so that a drift of the
            # clocks during tuning hits all of them alike; a candidate the library refuses is dropped.
            cands = list(dict.fromkeys(cands))
            times = {}
            for c in cands:
                try:
                    for _ in range(2):
                        ops.conv_fused_into(x, self.w, self.b, res, self.padding, self.stride, act, out,
                                            dilation=self.dilation, scale=self.scale, tile_n=c)
                    times[c] = float("inf")
                except ops.FvmError:
                    continue
            # Each timed launch sees the cache state it has inside a forward pass: weights, residual and output cold
            # (a buffer larger than L2 is overwritten first), the input freshly written (as by the previous layer).
            flush = _l2_flush_buffer(x.device)
            for _round in range(4):
                for c in times:
                    for _ in range(2):
                        flush.zero_()
                        x.mul_(1)           # exact identity: rewrites the input, which puts it back into L2
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record()
                        ops.conv_fused_into(x, self.w, self.b, res, self.padding, self.stride, act, out,
                                            dilation=self.dilation, scale=self.scale, tile_n=c)
                        e1.record()
                        e1.synchronize()
                        times[c] = min(times[c], e0.elapsed_time(e1))
            best_ms = times.get(0, float("inf"))
            for c, ms in times.items():
                if ms < best_ms * 0.97:      # a different tile must be clearly faster than the incumbent
                    best, best_ms = c, ms
        self._tiles[key] = best
        TileCache.put(dev_idx, ckey, best)
        return best

    def forward_image(self, x: torch.Tensor) -> torch.Tensor:
        """The stem applied to an fp32 NCHW image batch (at most 8 channels). A stride-2 stem with an even image width
        runs on the column-parity-split input (`ops.input_nhwc8_split` + `ops.stem_conv_s2`), where the input patch of
        each output tile is staged once; anything else converts to NHWC8 (`ops.input_nhwc8`, the reference's
        clf::input_nhwc8) and takes the general convolution."""
        K, C, R, S = self.w.shape
        if (SPLIT_STEMS and C == 8 and self.stride == (2, 2) and self.dilation == (1, 1) and self.scale is None
                and R <= 8 and S <= 8 and K <= 256 and self.padding[0] < R and self.padding[1] < S
                and x.shape[3] % 2 == 0 and (R + R % 2) * S * ((K + 31) // 32 * 32) * 16 <= 96 * 1024):
            return ops.stem_conv_s2(ops.input_nhwc8_split(x), self.w, self.b, self.padding, self.act)
        return self.forward(ops.input_nhwc8(x))

    @classmethod
    def from_conv_bn(cls, conv: nn.Conv2d, bn: Optional[nn.Module] = None, act: int = 0, **kw) -> "FusedConv":
        if conv.groups != 1:
            raise ValueError("FusedConv: dense convolutions only")
        if conv.padding_mode != "zeros":
            raise ValueError("FusedConv: zero padding only")
        w, b = fold.fold_conv_bn(conv, bn if isinstance(bn, nn.BatchNorm2d) else None)
        return cls(w, b, conv.stride, conv.padding, conv.dilation, act, **kw)

    @classmethod
    def from_linear(cls, lin: nn.Linear, act: int = 0, gamma: Optional[torch.Tensor] = None) -> "FusedConv":
        w = lin.weight.detach().float()
        b = lin.bias.detach().float() if lin.bias is not None else None
        if gamma is not None:
            w, b = fold.fold_layer_scale(w, b, gamma)
        return cls(w.view(w.shape[0], w.shape[1], 1, 1), b, act=act)

    def forward(self, x: torch.Tensor, res: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                act: Optional[int] = None) -> torch.Tensor:
        a = self.act if act is None else act
        if out is None:
            N, _, H, W = x.shape
            K, _, R, S = self.w.shape
            P = (H + 2 * self.padding[0] - self.dilation[0] * (R - 1) - 1) // self.stride[0] + 1
            Q = (W + 2 * self.padding[1] - self.dilation[1] * (S - 1) - 1) // self.stride[1] + 1
            out = ops.empty_nhwc(N, K, P, Q, x.device)
        if self._pair is not None and x.shape[3] % 2 == 0 and x.is_contiguous(memory_format=torch.channels_last):
            S2, lo2, sw2 = self._pair
            N, _, H, W = x.shape
            Q = out.shape[3]
            hi2 = (Q - 1) * sw2 + S2 - W // 2 - lo2
            if hi2 >= 0:
                x2 = x.permute(0, 2, 3, 1).reshape(N, H, W // 2, 16).permute(0, 3, 1, 2)    # a view: no copy
                ops.conv_fused_into(x2, self.w_pair, self.b, res, (self.padding[0], lo2), (self.stride[0], sw2), a, out,
                                    scale=self.scale, pad_hi=(self.padding[0], hi2))
                return out
        tile = self._tile_for(x, res, out, a)
        ops.conv_fused_into(x, self.w, self.b, res, self.padding, self.stride, a, out, dilation=self.dilation,
                            scale=self.scale, tile_n=tile)
        return out


class DepthwiseConv(nn.Module):
    """Depthwise conv + folded BatchNorm bias + activation (reference: clf.dwconv / clfr3.dwconv2)."""

    def __init__(self, conv: nn.Conv2d, bn: Optional[nn.Module], act: int):
        super().__init__()
        if conv.groups != conv.in_channels or conv.out_channels != conv.in_channels:
            raise ValueError("DepthwiseConv: groups == in_channels == out_channels only")
        w, b = fold.fold_conv_bn(conv, bn if isinstance(bn, nn.BatchNorm2d) else None)
        self.register_buffer("w", fold.dw_to_rsc_half(w))
        self.register_buffer("b", b.half().contiguous())
        self.stride, self.padding, self.dilation, self.act = conv.stride, conv.padding, conv.dilation, int(act)

    def forward(self, x: torch.Tensor, pool: bool = False):
        """pool=True: returns (y, partial sums per tile) for a squeeze-excite block that follows (fused squeeze)."""
        return ops.dwconv(x, self.w, self.b, self.stride, self.padding, self.act, dilation=self.dilation, pool=pool)


class SqueezeExcite(nn.Module):
    """x * sigmoid(W2 act(W1 mean(x) + b1) + b2). Squeeze channels are zero-padded to a multiple of 8, which is exact
    because act(0) = 0 for the supported activations (reference: pad_conv_pairs, fused.py:400-434)."""

    def __init__(self, fc1: nn.Conv2d, fc2: nn.Conv2d, act: int):
        super().__init__()
        if act not in (ops.ACT_NONE, ops.ACT_RELU, ops.ACT_RELU6, ops.ACT_SILU, ops.ACT_HARDSWISH, ops.ACT_GELU_ERF,
                       ops.ACT_GELU_TANH):
            raise ValueError("SqueezeExcite: unsupported activation")
        w1 = fc1.weight.detach().float().flatten(1)     # [Cs, C]
        b1 = fc1.bias.detach().float() if fc1.bias is not None else torch.zeros(w1.shape[0])
        w2 = fc2.weight.detach().float().flatten(1)     # [C, Cs]
        b2 = fc2.bias.detach().float() if fc2.bias is not None else torch.zeros(w2.shape[0])
        Cs, C = w1.shape
        Csp = fold.round_up(Cs, 8)
        w1p = torch.zeros(Csp, C)
        w1p[:Cs] = w1
        b1p = torch.zeros(Csp)
        b1p[:Cs] = b1
        w2p = torch.zeros(C, Csp)
        w2p[:, :Cs] = w2
        self.register_buffer("w1", w1p.half().contiguous())
        self.register_buffer("b1", b1p.half().contiguous())
        self.register_buffer("w2", w2p.half().contiguous())
        self.register_buffer("b2", b2.half().contiguous())
        self.act = int(act)

    def forward(self, x: torch.Tensor, partial: Optional[torch.Tensor] = None) -> torch.Tensor:
        """`partial`: the per-tile sums the producing depthwise conv emitted (`DepthwiseConv.forward(pool=True)`); the
        squeeze then costs no pass over x (the reference's fused form: gconv2_pool + sums_to_mean_k, r3.cu:181-203,
        283-299). Without it the squeeze is a global average pool of x."""
        return ops.se_scale(x, self.gate(x, partial))

    def gate(self, x: torch.Tensor, partial: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The pre-sigmoid gate s [N, C, 1, 1] of x."""
        if partial is not None and FUSED_SQUEEZE:
            return ops.se_gate_pooled(partial, x.shape[2] * x.shape[3], self.w1, self.b1, self.w2, self.b2, self.act)
        return ops.se_gate(ops.global_avgpool(x), self.w1, self.b1, self.w2, self.b2, self.act)


class LayerNormCL(nn.Module):
    """LayerNorm over the channels of a channels-last tensor (torchvision LayerNorm2d / nn.LayerNorm on NHWC)."""

    def __init__(self, ln: nn.LayerNorm):
        super().__init__()
        self.register_buffer("w", ln.weight.detach().half().contiguous())
        self.register_buffer("b", ln.bias.detach().half().contiguous())
        self.eps = float(ln.eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.layernorm_cl(x, self.w, self.b, self.eps)
