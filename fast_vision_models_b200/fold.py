"""Host-side weight preparation, all in fp32 with one final rounding to fp16.

Arithmetic follows the reference:
  * BatchNorm fold (classification/fast/__init__.py:201-208; segmentation/fast/cnn.py:54-61):
      sc = gamma / sqrt(running_var + eps);  w' = w * sc[k];  b' = b_conv * sc + (beta - running_mean * sc)
  * LayerScale fold (classification/fast/fused.py:151-155; convnext.py:17-23):  w' = w * gamma[k];  b' = b * gamma
  * stem / head channel padding (fused.py:90-105; segmentation/fast/cnn_fuse.py:30-40): zero weights, exact.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn


def fold_conv_bn(conv: nn.Conv2d, bn: Optional[nn.BatchNorm2d]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (weight [K,C/groups,R,S] fp32, bias [K] fp32) of conv followed by eval-mode BatchNorm."""
    w = conv.weight.detach().float()
    b = conv.bias.detach().float() if conv.bias is not None else None
    if bn is None:
        return w, (b if b is not None else torch.zeros(w.shape[0]))
    sc = (bn.weight.detach().float() if bn.affine else 1.0) / torch.sqrt(bn.running_var.detach().float() + bn.eps)
    shift = (bn.bias.detach().float() if bn.affine else 0.0) - bn.running_mean.detach().float() * sc
    w = w * sc.view(-1, 1, 1, 1)
    b = b * sc + shift if b is not None else shift
    return w, b


def fold_layer_scale(w: torch.Tensor, b: Optional[torch.Tensor], gamma: torch.Tensor):
    """Folds a per-output-channel scale into a linear / 1x1 weight [K, ...] and its bias."""
    g = gamma.detach().float().reshape(-1)
    w = w.float() * g.view(-1, *([1] * (w.dim() - 1)))
    b = b.float() * g if b is not None else None
    return w, b


def pad_in_channels(w: torch.Tensor, to: int) -> torch.Tensor:
    """[K,C,R,S] -> [K,to,R,S] with zero weights for the added input channels."""
    K, C, R, S = w.shape
    if C >= to:
        return w
    out = torch.zeros((K, to, R, S), dtype=w.dtype)
    out[:, :C] = w
    return out


def pad_out_channels(w: torch.Tensor, b: Optional[torch.Tensor], to: int):
    """Zero-pads the output channels of a weight [K,...] (and bias) to `to`."""
    K = w.shape[0]
    if K >= to:
        return w, b
    wo = torch.zeros((to,) + tuple(w.shape[1:]), dtype=w.dtype)
    wo[:K] = w
    bo = None
    if b is not None:
        bo = torch.zeros(to, dtype=b.dtype)
        bo[:K] = b
    return wo, bo


def round_up(v: int, m: int) -> int:
    return (v + m - 1) // m * m


def to_krsc_half(w: torch.Tensor) -> torch.Tensor:
    """[K,C,R,S] fp32 -> fp16 tensor of the same shape stored KRSC (channels-last)."""
    return w.half().contiguous(memory_format=torch.channels_last)


def grouped_runs(C: int, K: int, groups: int):
    """Super-group shape for fvm_gconv2d_f16: the fewest whole groups per run such that a run's input channels are a
    multiple of 8 and its output channels a multiple of 64 (or one run covers everything). Returns (gsg, gsk)."""
    if groups <= 0 or C % groups or K % groups:
        raise ValueError(f"grouped conv: {C} -> {K} channels do not divide into {groups} groups")
    gw, kg = C // groups, K // groups
    for r in range(1, groups + 1):
        if r == groups or ((r * gw) % 8 == 0 and (r * kg) % 64 == 0):
            return r * gw, r * kg
    return C, K


def pack_grouped(w: torch.Tensor, groups: int):
    """Grouped-conv weight [K, GW, R, S] (the reference's clfr3.gconv2 layout, r3.cu:230-232) -> ([K, gsg, R, S] fp16
    stored KRSC, gsg, gsk): every output channel's GW weights sit at its group's place inside its run of gsg input
    channels, zeros elsewhere, so that a run is a dense gsg -> gsk convolution."""
    K, GW, R, S = w.shape
    C = GW * groups
    gsg, gsk = grouped_runs(C, K, groups)
    kg = K // groups
    per_run = gsg // GW
    out = torch.zeros((K, gsg, R, S), dtype=torch.float16, device=w.device)
    wh = w.to(torch.float16)
    for j in range(per_run):                       # position of the group inside its run
        ks = torch.arange(K, device=w.device)
        sel = ((ks // kg) % per_run) == j
        out[sel, j * GW:(j + 1) * GW] = wh[sel]
    return out.contiguous(memory_format=torch.channels_last), gsg, gsk


def dw_to_rsc_half(w: torch.Tensor) -> torch.Tensor:
    """Depthwise weight [C,1,R,S] fp32 -> [R,S,C] fp16 contiguous (reference: fused.py:221)."""
    return w[:, 0].permute(1, 2, 0).contiguous().half()
