"""Helpers shared by segmentation callers (reference: segmentation/common.py:131-135)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def run_scores(model, x, out_size=None):
    """Full-resolution class scores by plain bilinear upsampling of the model's low-resolution logits."""
    s = model.logits(x)
    size = tuple(out_size) if out_size is not None else tuple(x.shape[2:])
    return F.interpolate(s.float(), size=size, mode="bilinear", align_corners=False)


def classmap(model, x, out_size=None):
    """Integer class map [N, H, W] at out_size (default: x's size): the model's fused path if it has one."""
    if getattr(model, "predict", None) is not None:
        return model.predict(x, out_size)
    return run_scores(model, x, out_size).argmax(1)
