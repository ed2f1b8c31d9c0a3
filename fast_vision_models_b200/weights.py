"""Where weights come from.

The reference fetches pretrained checkpoints (fast_vision_models/weights.py:15-26: local `FVM_WEIGHTS` directories, else
a download). This build runs without a network, so the registries build every model with `weights=None` and give it a
seeded random initialisation; a user who has a checkpoint passes `state_dict=` to the registry call instead.

`seeded_init` is the recipe the parity tests and the benchmark use on both sides of every comparison:
  * conv / linear weights: Kaiming-normal (fan_out, ReLU) for BatchNorm networks, truncated normal (std 0.02) for
    LayerNorm networks (ConvNeXt), biases 0 (conv) / small uniform (linear heads);
  * every BatchNorm: gamma ~ U(0.5, 1.5), beta ~ N(0, 0.1), running_mean ~ N(0, 0.1), running_var ~ U(0.5, 1.5), so
    that folding the statistics into the convolution is really exercised;
  * ConvNeXt layer_scale = `layer_scale` (1e-6 is the published initial value; the tests also run U(0.1, 1)).
All draws come from CPU generators, so the values do not depend on the device.
"""
from __future__ import annotations

import math
from typing import Optional, Union

import torch
from torch import nn


def seeded_init(model: nn.Module, style: str = "bn", seed: int = 1, layer_scale: Union[float, str, None] = None
                ) -> nn.Module:
    g_w = torch.Generator().manual_seed(seed)
    g_bn = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, (nn.Conv2d, nn.Linear)):
                w = m.weight
                if style == "ln":
                    t = torch.empty(w.shape)
                    nn.init.trunc_normal_(t, std=0.02, generator=g_w)
                    w.copy_(t)
                    if m.bias is not None:
                        m.bias.zero_()
                else:
                    if isinstance(m, nn.Conv2d):
                        fan_out = w.shape[0] * w.shape[2] * w.shape[3] // m.groups
                    else:
                        fan_out = w.shape[0]
                    std = math.sqrt(2.0 / fan_out)
                    w.copy_(torch.randn(w.shape, generator=g_w) * std)
                    if m.bias is not None:
                        if isinstance(m, nn.Linear):
                            bound = 1.0 / math.sqrt(w.shape[0])
                            m.bias.copy_((torch.rand(m.bias.shape, generator=g_w) * 2 - 1) * bound)
                        else:
                            m.bias.zero_()
            elif isinstance(m, (nn.BatchNorm2d,)):
                c = m.num_features
                m.weight.copy_(torch.rand(c, generator=g_bn) + 0.5)
                m.bias.copy_(torch.randn(c, generator=g_bn) * 0.1)
                m.running_mean.copy_(torch.randn(c, generator=g_bn) * 0.1)
                m.running_var.copy_(torch.rand(c, generator=g_bn) + 0.5)
            elif isinstance(m, (nn.LayerNorm,)):
                # includes torchvision's LayerNorm2d subclass
                m.weight.fill_(1.0)
                m.bias.zero_()
        if layer_scale is not None:
            for name, prm in model.named_parameters():
                if name.endswith("layer_scale"):
                    if layer_scale == "uniform":
                        prm.copy_((torch.rand(prm.shape, generator=g_w) * 0.9 + 0.1))
                    else:
                        prm.fill_(float(layer_scale))
    return model.eval()


def seeded_input(shape, seed: int = 0) -> torch.Tensor:
    """fp32 N(0,1) input drawn on the CPU."""
    return torch.randn(tuple(shape), generator=torch.Generator().manual_seed(seed))
