"""Feature-extractor registry of the B200 tier: build(name, tier, spec) -> Backbone(fn, mean, std, multiple, module,
info), the reference's contract (backbones/__init__.py:37-44, 112-124).

The reference delegates its CNN backbones to an external package that is not part of its tree; here the same
compilers as the classifiers are used and `fn(x)` returns the final feature map before pooling:
  resnet*      -> [B, C, H/32, W/32] fp32 (NCHW)
  convnext_*   -> [B, C, H/32, W/32] fp32 (NCHW), before the head LayerNorm
Names follow the reference's "tv-"/"timm-" style with torchvision builders: "tv-resnet50", "tv-convnext_tiny", ...
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..classification import zoo as _zoo

IMNET_MEAN, IMNET_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
TV = ["resnet18", "resnet50", "resnet101", "convnext_tiny", "convnext_small"]


@dataclass
class Backbone:
    fn: object
    mean: tuple
    std: tuple
    multiple: int
    module: object = None
    info: dict = None


def names():
    return [f"tv-{m}" for m in TV]


def build(name: str, tier: str = "cuda-kernels", spec=None, device: str = "cuda", seed: int = 1, graphs: bool = True
          ) -> Backbone:
    """name from names(); tier upstream | portable | cuda-kernels | b200 (max = old name of cuda-kernels)."""
    if tier not in ("upstream", "portable", "max", "cuda-kernels", "b200"):
        raise ValueError(tier)
    fam, _, model = name.partition("-")
    if fam != "tv" or model not in TV:
        raise KeyError(f"{name!r}: the b200 tier registers {names()}")
    up = _zoo.build_upstream(model, seed=seed)
    if tier == "upstream":
        up = up.to(device)
        if model.startswith("resnet"):
            body = torch.nn.Sequential(up.conv1, up.bn1, up.relu, up.maxpool, up.layer1, up.layer2, up.layer3, up.layer4)
        else:
            body = up.features

        def fn(x):
            with torch.inference_mode():
                return body(x)
        return Backbone(fn, IMNET_MEAN, IMNET_STD, 32, up, {"tier": tier})
    if tier == "portable":
        from ..classification.fast import fold_bn_inplace
        import copy
        h = fold_bn_inplace(copy.deepcopy(up)).half().to(device).to(memory_format=torch.channels_last)
        if model.startswith("resnet"):
            body = torch.nn.Sequential(h.conv1, h.bn1, h.relu, h.maxpool, h.layer1, h.layer2, h.layer3, h.layer4)
        else:
            body = h.features

        def fn(x):
            with torch.inference_mode():
                return body(x.to(torch.float16, memory_format=torch.channels_last)).float()
        return Backbone(fn, IMNET_MEAN, IMNET_STD, 32, up, {"tier": tier})
    from .. import ops
    from ..classification import fast as clf_fast
    from ..classification.fast import as_image
    from ..runtime import GraphRunner
    net = clf_fast.compile_model(up).to(device)
    if model.startswith("resnet"):
        def raw(x):
            return net.trunk(x).float().contiguous()
    else:
        def raw(x):
            return net.features(x).float().contiguous()
    runner = GraphRunner(raw, enabled=graphs)

    def fn(x):
        with torch.no_grad():
            return runner(as_image(x))
    return Backbone(fn, IMNET_MEAN, IMNET_STD, 32, up, {"tier": "b200", "compiled": type(net).__name__})
