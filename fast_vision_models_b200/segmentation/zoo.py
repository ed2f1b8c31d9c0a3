"""Segmentation registry of the B200 tier: build(name, impl) -> Wrap with .logits(x), .predict(x, out_size), .norm,
.protocol, .info, .module -- the reference's contract (segmentation/zoo.py:38-42, 67-75).

The reference builds DeepLabV3 through mmseg, which is not available here; the registered model is torchvision's
`deeplabv3_resnet50` (dilated ResNet-50, output stride 8, ASPP rates 12/24/36) with a configurable class count
(19 = Cityscapes-style head of the benchmark configuration) and seeded random weights.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import weights as W

ALIASES = {"upstream": "base", "portable": "uf", "cuda-kernels": "opt", "max": "opt", "b200": "opt"}
IMNET = ((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))
REG = {}


def register(name):
    def deco(f):
        REG[name] = f
        return f
    return deco


class Wrap:
    def __init__(self, fn, norm, protocol, info, module=None, predict=None):
        self.logits, self.norm, self.protocol, self.info, self.module = fn, norm, protocol, info, module
        self.predict = predict  # fused path: predict(x, out_size) -> int class map [N, H, W]


def build_upstream(name: str, num_classes: int = 19, seed: int = 1, state_dict: Optional[dict] = None):
    import torchvision
    fn = {"deeplabv3-r50": torchvision.models.segmentation.deeplabv3_resnet50,
          "deeplabv3-r101": torchvision.models.segmentation.deeplabv3_resnet101}[name]
    m = fn(weights=None, weights_backbone=None, num_classes=num_classes, aux_loss=False)
    if state_dict is not None:
        m.load_state_dict(state_dict)
        return m.eval()
    return W.seeded_init(m, style="bn", seed=seed)


def _deeplab(name, impl, device, num_classes, seed, state_dict, graphs):
    m = build_upstream(name, num_classes, seed, state_dict)
    proto = {"resize": ("keep", None), "infer": "whole", "pad": 8}
    info = {"weights": "seeded-random" if state_dict is None else "state_dict", "classes": num_classes}
    if impl == "base":
        m = m.to(device)

        def logits(x):
            with torch.inference_mode():
                feat = m.backbone(x)["out"]
                return m.classifier(feat)
        return Wrap(logits, IMNET, proto, info, m)
    if impl == "uf":
        from ..classification.fast import fold_bn_inplace
        import copy
        h = fold_bn_inplace(copy.deepcopy(m)).half().to(device).to(memory_format=torch.channels_last)

        def logits(x):
            with torch.inference_mode():
                x = x.to(device, torch.float16, memory_format=torch.channels_last)
                return h.classifier(h.backbone(x)["out"]).float()
        return Wrap(logits, IMNET, proto, info, m)
    from .fast import B200DeepLabV3, FastSeg
    f = FastSeg(B200DeepLabV3(m), graphs=graphs).to(device)
    return Wrap(f.logits, IMNET, proto, dict(info, **f.info), m, f.predict)


@register("deeplabv3-r50")
def deeplabv3_r50(impl, **kw):
    return _deeplab("deeplabv3-r50", impl, **kw)


@register("deeplabv3-r101")
def deeplabv3_r101(impl, **kw):
    return _deeplab("deeplabv3-r101", impl, **kw)


def names():
    return sorted(REG)


def build(name: str, impl: str = "b200", device: str = "cuda", num_classes: int = 19, seed: int = 1,
          state_dict: Optional[dict] = None, graphs: bool = True) -> Wrap:
    impl = ALIASES.get(impl, impl)
    if name not in REG:
        raise KeyError(f"{name!r} is not registered in the b200 tier (conv hot path only): {names()}")
    if impl not in ("base", "uf", "opt"):
        raise ValueError(impl)
    return REG[name](impl, device=device, num_classes=num_classes, seed=seed, state_dict=state_dict, graphs=graphs)
