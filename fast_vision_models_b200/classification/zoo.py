"""ImageNet-1k classifier registry of the B200 tier.

    from fast_vision_models_b200.classification import zoo
    m = zoo.load("resnet50", impl="b200")        # -> Loaded(model, transform, input_size, spec, info)
    logits = m.model(x)                           # x: [B,3,H,W] fp32 normalised, on the GPU

Same call and return type as the reference registry (classification/zoo.py:68-74, 160-186). Tiers: "upstream"/"base"
= the unmodified torchvision model in fp32; "portable"/"friendly" = folded fp16 channels-last on plain PyTorch;
"b200" (and the reference's names for its kernel tier, "cuda-kernels"/"opt"/"max") = this library's kernels.
Only the convolutional families of the hot path are registered. Weights: there is no network here, so models are built
with weights=None and `weights.seeded_init`; pass `state_dict=` to load a checkpoint instead.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import weights as W

ALIASES = {"upstream": "base", "portable": "friendly", "cuda-kernels": "opt", "max": "opt", "b200": "opt"}


@dataclass
class Spec:
    name: str
    year: int
    src: str            # tv
    ident: str          # torchvision builder name
    family: str         # cnn | dwcnn
    init: str = "bn"    # seeded-init style: "bn" (Kaiming + randomised BN statistics) or "ln" (trunc-normal 0.02)
    size: int = 224
    extra: dict = field(default_factory=dict)


SPECS = [
    Spec("resnet18", 2015, "tv", "resnet18", "cnn"),
    Spec("resnet50", 2015, "tv", "resnet50", "cnn"),
    Spec("resnet101", 2015, "tv", "resnet101", "cnn"),
    Spec("resnet152", 2015, "tv", "resnet152", "cnn"),
    Spec("efficientnet_b0", 2019, "tv", "efficientnet_b0", "dwcnn", size=224),
    Spec("efficientnet_b4", 2019, "tv", "efficientnet_b4", "dwcnn", size=380),
    Spec("convnext_tiny", 2022, "tv", "convnext_tiny", "dwcnn", init="ln", extra={"layer_scale": 1e-6}),
    Spec("convnext_small", 2022, "tv", "convnext_small", "dwcnn", init="ln", extra={"layer_scale": 1e-6}),
]
BY_NAME = {s.name: s for s in SPECS}


@dataclass
class Loaded:
    model: torch.nn.Module
    transform: object
    input_size: tuple
    spec: Spec
    info: dict


def names():
    return [s.name for s in SPECS]


def build_upstream(name: str, seed: int = 1, layer_scale=None, state_dict: Optional[dict] = None) -> torch.nn.Module:
    """The upstream fp32 torchvision model with seeded random weights (or `state_dict`)."""
    import torchvision
    spec = BY_NAME[name]
    model = torchvision.models.get_model(spec.ident, weights=None)
    if state_dict is not None:
        model.load_state_dict(state_dict)
        return model.eval()
    ls = spec.extra.get("layer_scale") if layer_scale is None else layer_scale
    return W.seeded_init(model, style=spec.init, seed=seed, layer_scale=ls)


def _transform(size: int):
    """Normalisation of a [0,1] image batch (ImageNet mean / std), the tensor part of torchvision's eval preset."""
    mean = torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1)
    std = torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1)

    def tf(x: torch.Tensor) -> torch.Tensor:
        return (x - mean.to(x.device)) / std.to(x.device)
    return tf


def load(name: str, impl: str = "base", device: str = "cuda", seed: int = 1, layer_scale=None,
         state_dict: Optional[dict] = None, graphs: bool = True, **kw) -> Loaded:
    impl = ALIASES.get(impl, impl)
    if name not in BY_NAME:
        raise KeyError(f"{name!r} is not registered in the b200 tier (hot-path families only): {names()}")
    spec = BY_NAME[name]
    model = build_upstream(name, seed=seed, layer_scale=layer_scale, state_dict=state_dict)
    info = {"weights": "seeded-random" if state_dict is None else "state_dict",
            "params_M": round(sum(p.numel() for p in model.parameters()) / 1e6, 2)}
    if impl in ("opt", "friendly"):
        from . import fast as clf_fast
        mode = "friendly" if impl == "friendly" else "max"
        # fold + fp16 on the CPU, then move: no fp32 copy on the device (as the reference, classification/zoo.py:180-181)
        model = clf_fast.optimize(model, spec, mode, graphs=graphs, **kw).to(device)
    elif impl == "base":
        model = model.to(device)
    else:
        raise ValueError(impl)
    return Loaded(model, _transform(spec.size), (3, spec.size, spec.size), spec, info)
