"""Generates tests/golden/*.npz from the reference's OWN code (run in the development container only).

For each hot-path family the upstream torchvision model is built with this repo's seeded initialisation, then run
through the reference's portable tier on the CPU (`fast_vision_models.classification.fast.optimize(model, spec,
"friendly")`: BatchNorm fold, fp16, channels-last) and in plain fp32. The logits are the golden vectors that pin the
CPU oracle. Inputs and weights are regenerated from seeds by the tests, so only the outputs are stored.

    FVM_REFERENCE=<path of the reference checkout> python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("FVM_REFERENCE", os.path.join(os.sep, "root", "reference"))
sys.path.insert(0, REF)
sys.path.insert(0, ROOT)

from fast_vision_models.classification import fast as ref_fast          # noqa: E402  (the reference)
from fast_vision_models.classification import zoo as ref_zoo            # noqa: E402
from fast_vision_models_b200.classification import zoo as zoo           # noqa: E402
from fast_vision_models_b200.weights import seeded_input                # noqa: E402

CASES = [
    # name, input shape, layer_scale
    ("resnet50", (2, 3, 64, 64), None),
    ("resnet50", (2, 3, 224, 224), None),
    ("efficientnet_b4", (2, 3, 96, 96), None),
    ("convnext_tiny", (2, 3, 64, 64), 1e-6),
    ("convnext_tiny", (2, 3, 64, 64), "uniform"),
]


def ref_spec(name):
    if name in ref_zoo.BY_NAME:
        return ref_zoo.BY_NAME[name]
    # torchvision ConvNeXt is not in the reference registry: a synthetic spec of its depthwise-CNN family
    return ref_zoo.Spec(name, 2022, "tv", name, "dwcnn")


def main():
    torch.manual_seed(0)
    for name, shape, ls in CASES:
        model = zoo.build_upstream(name, seed=1, layer_scale=ls)
        x = seeded_input(shape, seed=0)
        with torch.inference_mode():
            y32 = model(x).float()
        import copy
        port = ref_fast.optimize(copy.deepcopy(model), ref_spec(name), "friendly")
        with torch.inference_mode():
            yp = port(x).float()
        tag = f"{name}_{shape[0]}x{shape[2]}" + ("" if ls is None else f"_ls{ls}")
        rel = float((yp - y32).norm() / y32.norm())
        np.savez_compressed(os.path.join(HERE, tag + ".npz"), portable=yp.numpy(), fp32=y32.numpy(),
                            shape=np.array(shape), rel_l2_portable_vs_fp32=np.array(rel))
        print(tag, "portable vs fp32 rel-L2", rel, "argmax agree", float((yp.argmax(1) == y32.argmax(1)).float().mean()))


if __name__ == "__main__":
    main()
