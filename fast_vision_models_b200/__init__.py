"""B200 (sm_100a) tier of the fast-vision-models convolutional hot path.

    from fast_vision_models_b200 import zoo, seg, backbones
    m = zoo.load("resnet50", "b200")             # classification registry (reference: classification/zoo.py)
    w = seg.build("deeplabv3-r50", "b200")       # segmentation registry   (reference: segmentation/zoo.py)
    b = backbones.build("tv-resnet50", "b200")   # feature extractors      (reference: backbones/__init__.py)

`ops` is the operator layer over the C-ABI library, `torch_ops.register()` exposes it as `torch.ops.clf / clfr3 / segx`.
Importing this package does not load the CUDA library; the first op does.
"""
from . import backbones  # noqa: F401
from .classification import zoo  # noqa: F401
from .segmentation import zoo as seg  # noqa: F401
