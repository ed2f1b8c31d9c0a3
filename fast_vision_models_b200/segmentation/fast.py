"""DeepLabV3 (dilated ResNet backbone, ASPP head) on the B200 kernels.

Counterpart of the reference's CNN segmentation path (segmentation/fast/cnn.py:144-174 optimize, cnn_fuse.py:19-133
conv + bias + ReLU + residual epilogues, mmseg_fast.py:59-105 FastMMSeg with the fused upsample+argmax):
  * every conv + BatchNorm (+ ReLU) is one fused conv; dilated 3x3 convs (rates 2/4 in the backbone, 12/24/36 in ASPP)
    run on the same implicit-GEMM kernel, the dilation is resolved by the im2col tensor map;
  * the five ASPP branches write straight into channel slices of one [N, 5*256, h, w] buffer (no concat copy,
    the reference's `conv_fused_into`, fused_conv.cu:303-306); the image-pool branch is GAP -> 1x1 conv -> bilinear
    resize (align_corners=False) into its slice;
  * the class head is zero-padded to a multiple of 8 channels (cnn_fuse.py:30-40);
  * `predict` upsamples and takes the arg-max in one kernel without materialising full-resolution scores.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import ops
from ..classification.fast import ResNetTrunk, as_image
from ..layers import FusedConv
from ..runtime import GraphRunner


class B200DeepLabV3(nn.Module):
    def __init__(self, m: nn.Module):
        super().__init__()
        self.trunk = ResNetTrunk(m.backbone)
        head = m.classifier
        aspp = head[0]
        branches = []
        self.pool_branch = None
        for br in aspp.convs:
            mods = list(br)
            if isinstance(mods[0], nn.AdaptiveAvgPool2d):
                self.pool_branch = FusedConv.from_conv_bn(mods[1], mods[2], ops.ACT_RELU)
            else:
                branches.append(FusedConv.from_conv_bn(mods[0], mods[1], ops.ACT_RELU))
        self.branches = nn.ModuleList(branches)
        proj = list(aspp.project)
        self.project = FusedConv.from_conv_bn(proj[0], proj[1], ops.ACT_RELU)     # Dropout: identity in eval mode
        self.head_conv = FusedConv.from_conv_bn(head[1], head[2], ops.ACT_RELU)
        self.cls = FusedConv.from_conv_bn(head[4], None, ops.ACT_NONE)
        self.num_classes = head[4].out_channels
        self.branch_channels = self.branches[0].out_channels

    def logits_nhwc(self, x: torch.Tensor) -> torch.Tensor:
        """fp32 NCHW image batch -> low-resolution fp16 scores [N, round_up(classes, 8), H/8, W/8] (channels-last)."""
        feat = self.trunk(x)
        N, _, h, w = feat.shape
        C = self.branch_channels
        nb = len(self.branches) + (1 if self.pool_branch is not None else 0)
        cat = ops.empty_nhwc(N, nb * C, h, w, feat.device)
        for i, br in enumerate(self.branches):
            br(feat, out=cat[:, i * C:(i + 1) * C])
        if self.pool_branch is not None:
            g = self.pool_branch(ops.global_avgpool(feat))
            i = len(self.branches)
            ops.upsample_bilinear(g, h, w, align=False, out=cat[:, i * C:(i + 1) * C])
        y = self.project(cat)
        y = self.head_conv(y)
        return self.cls(y)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Low-resolution fp32 logits [N, classes, H/8, W/8] (NCHW)."""
        return self.logits_nhwc(x)[:, : self.num_classes].float().contiguous()

    def classmap(self, x: torch.Tensor) -> torch.Tensor:
        s = self.logits_nhwc(x)
        return ops.up_argmax(s, x.shape[2], x.shape[3], align=False, num_classes=self.num_classes)


class FastSeg(nn.Module):
    """Wrapper with CUDA-graph replay: .logits(x) -> fp32 low-res logits, .predict(x, out_size) -> int32 class map."""

    def __init__(self, net: B200DeepLabV3, graphs: bool = True):
        super().__init__()
        self.net = net
        self._logits = GraphRunner(lambda x: self.net(x), enabled=graphs)
        self._classmap = GraphRunner(lambda x: self.net.classmap(x), enabled=graphs)
        self.info = {"tier": "b200", "fused_upsample_argmax": True}

    @torch.no_grad()
    def logits(self, x: torch.Tensor) -> torch.Tensor:
        return self._logits(as_image(x))

    @torch.no_grad()
    def predict(self, x: torch.Tensor, out_size=None) -> torch.Tensor:
        if out_size is not None and tuple(out_size) != tuple(x.shape[2:]):
            s = self.net.logits_nhwc(as_image(x))
            return ops.up_argmax(s, int(out_size[0]), int(out_size[1]), align=False, num_classes=self.net.num_classes)
        return self._classmap(as_image(x))

    forward = logits
