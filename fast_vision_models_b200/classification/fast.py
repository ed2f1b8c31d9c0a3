"""`optimize(model, spec, mode)`: turns an upstream fp32 torchvision classifier into its B200 tier.

Counterpart of the reference's optimiser (classification/fast/__init__.py:283-374), which folds BatchNorm, casts to
fp16 channels-last and rewrites the fx graph into `clf.*` ops. Here the same partition into fused ops is produced by
walking the upstream module tree of the supported families:

  ResNet (Bottleneck / BasicBlock; also the dilated variant DeepLabV3 uses)
      conv+BN+ReLU -> FusedConv(act=relu); the block's last conv takes the identity as fused residual (+ReLU);
      stem: fp32 NCHW -> fp16 NHWC8 (input_nhwc8) + 7x7 conv on zero-padded channels; 3x3 max pool; GAP; FC as GEMM.
  EfficientNet (MBConv)
      expand 1x1 (SiLU) -> depthwise kxk (SiLU) -> squeeze-excite (GAP, gate, scale) -> project 1x1 with the
      residual add fused into its epilogue (the reference leaves those adds to aten).
  ConvNeXt (CNBlock)
      depthwise 7x7 -> channels-last LayerNorm -> fc1+GELU -> fc2 with LayerScale folded (or applied as an fp32
      epilogue scale) and the residual fused: the op order of the reference's ConvNeXt block
      (classification/fast/convnext.py:50-61).

Modes: "max" / "b200" = this tier; "friendly" = fold + fp16 channels-last on plain PyTorch (the portable tier, kept as
an on-device second opinion in tests). Every returned module maps fp32 NCHW input to fp32 logits, as `Fast` does
(classification/fast/__init__.py:81-95).
"""
from __future__ import annotations

import copy
import os
from typing import Optional

import torch
from torch import nn

from .. import fold, ops
from ..layers import GATE_IN_WEIGHTS, DepthwiseConv, FusedConv, LayerNormCL, SqueezeExcite, act_code
from ..runtime import GraphRunner, HostPipeline

# Bottleneck stages as chain launches (ops.chain_begin): measured on B200 at batch 64, one launch per layer is as fast
# (stage 4 only: 1.127 against 1.129 ms per forward) or faster (from stage 3: 1.16 ms, from stage 2: 1.17-1.19 ms),
# because a layer of these stages has about as many tiles as there are CTA pairs and the next layer's tiles wait for
# them just as a next launch would. Off unless asked for.
CHAIN_RESNET = os.environ.get("FVM_B200_CHAIN_RESNET", "0") == "1"
# The last convolution of a bottleneck block and the first of the next block as one launch (ops.pw_dual) where the
# shapes allow it (64 -> 256 -> 64 channels: the first stage of a ResNet-50/101/152). FVM_B200_DUAL=0: one launch each.
DUAL_RESNET = os.environ.get("FVM_B200_DUAL", "1") != "0"
# Also where the second layer has more than 64 channels (the first block of stage 2: 64 -> 256 -> 128): 62 against 78 us
# when the pair is timed alone, but 0.4 % slower inside a ResNet-50 forward at batch 64 (59.55 against 59.81 k img/s on
# one B200: as its own launch that layer reads most of y from L2, back to front). Off unless asked for.
DUAL_WIDE = os.environ.get("FVM_B200_DUAL_WIDE", "0") == "1"


# ------------------------------------------------------------------------------------------------ ResNet
class ResNetTrunk(nn.Module):
    """conv1..layer4 of a torchvision ResNet on fp16 NHWC tensors. Returns the layer4 feature map (and layer3's)."""

    def __init__(self, m: nn.Module):
        super().__init__()
        self.stem = FusedConv.from_conv_bn(m.conv1, m.bn1, ops.ACT_RELU)
        mp = m.maxpool
        self.pool = (mp.kernel_size, mp.stride, mp.padding, bool(mp.ceil_mode))
        blocks = []
        self.stage_ends = []
        for layer in (m.layer1, m.layer2, m.layer3, m.layer4):
            for blk in layer:
                convs = nn.ModuleList()
                if hasattr(blk, "conv3"):
                    convs.append(FusedConv.from_conv_bn(blk.conv1, blk.bn1, ops.ACT_RELU))
                    convs.append(FusedConv.from_conv_bn(blk.conv2, blk.bn2, ops.ACT_RELU))
                    convs.append(FusedConv.from_conv_bn(blk.conv3, blk.bn3, ops.ACT_RELU))   # + residual, then ReLU
                else:
                    convs.append(FusedConv.from_conv_bn(blk.conv1, blk.bn1, ops.ACT_RELU))
                    convs.append(FusedConv.from_conv_bn(blk.conv2, blk.bn2, ops.ACT_RELU))
                ds = None
                if blk.downsample is not None:
                    ds = FusedConv.from_conv_bn(blk.downsample[0], blk.downsample[1], ops.ACT_NONE)
                blocks.append(nn.ModuleDict({"convs": convs, **({"ds": ds} if ds is not None else {})}))
            self.stage_ends.append(len(blocks))
        self.blocks = nn.ModuleList(blocks)
        self.out_channels = self.blocks[-1]["convs"][-1].out_channels
        # first block whose convolutions run as chain launches (FVM_B200_CHAIN_STAGE = 2, 3 or 4: from that stage on; the
        # first stage's 3x3 layers over 64 channels are faster on staged input patches, which the chain kernel lacks)
        stage = min(4, max(2, int(os.environ.get("FVM_B200_CHAIN_STAGE", "2"))))
        self.chain_from = self.stage_ends[stage - 2] if CHAIN_RESNET else len(blocks)
        # blocks whose last convolution runs together with the next block's first one
        self.dual_after = set()
        for i in range(len(blocks) - 1):
            last, nxt = blocks[i]["convs"][-1], blocks[i + 1]["convs"][0]
            plain = all(c.stride == (1, 1) and c.padding == (0, 0) and c.scale is None and tuple(c.w.shape[2:]) == (1, 1)
                        for c in (last, nxt))
            if DUAL_RESNET and plain and len(blocks[i]["convs"]) == 3 and len(blocks[i + 1]["convs"]) == 3 \
                    and nxt.w.shape[1] == last.w.shape[0] and ops.pw_dual_ok(last.w.shape[1], last.w.shape[0], nxt.w.shape[0]) \
                    and (DUAL_WIDE or nxt.w.shape[0] <= 64):
                self.dual_after.add(i)

    def forward(self, x: torch.Tensor, want_stage3: bool = False):
        # fp32 / fp16 NCHW image batch (fewer than 8 channels), or an fp16 NHWC8 tensor (clf::input_nhwc8's output)
        x = self.stem.forward_image(x) if x.shape[1] < 8 else self.stem(x)
        k, s, p, ceil = self.pool
        x = ops.maxpool(x, k, s, p, ceil)
        aux = None
        chained = False
        head = None
        try:
            for i, blk in enumerate(self.blocks):
                if i == self.chain_from:
                    # from here on the convolutions are recorded and go out as chain launches (one kernel per run of up
                    # to 48 layers, tiles ordered by their data dependencies) instead of one launch per layer
                    chained = ops.chain_begin()
                identity = blk["ds"](x) if "ds" in blk else x
                convs = blk["convs"]
                if head is not None:
                    y, first = head, 1       # this block's first convolution already ran with the previous block's last
                    head = None
                else:
                    y, first = x, 0
                for c in convs[first:-1]:
                    y = c(y)
                nxt = self.blocks[i + 1]["convs"][0] if i in self.dual_after and not chained else None
                if nxt is not None:
                    last = convs[-1]
                    x, head = ops.pw_dual(y, last.w, last.b, identity, last.act, nxt.w, nxt.b, nxt.act)
                else:
                    x = convs[-1](y, res=identity)
                if want_stage3 and i + 1 == self.stage_ends[2]:
                    aux = x
        finally:
            if chained:
                ops.chain_end()
        return (x, aux) if want_stage3 else x


class B200ResNet(nn.Module):
    def __init__(self, m: nn.Module):
        super().__init__()
        self.trunk = ResNetTrunk(m)
        self.fc = FusedConv.from_linear(m.fc)
        self.num_classes = m.fc.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.trunk(x)
        g = ops.global_avgpool(x)
        y = self.fc(g)
        return y.flatten(1)[:, : self.num_classes].float()


# ------------------------------------------------------------------------------------------------ EfficientNet
def _cna(seq) -> tuple:
    """torchvision Conv2dNormActivation -> (conv, norm or None, activation code)."""
    conv = seq[0]
    norm = seq[1] if len(seq) > 1 and isinstance(seq[1], (nn.BatchNorm2d, nn.LayerNorm)) else None
    act = None
    for mod in list(seq)[1:]:
        if not isinstance(mod, (nn.BatchNorm2d, nn.LayerNorm)):
            act = mod
    return conv, norm, act_code(act)


class MBConvBlock(nn.Module):
    def __init__(self, blk: nn.Module):
        super().__init__()
        layers = list(blk.block)
        self.expand = None
        i = 0
        if len(layers) == 4:
            conv, bn, act = _cna(layers[0])
            self.expand = FusedConv.from_conv_bn(conv, bn, act)
            i = 1
        conv, bn, act = _cna(layers[i])
        self.dw = DepthwiseConv(conv, bn, act)
        se = layers[i + 1]
        self.se = SqueezeExcite(se.fc1, se.fc2, act_code(se.activation))
        if not isinstance(se.scale_activation, nn.Sigmoid):
            raise ValueError("MBConv: squeeze-excite gate must be a sigmoid")
        conv, bn, act = _cna(layers[i + 2])
        self.project = FusedConv.from_conv_bn(conv, bn, act)
        self.use_res = bool(blk.use_res_connect)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.expand(x) if self.expand is not None else x
        y, partial = self.dw(y, pool=True)      # the squeeze sums come out of the depthwise conv's epilogue
        res = x if self.use_res else None      # eval-mode stochastic depth is the identity: the add rides in the epilogue
        pj = self.project
        if (GATE_IN_WEIGHTS and pj.scale is None and pj.w.shape[2] == 1 and pj.w.shape[3] == 1 and pj.stride == (1, 1)
                and 2 * pj.w.shape[0] <= y.shape[2] * y.shape[3]):
            # the gate multiplies the project conv's weights (per image) instead of the activations: no pass over y.
            # Only where an image has at least twice as many pixels as the conv has output channels: the per-image
            # weights [K][C] are then less than half the size of the tensor [pixels][C] they save a pass over.
            w_n = ops.gate_weights(pj.w, self.se.gate(y, partial))
            return ops.conv1x1_wbatch(y, w_n, pj.b, res, pj.act)
        return pj(self.se(y, partial), res=res)


class B200EfficientNet(nn.Module):
    def __init__(self, m: nn.Module):
        super().__init__()
        feats = list(m.features)
        conv, bn, act = _cna(feats[0])
        self.stem = FusedConv.from_conv_bn(conv, bn, act)
        blocks = []
        for stage in feats[1:-1]:
            for blk in stage:
                blocks.append(MBConvBlock(blk))
        self.blocks = nn.ModuleList(blocks)
        conv, bn, act = _cna(feats[-1])
        self.head = FusedConv.from_conv_bn(conv, bn, act)
        lin = [c for c in m.classifier if isinstance(c, nn.Linear)][0]
        self.fc = FusedConv.from_linear(lin)
        self.num_classes = lin.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.stem.forward_image(x)
        for blk in self.blocks:
            x = blk(x)
        x = self.head(x)
        g = ops.global_avgpool(x)
        return self.fc(g).flatten(1)[:, : self.num_classes].float()


# ------------------------------------------------------------------------------------------------ ConvNeXt
class CNBlockB200(nn.Module):
    def __init__(self, blk: nn.Module, fold_scale: bool = True):
        super().__init__()
        dwc, _, ln, fc1, gelu, fc2, _ = list(blk.block)
        self.dw = DepthwiseConv(dwc, None, ops.ACT_NONE)
        self.ln = LayerNormCL(ln)
        self.fc1 = FusedConv.from_linear(fc1, act_code(gelu))
        gamma = blk.layer_scale.detach().float().reshape(-1)
        if fold_scale:
            self.fc2 = FusedConv.from_linear(fc2, ops.ACT_NONE, gamma=gamma)
        else:
            self.fc2 = FusedConv.from_linear(fc2, ops.ACT_NONE)
            self.fc2.scale = gamma.contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.dw(x)
        y = self.ln(y)
        y = self.fc1(y)
        return self.fc2(y, res=x)


class B200ConvNeXt(nn.Module):
    """torchvision ConvNeXt. `fold_scale=True` folds LayerScale into fc2 in fp32 before the fp16 cast, as the reference
    does (convnext.py:17-23); with the published init of 1e-6 the folded fp16 weights underflow (in the reference too).
    `fold_scale=False` keeps LayerScale as an fp32 per-channel scale in the GEMM epilogue instead."""

    def __init__(self, m: nn.Module, fold_scale: bool = True):
        super().__init__()
        feats = list(m.features)
        conv, ln, _ = _cna(feats[0])
        self.stem = FusedConv.from_conv_bn(conv, None, ops.ACT_NONE)
        self.stem_ln = LayerNormCL(ln)
        stages = []
        for f in feats[1:]:
            if isinstance(f[0], nn.LayerNorm):      # downsample: LayerNorm2d + 2x2 stride-2 conv
                stages.append(nn.ModuleList([LayerNormCL(f[0]), FusedConv.from_conv_bn(f[1], None, ops.ACT_NONE)]))
            else:
                stages.append(nn.ModuleList([CNBlockB200(b, fold_scale) for b in f]))
        self.stages = nn.ModuleList(stages)
        self.kinds = [isinstance(f[0], nn.LayerNorm) for f in feats[1:]]
        self.head_ln = LayerNormCL(m.classifier[0])
        lin = m.classifier[2]
        self.fc = FusedConv.from_linear(lin)
        self.num_classes = lin.out_features

    def features(self, x: torch.Tensor) -> torch.Tensor:
        x = ops.input_nhwc8(x)
        x = self.stem_ln(self.stem(x))
        for is_ds, st in zip(self.kinds, self.stages):
            if is_ds:
                x = st[1](st[0](x))
            else:
                for blk in st:
                    x = blk(x)
        return x

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.features(x)
        g = self.head_ln(ops.global_avgpool(x))
        return self.fc(g).flatten(1)[:, : self.num_classes].float()


# ------------------------------------------------------------------------------------------------ wrappers
def as_image(x: torch.Tensor) -> torch.Tensor:
    """Network input as the kernels take it: contiguous NCHW, fp32 or fp16 (an fp16 host batch halves the bytes that
    cross PCIe; the first kernel converts either type to fp16 NHWC, as the reference's templated input kernel does)."""
    if x.dtype not in (torch.float32, torch.float16):
        x = x.float()
    return x.contiguous()


class Fast(nn.Module):
    """fp32 (or fp16) NCHW in -> compiled fp16 NHWC network -> fp32 out, replayed as one CUDA graph per input shape
    (counterpart of the reference's `Fast`, classification/fast/__init__.py:45-95)."""

    def __init__(self, net: nn.Module, graphs: bool = True):
        super().__init__()
        self.net = net
        self._runner = GraphRunner(self._run, enabled=graphs)

    def _run(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise ops.FvmError("the b200 tier runs on a CUDA device only (no CPU path)")
        return self._runner(as_image(x))

    @property
    def runner(self) -> GraphRunner:
        return self._runner

    def host_pipeline(self, example: torch.Tensor, replicas: int = 2) -> HostPipeline:
        """A serving loop for batches that arrive in pinned host memory: `replicas` graph replicas of this network in
        rotation, host -> device and device -> host copies on their own streams (runtime.HostPipeline). `example` is a
        batch of the shape and dtype (fp32 or fp16 NCHW image batch) that will be submitted."""
        runners = [self._runner] + [Fast(self.net).runner for _ in range(max(2, replicas) - 1)]
        return HostPipeline(runners, as_image(example))


class Portable(nn.Module):
    """The portable tier: BatchNorm folded in fp32, fp16, channels-last, plain PyTorch ops (reference mode "friendly")."""

    def __init__(self, model: nn.Module):
        super().__init__()
        self.net = fold_bn_inplace(copy.deepcopy(model)).half().to(memory_format=torch.channels_last)

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(x.to(torch.float16, memory_format=torch.channels_last)).float()


def fold_bn_inplace(model: nn.Module) -> nn.Module:
    """Folds every (Conv2d, BatchNorm2d) pair that sits back to back inside an nn.Sequential or as convN/bnN attributes."""
    for mod in model.modules():
        kids = list(mod.named_children())
        for (n1, c), (n2, b) in zip(kids, kids[1:]):
            if isinstance(c, nn.Conv2d) and isinstance(b, nn.BatchNorm2d):
                w, bias = fold.fold_conv_bn(c, b)
                c.weight.data = w
                c.bias = nn.Parameter(bias)
                setattr(mod, n2, nn.Identity())
    return model


def compile_model(model: nn.Module, family_hint: Optional[str] = None, **kw) -> nn.Module:
    name = type(model).__name__
    if name == "ResNet":
        return B200ResNet(model)
    if name == "EfficientNet":
        return B200EfficientNet(model)
    if name == "ConvNeXt":
        return B200ConvNeXt(model, **kw)
    # every other architecture: the generic graph pass (conv -> [add] -> [act] chains, depthwise, pools, ...)
    from .fused import fuse_graph
    return fuse_graph(model)


def optimize(model: nn.Module, spec=None, mode: str = "max", graphs: bool = True, **kw) -> nn.Module:
    """optimize(model, spec, mode) -> module (reference: classification/fast/__init__.py:283)."""
    model = model.eval()
    if mode in ("max", "opt", "b200", "cuda-kernels"):
        return Fast(compile_model(model, getattr(spec, "family", None), **kw), graphs=graphs)
    if mode in ("friendly", "portable"):
        return Portable(model)
    raise ValueError(mode)
