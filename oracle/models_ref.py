"""Whole-network CPU restatements of the reference's fused-op partition (TEST INFRASTRUCTURE ONLY).

Each function takes the upstream fp32 torchvision model and an fp32 NCHW input and evaluates the network the way the
reference's kernel tier partitions it: BatchNorm folded in fp32 (classification/fast/__init__.py:201-208), weights and
activations rounded to fp16 at every fused-op boundary, fp32 arithmetic inside each op (oracle/ops_ref.py).
Also here: the upstream fp32 forward timed as the CPU baseline (`upstream_fp32`).
"""
from __future__ import annotations

import time

import torch
from torch import nn

from . import ops_ref as R


def fold_bn_ref(conv: nn.Conv2d, bn):
    """sc = gamma / sqrt(var + eps); w' = w*sc; b' = b*sc + beta - mean*sc  (classification/fast/__init__.py:203-208)."""
    w = conv.weight.detach().float()
    b = conv.bias.detach().float() if conv.bias is not None else None
    if bn is None or not isinstance(bn, nn.BatchNorm2d):
        return w.half(), (b if b is not None else torch.zeros(w.shape[0])).half()
    sc = bn.weight.detach().float() / torch.sqrt(bn.running_var.detach().float() + bn.eps)
    sh = bn.bias.detach().float() - bn.running_mean.detach().float() * sc
    w = w * sc.view(-1, 1, 1, 1)
    b = b * sc + sh if b is not None else sh
    return w.half(), b.half()


_ACTS = {nn.ReLU: 1, nn.ReLU6: 2, nn.SiLU: 3, nn.Hardswish: 4}


def _act_code(m):
    if m is None or isinstance(m, nn.Identity):
        return 0
    for k, v in _ACTS.items():
        if isinstance(m, k):
            return v
    if isinstance(m, nn.GELU):
        return 6 if getattr(m, "approximate", "none") == "tanh" else 5
    raise ValueError(type(m))


def _conv(x, conv, bn, act, res=None):
    w, b = fold_bn_ref(conv, bn)
    return R.conv_fused_ref(x, w, b, res, conv.padding, conv.stride, act, conv.dilation)


def _dw(x, conv, bn, act):
    w, b = fold_bn_ref(conv, bn)
    return R.dwconv_ref(x, w[:, 0].permute(1, 2, 0).contiguous(), b, conv.stride, conv.padding, act, conv.dilation)


@torch.no_grad()
def resnet_trunk_ref(m, x, want_stage3=False):
    x = _conv(x, m.conv1, m.bn1, 1)
    mp = m.maxpool
    x = R.maxpool_ref(x, mp.kernel_size, mp.stride, mp.padding, mp.ceil_mode)
    aux = None
    for li, layer in enumerate((m.layer1, m.layer2, m.layer3, m.layer4)):
        for blk in layer:
            idn = x if blk.downsample is None else _conv(x, blk.downsample[0], blk.downsample[1], 0)
            if hasattr(blk, "conv3"):
                y = _conv(x, blk.conv1, blk.bn1, 1)
                y = _conv(y, blk.conv2, blk.bn2, 1)
                x = _conv(y, blk.conv3, blk.bn3, 1, res=idn)
            else:
                y = _conv(x, blk.conv1, blk.bn1, 1)
                x = _conv(y, blk.conv2, blk.bn2, 1, res=idn)
        if li == 2:
            aux = x
    return (x, aux) if want_stage3 else x


@torch.no_grad()
def resnet_ref(m, x):
    x = R.input_nhwc8_ref(x)[:, :3]
    x = resnet_trunk_ref(m, x)
    g = R.global_avgpool_ref(x)
    w = m.fc.weight.detach().half()
    return R.conv_fused_ref(g, w.view(w.shape[0], -1, 1, 1), m.fc.bias.detach().half()).flatten(1).float()


def _cna(seq):
    conv = seq[0]
    norm = seq[1] if len(seq) > 1 and isinstance(seq[1], (nn.BatchNorm2d, nn.LayerNorm)) else None
    act = None
    for mod in list(seq)[1:]:
        if not isinstance(mod, (nn.BatchNorm2d, nn.LayerNorm)):
            act = mod
    return conv, norm, _act_code(act)


@torch.no_grad()
def efficientnet_ref(m, x):
    """MBConv partition: expand conv_fused(SiLU) -> dwconv(SiLU) -> GAP -> 2 FCs -> se_scale -> project conv_fused with
    the residual in its epilogue (eval-mode stochastic depth is the identity)."""
    x = R.input_nhwc8_ref(x)[:, :3]
    feats = list(m.features)
    conv, bn, act = _cna(feats[0])
    x = _conv(x, conv, bn, act)
    for stage in feats[1:-1]:
        for blk in stage:
            layers = list(blk.block)
            y = x
            i = 0
            if len(layers) == 4:
                conv, bn, act = _cna(layers[0])
                y = _conv(y, conv, bn, act)
                i = 1
            conv, bn, act = _cna(layers[i])
            y = _dw(y, conv, bn, act)
            se = layers[i + 1]
            g = R.global_avgpool_ref(y)
            s = R.se_gate_ref(g, se.fc1.weight.detach().half().flatten(1), se.fc1.bias.detach().half(),
                              se.fc2.weight.detach().half().flatten(1), se.fc2.bias.detach().half(),
                              _act_code(se.activation))
            y = R.se_scale_ref(y, s)
            conv, bn, act = _cna(layers[i + 2])
            x = _conv(y, conv, bn, act, res=x if blk.use_res_connect else None)
    conv, bn, act = _cna(feats[-1])
    x = _conv(x, conv, bn, act)
    g = R.global_avgpool_ref(x)
    lin = [c for c in m.classifier if isinstance(c, nn.Linear)][0]
    w = lin.weight.detach().half()
    return R.conv_fused_ref(g, w.view(w.shape[0], -1, 1, 1), lin.bias.detach().half()).flatten(1).float()


def _ln2d(x, ln):
    return R.layernorm_cl_ref(x, ln.weight.detach().half(), ln.bias.detach().half(), ln.eps)


@torch.no_grad()
def convnext_features_ref(m, x, fold_scale=True):
    """ConvNeXt block order of the reference (classification/fast/convnext.py:50-61): dwconv 7x7 -> LayerNorm ->
    fc1 + GELU -> fc2 (LayerScale folded in fp32 then cast, :17-23) + residual."""
    x = R.input_nhwc8_ref(x)[:, :3]
    feats = list(m.features)
    conv, ln, _ = _cna(feats[0])
    x = _ln2d(_conv(x, conv, None, 0), ln)
    for f in feats[1:]:
        if isinstance(f[0], nn.LayerNorm):
            x = _conv(_ln2d(x, f[0]), f[1], None, 0)
            continue
        for blk in f:
            dwc, _, ln, fc1, gelu, fc2, _ = list(blk.block)
            y = _dw(x, dwc, None, 0)
            y = _ln2d(y, ln)
            w1 = fc1.weight.detach().half()
            y = R.conv_fused_ref(y, w1.view(w1.shape[0], -1, 1, 1), fc1.bias.detach().half(), act=_act_code(gelu))
            gamma = blk.layer_scale.detach().float().reshape(-1)
            if fold_scale:
                w2 = (fc2.weight.detach().float() * gamma.view(-1, 1)).half()
                b2 = (fc2.bias.detach().float() * gamma).half()
                x = R.conv_fused_ref(y, w2.view(w2.shape[0], -1, 1, 1), b2, res=x)
            else:
                w2 = fc2.weight.detach().half()
                x = R.conv_fused_ref(y, w2.view(w2.shape[0], -1, 1, 1), fc2.bias.detach().half(), res=x, scale=gamma)
    return x


@torch.no_grad()
def convnext_ref(m, x, fold_scale=True):
    x = convnext_features_ref(m, x, fold_scale)
    g = _ln2d(R.global_avgpool_ref(x), m.classifier[0])
    lin = m.classifier[2]
    w = lin.weight.detach().half()
    return R.conv_fused_ref(g, w.view(w.shape[0], -1, 1, 1), lin.bias.detach().half()).flatten(1).float()


@torch.no_grad()
def deeplabv3_logits_ref(m, x):
    """torchvision DeepLabV3-ResNet50 (output stride 8) up to the low-resolution logits: every conv+BN(+ReLU) is one
    fused conv (segmentation/fast/cnn_fuse.py:46-64), the ASPP image-pool branch is GAP -> 1x1 -> bilinear resize
    (align_corners=False), the class head is zero-padded to a multiple of 8 channels and sliced (cnn_fuse.py:30-40)."""
    x = R.input_nhwc8_ref(x)[:, :3]
    feat = resnet_trunk_ref(m.backbone, x)
    aspp = m.classifier[0]
    outs = []
    for br in aspp.convs:
        mods = list(br)
        if isinstance(mods[0], nn.AdaptiveAvgPool2d):
            g = R.global_avgpool_ref(feat)
            g = _conv(g, mods[1], mods[2], 1)
            outs.append(R.bilinear_ref(g, feat.shape[2], feat.shape[3], align=False))
        else:
            outs.append(_conv(feat, mods[0], mods[1], 1))
    cat = torch.cat(outs, dim=1)
    proj = list(aspp.project)
    y = _conv(cat, proj[0], proj[1], 1)          # Dropout is the identity in eval mode
    y = _conv(y, m.classifier[1], m.classifier[2], 1)
    return _conv(y, m.classifier[4], None, 0)


@torch.no_grad()
def deeplabv3_classmap_ref(m, x):
    logits = deeplabv3_logits_ref(m, x)
    return R.up_argmax_ref(logits, x.shape[2], x.shape[3], align=False)


REFS = {"ResNet": resnet_ref, "EfficientNet": efficientnet_ref, "ConvNeXt": convnext_ref}


def model_ref(m, x, **kw):
    return REFS[type(m).__name__](m, x, **kw)


@torch.no_grad()
def upstream_fp32(m, x, warmup=1, iters=3, threads=None):
    """The reference's upstream tier on the CPU (the unmodified fp32 model, classification/zoo.py:182-183), timed.
    Returns (logits, seconds per forward (median), threads used)."""
    import statistics
    if threads:
        torch.set_num_threads(int(threads))
    m = m.eval().float()
    for _ in range(warmup):
        y = m(x)
    ts = []
    for _ in range(iters):
        t0 = time.perf_counter()
        y = m(x)
        ts.append(time.perf_counter() - t0)
    return y, statistics.median(ts), torch.get_num_threads()
