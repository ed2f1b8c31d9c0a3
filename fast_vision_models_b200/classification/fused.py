"""Generic graph pass: any torch.fx-traceable eval-mode CNN -> fp16 channels-last graph on the registered `torch.ops`.

Counterpart of the reference's `fuse_graph` / `fuse_dw` / `replace_bn_act` / `replace_maxpool` / `replace_avgpool`
(classification/fast/fused.py:163-312): the traced graph is rewritten so that

  Conv2d(groups=1, zero padding, C % 8 == 0, K % 8 == 0) [-> BatchNorm2d] [-> add(other)] [-> activation]
  Conv2d(1 < groups < C, C % 8 == 0, K % 8 == 0) [-> BatchNorm2d] [-> activation]          -> clfr3.gconv2
                                                  ==> torch.ops.clf.conv_fused(x, w, b, res, padding, stride, act)
  (dilated)                                       ==> torch.ops.segx.conv_fused_d(..., dilation, act)
  depthwise Conv2d [-> BatchNorm2d] [-> activation] ==> torch.ops.clf.dwconv(x, w_rsc, b, stride, padding, act)
  BatchNorm2d that cannot be folded [-> ReLU]     ==> torch.ops.clf.affine_act(x, scale, shift, act)
  MaxPool2d / AvgPool2d                           ==> torch.ops.clf.maxpool / clf.avgpool
  sigmoid(s) * x  (squeeze-excite scale)          ==> torch.ops.clfr3.se_scale(x, s)
  AdaptiveAvgPool2d(1), Linear                    ==> this library's global average pool and GEMM modules
  first conv on an image with fewer than 8 channels: weights zero-padded to 8, input through torch.ops.clf.input_nhwc8

BatchNorm and the weights are folded in fp32 and rounded once (fold.py). Everything the patterns do not cover
(channel counts that are not multiples of 8, concatenations, ...) stays an aten op on fp16 channels-last
tensors, as in the reference. `classification/fast.py` keeps hand-built compilers for ResNet, EfficientNet and ConvNeXt
(per-layer tile tuning, fused squeeze); this pass is what every other architecture gets.
"""
from __future__ import annotations

import copy
import operator
from typing import Dict, Optional

import torch
import torch.fx as fx
import torch.nn.functional as F
from torch import nn

from .. import fold, ops, torch_ops
from ..layers import act_code

_ADDS = (operator.add, operator.iadd, torch.add)
_FN_ACTS = {F.relu: ops.ACT_RELU, torch.relu: ops.ACT_RELU, F.relu6: ops.ACT_RELU6, F.silu: ops.ACT_SILU,
            F.hardswish: ops.ACT_HARDSWISH}


class GapModule(nn.Module):
    """AdaptiveAvgPool2d(1) on a channels-last fp16 tensor -> [N, C, 1, 1] (deterministic fp32 reduction)."""

    def forward(self, x):
        return ops.global_avgpool(x)


class LinearGemm(nn.Module):
    """nn.Linear on [N, C] fp16 rows through the convolution kernel's GEMM view (reference: vit.py:56-64)."""

    def __init__(self, lin: nn.Linear):
        super().__init__()
        K = lin.out_features
        Kp = fold.round_up(K, 8)
        w = torch.zeros(Kp, lin.in_features)
        w[:K] = lin.weight.detach().float()
        b = torch.zeros(Kp)
        if lin.bias is not None:
            b[:K] = lin.bias.detach().float()
        self.register_buffer("w", w.half().contiguous())
        self.register_buffer("b", b.half().contiguous())
        self.out_features = K

    def forward(self, x):
        return ops.linear(x.half(), self.w, self.b)[:, : self.out_features]


class _Tracer(fx.Tracer):
    def is_leaf_module(self, m, qualname):
        return type(m).__name__ == "StochasticDepth" or super().is_leaf_module(m, qualname)


def _act_of(node: fx.Node, mods: Dict[str, nn.Module]) -> Optional[int]:
    """Activation code of a node that is an activation (module, function or method), else None."""
    if node.op == "call_module":
        try:
            code = act_code(mods.get(node.target))
        except ValueError:
            return None
        return code if code != ops.ACT_NONE else None
    if node.op == "call_function":
        if node.target is F.gelu:
            return ops.ACT_GELU_TANH if node.kwargs.get("approximate", "none") == "tanh" else ops.ACT_GELU_ERF
        return _FN_ACTS.get(node.target)
    if node.op == "call_method" and node.target in ("relu", "relu_"):
        return ops.ACT_RELU
    return None


def _single_user(node: fx.Node) -> Optional[fx.Node]:
    users = list(node.users)
    return users[0] if len(users) == 1 else None


class Rewriter:
    def __init__(self, model: nn.Module):
        torch_ops.register()
        model = copy.deepcopy(model).eval()          # the caller's fp32 model stays as it is
        self.gm = fx.GraphModule(model, _Tracer().trace(model))
        self.mods = dict(self.gm.named_modules())
        self.g = self.gm.graph
        self.stats = {"conv_fused": 0, "dwconv": 0, "affine_act": 0, "pool": 0, "se_scale": 0, "gemm": 0, "stem_pad": 0,
                      "left_to_aten": 0}
        self._uid = 0

    # ------------------------------------------------------------------------------------------------ helpers
    def _buffer(self, stem: str, t: torch.Tensor) -> fx.Node:
        name = f"_fvm_{stem}_{self._uid}"
        self._uid += 1
        self.gm.register_buffer(name, t)
        return self.g.get_attr(name)

    def _drop_identities(self):
        for node in list(self.g.nodes):
            if node.op == "call_module" and type(self.mods.get(node.target)).__name__ in ("StochasticDepth", "Dropout", "Identity"):
                node.replace_all_uses_with(node.args[0])
                self.g.erase_node(node)

    # ------------------------------------------------------------------------------------------------ patterns
    def _conv_chain(self, node: fx.Node) -> bool:
        conv = self.mods[node.target]
        if type(conv) is not nn.Conv2d or conv.padding_mode != "zeros" or isinstance(conv.padding, str):
            return False
        C, K = conv.in_channels, conv.out_channels
        depthwise = conv.groups == C == K and C % 8 == 0 and conv.groups > 1
        image_stem = node.args[0].op == "placeholder" and conv.groups == 1 and C < 8 and K % 8 == 0
        dense = conv.groups == 1 and C % 8 == 0 and K % 8 == 0
        # grouped (not depthwise): clfr3.gconv2, the reference's rewrite of RegNet / ResNeXt convolutions (r3.py:166-214)
        grouped = (1 < conv.groups and not depthwise and C % conv.groups == 0 and K % conv.groups == 0 and C % 8 == 0
                   and K % 8 == 0 and conv.dilation == (1, 1))
        if not (depthwise or dense or image_stem or grouped):
            return False
        last, bn = node, None
        u = _single_user(last)
        if u is not None and u.op == "call_module" and type(self.mods.get(u.target)) is nn.BatchNorm2d:
            bn, last = self.mods[u.target], u
        res = None
        u = _single_user(last)
        if not depthwise and not grouped and u is not None and u.op == "call_function" and u.target in _ADDS and len(u.args) == 2 and not u.kwargs:
            other = u.args[1] if u.args[0] is last else u.args[0]
            if isinstance(other, fx.Node) and other is not last:
                res, last = other, u
        act = 0
        u = _single_user(last)
        if u is not None:
            a = _act_of(u, self.mods)
            if a is not None:
                act, last = a, u
        if depthwise and conv.dilation != (1, 1) and act not in (0, ops.ACT_GELU_ERF):
            return False       # segx::dwconv knows no other activation (segmentation/fast/seg_kernels.cu:151-154)
        w, b = fold.fold_conv_bn(conv, bn)
        x = node.args[0]
        with self.g.inserting_before(last.next):
            if depthwise:
                wn = self._buffer("dw_w", fold.dw_to_rsc_half(w))
                bn_ = self._buffer("dw_b", b.half().contiguous())
                if conv.dilation != (1, 1):
                    R, S = conv.kernel_size
                    wt = self._buffer("dw_wt", fold.dw_to_rsc_half(w).reshape(R * S, C).contiguous())
                    new = self.g.call_function(torch.ops.segx.dwconv, (x, wt, bn_, R, S, list(conv.stride), list(conv.padding),
                                                                       list(conv.dilation), 1 if act else 0))
                else:
                    new = self.g.call_function(torch.ops.clf.dwconv, (x, wn, bn_, list(conv.stride), list(conv.padding), act))
                self.stats["dwconv"] += 1
            elif grouped:
                wn = self._buffer("gw", fold.to_krsc_half(w))        # [K, C/groups, R, S], the reference's layout
                bn_ = self._buffer("gb", b.half().contiguous())
                new = self.g.call_function(torch.ops.clfr3.gconv2, (x, wn, bn_, list(conv.stride), list(conv.padding),
                                                                    conv.groups, act))
                self.stats["gconv"] = self.stats.get("gconv", 0) + 1
            else:
                if image_stem:
                    w = fold.pad_in_channels(w, 8)
                    x = self.g.call_function(torch.ops.clf.input_nhwc8, (x,))
                    self.stats["stem_pad"] += 1
                wn = self._buffer("w", fold.to_krsc_half(w))
                bn_ = self._buffer("b", b.half().contiguous())
                if conv.dilation != (1, 1):
                    new = self.g.call_function(torch.ops.segx.conv_fused_d, (x, wn, bn_, res, list(conv.padding), list(conv.stride),
                                                                            list(conv.dilation), act))
                else:
                    new = self.g.call_function(torch.ops.clf.conv_fused, (x, wn, bn_, res, list(conv.padding), list(conv.stride), act))
                self.stats["conv_fused"] += 1
        last.replace_all_uses_with(new)
        return True

    def _bn_alone(self, node: fx.Node) -> bool:
        bn = self.mods[node.target]
        if type(bn) is not nn.BatchNorm2d or bn.num_features % 8:
            return False
        with torch.no_grad():
            sc = (bn.weight.float() if bn.affine else 1.0) / torch.sqrt(bn.running_var.float() + bn.eps)
            sh = (bn.bias.float() if bn.affine else 0.0) - bn.running_mean.float() * sc
        last, act = node, 0
        u = _single_user(node)
        if u is not None and _act_of(u, self.mods) == ops.ACT_RELU:
            last, act = u, ops.ACT_RELU
        with self.g.inserting_before(last.next):
            new = self.g.call_function(torch.ops.clf.affine_act, (node.args[0], self._buffer("bn_sc", sc.contiguous()),
                                                                  self._buffer("bn_sh", sh.contiguous()), act))
        last.replace_all_uses_with(new)
        self.stats["affine_act"] += 1
        return True

    def _pool(self, node: fx.Node) -> bool:
        m = self.mods[node.target]
        pair = ops._pair
        if type(m) is nn.MaxPool2d and pair(m.dilation) == (1, 1) and not m.return_indices:
            args = (node.args[0], list(pair(m.kernel_size)), list(pair(m.stride or m.kernel_size)), list(pair(m.padding)), bool(m.ceil_mode))
            target = torch.ops.clf.maxpool
        elif type(m) is nn.AvgPool2d and not m.ceil_mode and m.divisor_override is None:
            args = (node.args[0], list(pair(m.kernel_size)), list(pair(m.stride or m.kernel_size)), list(pair(m.padding)),
                    bool(m.count_include_pad))
            target = torch.ops.clf.avgpool
        elif type(m) is nn.AdaptiveAvgPool2d and m.output_size in (1, (1, 1)):
            self.gm.add_submodule(node.target, GapModule())
            self.stats["pool"] += 1
            return True
        else:
            return False
        with self.g.inserting_before(node.next):
            new = self.g.call_function(target, args)
        node.replace_all_uses_with(new)
        self.stats["pool"] += 1
        return True

    def _se_scale(self, node: fx.Node) -> bool:
        """sigmoid(s) * x with s [N,C,1,1] -> se_scale(x, s)."""
        is_sig = (node.op == "call_module" and type(self.mods.get(node.target)) is nn.Sigmoid) or \
                 (node.op == "call_function" and node.target in (torch.sigmoid, F.sigmoid))
        u = _single_user(node)
        if not is_sig or u is None or u.op != "call_function" or u.target not in (operator.mul, torch.mul) or len(u.args) != 2:
            return False
        other = u.args[1] if u.args[0] is node else u.args[0]
        if not isinstance(other, fx.Node):
            return False
        with self.g.inserting_before(u.next):
            new = self.g.call_function(torch.ops.clfr3.se_scale, (other, node.args[0]))
        u.replace_all_uses_with(new)
        self.stats["se_scale"] += 1
        return True

    # ------------------------------------------------------------------------------------------------ driver
    def run(self) -> fx.GraphModule:
        self._drop_identities()
        for node in list(self.g.nodes):
            if node.op == "call_module":
                m = self.mods.get(node.target)
                if isinstance(m, nn.Conv2d):
                    if not self._conv_chain(node):
                        self.stats["left_to_aten"] += 1
                elif isinstance(m, nn.Linear):
                    self.gm.add_submodule(node.target, LinearGemm(m))
                    self.stats["gemm"] += 1
                elif isinstance(m, (nn.MaxPool2d, nn.AvgPool2d, nn.AdaptiveAvgPool2d)):
                    self._pool(node)
        self.g.eliminate_dead_code()
        self.mods = dict(self.gm.named_modules())
        for node in list(self.g.nodes):      # what is left of BatchNorm could not be folded into a preceding conv
            if node.op == "call_module" and isinstance(self.mods.get(node.target), nn.BatchNorm2d):
                self._bn_alone(node)
        for node in list(self.g.nodes):
            self._se_scale(node)
        self.g.eliminate_dead_code()
        self.g.lint()
        self.gm.recompile()
        for m in self.gm.modules():           # what is left to aten runs in fp16, like the reference's `model.half()`;
            if m is not self.gm and not isinstance(m, (GapModule, LinearGemm)):      # buffers made here keep their types
                for name, t in list(m.named_parameters(recurse=False)) + list(m.named_buffers(recurse=False)):
                    if t.is_floating_point():
                        t.data = t.data.half()
        self.gm.fvm_stats = dict(self.stats)
        return self.gm


class GraphNet(nn.Module):
    """Runs a rewritten graph: fp32 / fp16 NCHW image batch in, fp32 out."""

    def __init__(self, gm: fx.GraphModule):
        super().__init__()
        self.gm = gm
        self.raw_image = gm.fvm_stats["stem_pad"] > 0

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise ops.FvmError("the b200 tier runs on a CUDA device only (no CPU path)")
        if not self.raw_image:
            x = x.to(torch.float16).contiguous(memory_format=torch.channels_last)
        y = self.gm(x)
        return y.float() if isinstance(y, torch.Tensor) else y


def fuse_graph(model: nn.Module) -> GraphNet:
    """model (fp32, eval) -> GraphNet on the library's ops; `.gm.fvm_stats` counts what each pattern replaced."""
    return GraphNet(Rewriter(model).run())
