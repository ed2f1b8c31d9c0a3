"""Per-op CPU restatements: fp32 arithmetic on fp16-rounded operands, one rounding to fp16 at each op output.

TEST INFRASTRUCTURE ONLY. Tensors are NCHW-shaped torch CPU tensors (values are fp16-representable fp32, or fp16);
every function returns fp16. Each function cites the reference lines whose arithmetic it follows.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def act_ref(v: torch.Tensor, act: int) -> torch.Tensor:
    """act_f, classification/fast/csrc/fused_conv.cu:33-43 (fp32)."""
    if act == 0:
        return v
    if act == 1:
        return v.clamp_min(0)
    if act == 2:
        return v.clamp(0, 6)
    if act == 3:
        return v / (1 + torch.exp(-v))
    if act == 4:
        return v * (v + 3).clamp(0, 6) * (1.0 / 6.0)
    if act == 5:
        return 0.5 * v * (1 + torch.erf(v * 0.70710678118654752))
    if act == 6:
        return 0.5 * v * (1 + torch.tanh(0.7978845608028654 * (v + 0.044715 * v * v * v)))
    raise ValueError(act)


def gconv2_ref(x, w, bias=None, stride=(1, 1), padding=(0, 0), groups=1, act=0):
    """Grouped convolution + bias + activation -- clfr3::gconv2 (classification/fast/csrc/r3.cu:49-299; w [K, C/groups, R, S]).
    The reference kernel accumulates in fp16, its portable tier (aten) in fp32 as here; one rounding to fp16 at the end."""
    v = F.conv2d(x.float(), w.float(), None, stride, padding, 1, groups)
    if bias is not None:
        v = v + bias.float().view(1, -1, 1, 1)
    return act_ref(v, act).half()


def conv_fused_ref(x, w, bias=None, res=None, padding=(0, 0), stride=(1, 1), act=0, dilation=(1, 1), scale=None):
    """y = half(act(conv(x,w) + bias + res)) -- epilogue order of Visitor::visit, fused_conv.cu:81-99 (fp32 epilogue,
    single rounding); accumulation in fp32 (the reference kernel accumulates in fp16, its portable tier in fp32).
    `scale` (fp32 per output channel) multiplies (conv + bias) before the residual: an un-folded LayerScale."""
    v = F.conv2d(x.float(), w.float(), None, stride, padding, dilation)
    if bias is not None:
        v = v + bias.float().view(1, -1, 1, 1)
    if scale is not None:
        v = v * scale.float().view(1, -1, 1, 1)
    if res is not None:
        v = v + res.float()
    return act_ref(v, act).half()


def _pair(v):
    return (v, v) if isinstance(v, int) else (int(v[0]), int(v[1]))


def dwconv2_ref(x, w_rsc, bias, stride, padding, act):
    """dwconv2_k MODE 2 (the reference's default for 3x3 / 5x5 / 7x7, classification/fast/csrc/r3.cu:354-415):
    af = float(bias); per kernel row: acc = 0 in fp16, acc = fma_fp16(x, w, acc) over the row's taps in order, then
    af += float(acc); v = half(af); relu / relu6 on the fp16 value, other activations in fp32 on float(v), rounded again.
    The fp16 FMA is emulated as half(float(x) * float(w) + float(acc)): the product is exact in fp32."""
    sh, sw = _pair(stride)
    ph, pw = _pair(padding)
    N, C, H, W = x.shape
    R, S, _ = w_rsc.shape
    P = (H + 2 * ph - R) // sh + 1
    Q = (W + 2 * pw - S) // sw + 1
    xp = F.pad(x.float(), (pw, pw, ph, ph))        # out-of-image taps: x = 0, fma(0, w, acc) = acc (the kernel skips them)
    wf = w_rsc.float()
    af = torch.zeros((N, C, P, Q)) if bias is None else bias.float().view(1, C, 1, 1).expand(N, C, P, Q).clone()
    for r in range(R):
        acc = torch.zeros((N, C, P, Q))
        for s in range(S):
            xs = xp[:, :, r:r + (P - 1) * sh + 1:sh, s:s + (Q - 1) * sw + 1:sw]
            acc = (xs * wf[r, s].view(1, C, 1, 1) + acc).half().float()
        af = af + acc
    v = af.half()
    if act == 0:
        return v
    if act in (1, 2):
        return act_ref(v.float(), act).half()
    return act_ref(v.float(), act).half()


def dwconv_ref(x, w_rsc, bias=None, stride=(1, 1), padding=(0, 0), act=0, dilation=(1, 1)):
    """Square 3/5/7-tap kernels without dilation follow dwconv2 (see dwconv2_ref), which is what the reference runs for
    them (r3.cu:443-447); every other shape follows dwconv_tw, fused_conv.cu:428-475: acc = float(bias);
    acc += float(x)*float(w) over in-image taps; half(act(acc))."""
    R, S = w_rsc.shape[0], w_rsc.shape[1]
    sh, sw = _pair(stride)
    if R == S and R in (3, 5, 7) and _pair(dilation) == (1, 1) and sh == sw and sh in (1, 2) \
            and (x.shape[3] + 2 * _pair(padding)[1] - S) // sw + 1 >= 4:
        return dwconv2_ref(x, w_rsc, bias, stride, padding, act)
    C = x.shape[1]
    w = w_rsc.float().permute(2, 0, 1).unsqueeze(1)     # [C,1,R,S]
    v = F.conv2d(x.float(), w, None if bias is None else bias.float(), stride, padding, dilation, groups=C)
    return act_ref(v, act).half()


def pool_out_ref(L, k, s, p, ceil):
    """Output-size rule, fused_conv.cu:363-367."""
    if not ceil:
        return (L + 2 * p - k) // s + 1
    o = (L + 2 * p - k + s - 1) // s + 1
    if (o - 1) * s >= L + p:
        o -= 1
    return o


def maxpool_ref(x, k, stride, pad, ceil=False):
    """maxpool_nhwc8, fused_conv.cu:338-356: -inf padding, max over in-image taps (exact in fp16)."""
    return F.max_pool2d(x.float(), k, stride, pad, ceil_mode=ceil).half()


def avgpool_ref(x, k, stride, pad, ceil=False, count_include_pad=True):
    """avgpool_nhwc8, fused_conv.cu:556-582: fp32 sum, PyTorch divisor rule."""
    return F.avg_pool2d(x.float(), k, stride, pad, ceil_mode=ceil, count_include_pad=count_include_pad).half()


def global_avgpool_ref(x):
    """AdaptiveAvgPool2d(1) on fp16 with fp32 accumulation, fp16 result (the aten module the reference leaves in the
    graph; fused alternative r3.cu:283-286 computes half(sum * (1/PQ)))."""
    return x.float().mean(dim=(2, 3), keepdim=True).half()


def se_gate_ref(g, w1, b1, w2, b2, act=3):
    """Two conv_fused calls on [N,C,1,1]: h = half(act(W1 g + b1)); s = half(W2 h + b2)."""
    h = conv_fused_ref(g, w1.view(w1.shape[0], -1, 1, 1), b1, act=act)
    return conv_fused_ref(h, w2.view(w2.shape[0], -1, 1, 1), b2, act=0)


def se_scale_ref(x, s):
    """se_scale_k, classification/fast/csrc/r3.cu:312-315: sigmoid in fp32 -> fp16, fp16 multiply."""
    sg = (1.0 / (1.0 + torch.exp(-s.float()))).half()
    return (x.half().float() * sg.float()).half()       # one fp16 multiply = exact product rounded once


def layernorm_cl_ref(x, weight, bias, eps=1e-6):
    """LayerNorm over channels of an NCHW-shaped tensor: two-pass fp32 statistics, fp32 affine, one rounding
    (ln_row, segmentation/fast/csrc/seg_kernels.cu:197-210; torch nn.LayerNorm at convnext.py:55)."""
    v = x.float()
    mean = v.mean(dim=1, keepdim=True)
    var = ((v - mean) ** 2).mean(dim=1, keepdim=True)
    y = (v - mean) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.float().view(1, -1, 1, 1)
    if bias is not None:
        y = y + bias.float().view(1, -1, 1, 1)
    return y.half()


def input_nhwc8_ref(x):
    """input_nhwc8_k, fused_conv.cu:597-606: half(x) with channels zero-padded to 8."""
    N, C, H, W = x.shape
    y = torch.zeros((N, 8, H, W), dtype=torch.float16)
    y[:, :C] = x.half()
    return y


def bias_act_ref(y, bias=None, res=None, relu=False):
    """bias_act_h, segmentation/fast/csrc/seg_kernels.cu:107-119."""
    v = y.float()
    if bias is not None:
        v = v + bias.float().view(1, -1, 1, 1)
    if res is not None:
        v = v + res.float()
    if relu:
        v = v.clamp_min(0)
    return v.half()


def affine_act_ref(x, scale, shift, act):
    """affine_act_k, fused_conv.cu:310-321."""
    return act_ref(x.float() * scale.float().view(1, -1, 1, 1) + shift.float().view(1, -1, 1, 1), act).half()


def add_act_ref(a, b, act=0):
    return act_ref(a.float() + b.float(), act).half()


def _src_index(out, inp, align, sf=None):
    """PyTorch bilinear source index math (bilin_k, segmentation/fast/csrc/segx_ops.cu:74-79, 142-152), in fp32."""
    i = torch.arange(out, dtype=torch.float32)
    if align:
        scale = torch.tensor((inp - 1) / (out - 1) if out > 1 else 0.0, dtype=torch.float32)
        f = i * scale
    else:
        scale = torch.tensor((1.0 / sf) if sf else inp / out, dtype=torch.float32)
        f = ((i + 0.5) * scale - 0.5).clamp_min(0)
    i0 = f.to(torch.int64).clamp_max(inp - 1)
    i1 = i0 + (i0 < inp - 1).to(torch.int64)
    l = f - i0.float()
    return i0, i1, l


def _bilinear_f32(x, H, W, align, sf_h=None, sf_w=None):
    v = x.float()
    y0, y1, ly = _src_index(H, x.shape[2], align, sf_h)
    x0, x1, lx = _src_index(W, x.shape[3], align, sf_w)
    ly = ly.view(1, 1, H, 1)
    lx = lx.view(1, 1, 1, W)
    hy, hx = 1 - ly, 1 - lx
    a = v[:, :, y0][:, :, :, x0]
    b = v[:, :, y0][:, :, :, x1]
    c = v[:, :, y1][:, :, :, x0]
    d = v[:, :, y1][:, :, :, x1]
    return hy * (hx * a + lx * b) + ly * (hx * c + lx * d)


def bilinear_ref(x, H, W, align=False, sf_h=None, sf_w=None, base=None, relu=False):
    """bilin_k, segx_ops.cu:62-111: fp32 lerp; with `base` the interpolated value is rounded to fp16 first, then added
    in fp32, then ReLU (:102-105)."""
    v = _bilinear_f32(x, H, W, align, sf_h, sf_w)
    if base is not None:
        v = v.half().float() + base.float()
        if relu:
            v = v.clamp_min(0)
    return v.half()


def up_argmax_ref(s, H, W, align=False, num_classes=None):
    """up_argmax_h, segmentation/fast/csrc/seg_kernels.cu:11-42: fp32 lerp per channel, first maximum wins, int32."""
    C = s.shape[1] if num_classes is None else num_classes
    v = _bilinear_f32(s[:, :C], H, W, align)
    return v.argmax(dim=1).to(torch.int32)      # torch.argmax returns the first maximal index
