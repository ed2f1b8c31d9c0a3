"""`torch.ops` registration of the hot-path operators under the reference's namespaces and schemas.

The reference's fx passes insert `torch.ops.clf.*`, `torch.ops.clfr3.*`, `torch.ops.clfmb.*` and `torch.ops.segx.*` calls whose schemas are
defined by the `TORCH_LIBRARY` blocks of its CUDA extensions (classification/fast/csrc/fused_conv.cu:622-631,
classification/fast/csrc/r3.cu:796-808, mbconv.cu:1243-1257, segmentation/fast/csrc/segx_conv.cu:619-629,
segx_ops.cu:294-322).
`register()` defines the same schema strings with `torch.library` and binds their CUDA implementations to the C-ABI
calls of libfvm_b200.so (through `ops.py`), plus Meta implementations (output shapes only) so that the ops trace under
fake tensors. Only the CUDA key is bound, as in the reference: a CPU tensor reaches no kernel and raises.

If the reference's own extension already defined a schema in this process, registration of that namespace is refused
(two CUDA kernels cannot sit behind one op); set FVM_B200_OPS_PREFIX (e.g. "b200_") to register under
`b200_clf` / `b200_clfr3` / `b200_segx` instead.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from . import ops

PREFIX = os.environ.get("FVM_B200_OPS_PREFIX", "")

# schema strings exactly as in the reference's m.def lines
SCHEMAS = {
    "clf": [
        "input_nhwc8(Tensor x) -> Tensor",
        "conv_fused_into(Tensor x, Tensor w, Tensor? bias, Tensor? res, int[] padding, int[] stride, int act, Tensor(a!) out) -> ()",
        "affine_act(Tensor x, Tensor scale, Tensor shift, int act) -> Tensor",
        "avgpool(Tensor x, int[] k, int[] stride, int[] pad, bool count_include_pad=True) -> Tensor",
        "dwconv(Tensor x, Tensor w_rsc, Tensor? bias, int[] stride, int[] padding, int act) -> Tensor",
        "maxpool(Tensor x, int[] k, int[] stride, int[] pad, bool ceil=False) -> Tensor",
        "conv_fused(Tensor x, Tensor w, Tensor? bias, Tensor? res, int[] padding, int[] stride, int act, int cfg=-1) -> Tensor",
    ],
    "clfr3": [
        "pw(Tensor x, Tensor w, Tensor? bias, Tensor? res, int act, int force=0) -> Tensor",
        "pw_into(Tensor x, Tensor w, Tensor? bias, Tensor? res, int act, Tensor(a!) out, int force=0) -> ()",
        "conv_tc(Tensor x, Tensor w, Tensor? bias, int[] stride, int[] pad, int act, int cfg=-1) -> Tensor",
        "conv_tc_into(Tensor x, Tensor w, Tensor? bias, int[] stride, int[] pad, int act, Tensor(a!) out) -> ()",
        "dwconv2(Tensor x, Tensor w_rsc, Tensor? bias, int[] stride, int[] padding, int act) -> Tensor",
        "se_scale(Tensor x, Tensor s) -> Tensor",
        "stem_pool(Tensor x, Tensor w_t, Tensor? bias, int[] stride, int[] pad, int act, int pk, int ps, int pp, bool ceil) -> Tensor",
        "gconv2(Tensor x, Tensor w, Tensor? bias, int[] stride, int[] pad, int groups, int act, int cfg=-1) -> Tensor",
        "gconv2_pool(Tensor x, Tensor w, Tensor? bias, int[] stride, int[] pad, int groups, int act) -> (Tensor, Tensor)",
    ],
    "clfmb": [
        "stem_direct(Tensor x, Tensor w_t, Tensor? bias, int[] stride, int[] pad, int act) -> Tensor",
        "dwmult(Tensor x, Tensor w_rsk, Tensor? bias, int[] stride, int[] pad, int act) -> Tensor",
    ],
    "segx": [
        "input_nhwc8(Tensor x) -> Tensor",
        "conv_fused_into(Tensor x, Tensor w, Tensor? bias, Tensor? res, int[] padding, int[] stride, int act, Tensor(a!) out) -> ()",
        "affine_act(Tensor x, Tensor scale, Tensor shift, int act) -> Tensor",
        "avgpool(Tensor x, int[] k, int[] stride, int[] pad, bool count_include_pad=True) -> Tensor",
        "dwconv8(Tensor x, Tensor w_rsc, Tensor? bias, int[] stride, int[] padding, int act) -> Tensor",
        "maxpool(Tensor x, int[] k, int[] stride, int[] pad, bool ceil=False) -> Tensor",
        "conv_fused_d(Tensor x, Tensor w, Tensor? bias, Tensor? res, int[] padding, int[] stride, int[] dilation, int act) -> Tensor",
        "conv_fused(Tensor x, Tensor w, Tensor? bias, Tensor? res, int[] padding, int[] stride, int act, int cfg=-1) -> Tensor",
        "bias_act_(Tensor(a!) y, Tensor? bias, Tensor? res, bool relu) -> Tensor(a!)",
        "dwconv(Tensor x, Tensor wt, Tensor? bias, int kh, int kw, int[] stride, int[] padding, int[] dilation, int act) -> Tensor",
        "upsample_bilinear(Tensor x, int H, int W, float? sf_h, float? sf_w, bool align) -> Tensor",
        "upsample_like(Tensor x, Tensor ref, bool align) -> Tensor",
        "upsample_bilinear_t(Tensor x, Tensor size, bool align) -> Tensor",
        "up_argmax(Tensor s, int H, int W, bool align) -> Tensor",
        "upsample_add(Tensor base, Tensor z, float sf, bool relu) -> Tensor",
        "upsample_add_(Tensor(a!) base, Tensor z, float sf, bool relu) -> Tensor(a!)",
    ],
}


def _conv_out(x, w, padding, stride, dilation=(1, 1)):
    N, _, H, W = x.shape
    K, _, R, S = w.shape
    P = (H + 2 * padding[0] - dilation[0] * (R - 1) - 1) // stride[0] + 1
    Q = (W + 2 * padding[1] - dilation[1] * (S - 1) - 1) // stride[1] + 1
    return N, K, P, Q


def _empty_cl(x, shape):
    return torch.empty(shape, dtype=torch.float16, device=x.device).to(memory_format=torch.channels_last)


def _cuda_impls():
    """name -> (CUDA implementation, Meta implementation); shared by the namespaces that define the name."""
    def conv_fused(x, w, bias, res, padding, stride, act, cfg=-1):
        return ops.conv_fused(x, w, bias, res, padding, stride, act, cfg)

    def conv_fused_meta(x, w, bias, res, padding, stride, act, cfg=-1):
        return _empty_cl(x, _conv_out(x, w, padding, stride))

    def conv_fused_d(x, w, bias, res, padding, stride, dilation, act):
        return ops.conv_fused_d(x, w, bias, res, padding, stride, dilation, act)

    def conv_fused_d_meta(x, w, bias, res, padding, stride, dilation, act):
        return _empty_cl(x, _conv_out(x, w, padding, stride, dilation))

    def conv_fused_into(x, w, bias, res, padding, stride, act, out):
        ops.conv_fused_into(x, w, bias, res, padding, stride, act, out)

    def nothing(*a, **k):
        return None

    def pw_meta(x, w, bias, res, act, force=0):
        return _empty_cl(x, _conv_out(x, w, (0, 0), (1, 1)))

    def conv_tc_meta(x, w, bias, stride, pad, act, cfg=-1):
        return _empty_cl(x, _conv_out(x, w, pad, stride))

    def dw_meta(x, w_rsc, bias, stride, padding, act):
        N, C, H, W = x.shape
        R, S = w_rsc.shape[0], w_rsc.shape[1]
        return _empty_cl(x, (N, C, (H + 2 * padding[0] - R) // stride[0] + 1, (W + 2 * padding[1] - S) // stride[1] + 1))

    def segx_dw_meta(x, wt, bias, kh, kw, stride, padding, dilation, act):
        N, C, H, W = x.shape
        return _empty_cl(x, (N, C, (H + 2 * padding[0] - dilation[0] * (kh - 1) - 1) // stride[0] + 1,
                             (W + 2 * padding[1] - dilation[1] * (kw - 1) - 1) // stride[1] + 1))

    def maxpool_meta(x, k, stride, pad, ceil=False):
        N, C, H, W = x.shape
        return _empty_cl(x, (N, C, ops._pool_out(H, k[0], stride[0], pad[0], ceil), ops._pool_out(W, k[-1], stride[-1], pad[-1], ceil)))

    def avgpool_meta(x, k, stride, pad, count_include_pad=True):
        return maxpool_meta(x, k, stride, pad, False)

    def same_meta(x, *a, **k):
        return torch.empty_like(x)

    def input_meta(x):
        N, _, H, W = x.shape
        return _empty_cl(x, (N, 8, H, W))

    def up_meta(x, H, W, sf_h, sf_w, align):
        return _empty_cl(x, (x.shape[0], x.shape[1], H, W))

    def stem_meta(x, w_t, bias, stride, pad, act):
        N, _, H, W = x.shape
        R, S, _, K = w_t.shape
        return _empty_cl(x, (N, K, (H + 2 * pad[0] - R) // stride[0] + 1, (W + 2 * pad[1] - S) // stride[1] + 1))

    def stem_pool_meta(x, w_t, bias, stride, pad, act, pk, ps, pp, ceil):
        y = stem_meta(x, w_t, bias, stride, pad, act)
        return _empty_cl(x, (y.shape[0], y.shape[1], ops._pool_out(y.shape[2], pk, ps, pp, ceil), ops._pool_out(y.shape[3], pk, ps, pp, ceil)))

    def gconv2_meta(x, w, bias, stride, pad, groups, act, cfg=-1):
        return _empty_cl(x, _conv_out(x, w, pad, stride))

    def gconv2_pool_meta(x, w, bias, stride, pad, groups, act):
        y = gconv2_meta(x, w, bias, stride, pad, groups, act)
        return y, _empty_cl(x, (y.shape[0], y.shape[1], 1, 1))

    def dwmult_meta(x, w_rsk, bias, stride, pad, act):
        N, _, H, W = x.shape
        R, S, K = w_rsk.shape
        return _empty_cl(x, (N, K, (H + 2 * pad[0] - R) // stride[0] + 1, (W + 2 * pad[1] - S) // stride[1] + 1))

    def up_argmax(s, H, W, align):
        # the reference passes the scores as an NHWC-shaped tensor [B, h, w, C] (segx_ops.cu:172-175)
        return ops.up_argmax(s.permute(0, 3, 1, 2), H, W, align)

    def up_argmax_meta(s, H, W, align):
        return torch.empty((s.shape[0], H, W), dtype=torch.int32, device=s.device)

    return {
        "conv_fused": (conv_fused, conv_fused_meta),
        "conv_fused_d": (conv_fused_d, conv_fused_d_meta),
        "conv_fused_into": (conv_fused_into, nothing),
        "input_nhwc8": (ops.input_nhwc8, input_meta),
        "affine_act": (ops.affine_act, same_meta),
        "avgpool": (lambda x, k, stride, pad, count_include_pad=True: ops.avgpool(x, k, stride, pad, count_include_pad),
                    avgpool_meta),
        "maxpool": (lambda x, k, stride, pad, ceil=False: ops.maxpool(x, k, stride, pad, ceil), maxpool_meta),
        "dwconv": (lambda x, w_rsc, bias, stride, padding, act: ops.dwconv(x, w_rsc, bias, stride, padding, act), dw_meta),
        "dwconv2": (lambda x, w_rsc, bias, stride, padding, act: ops.dwconv2(x, w_rsc, bias, stride, padding, act), dw_meta),
        "dwconv8": (lambda x, w_rsc, bias, stride, padding, act: ops.dwconv8(x, w_rsc, bias, stride, padding, act), dw_meta),
        "pw": (lambda x, w, bias, res, act, force=0: ops.pw(x, w, bias, res, act, force), pw_meta),
        "pw_into": (lambda x, w, bias, res, act, out, force=0: ops.pw_into(x, w, bias, res, act, out, force), nothing),
        "conv_tc": (lambda x, w, bias, stride, pad, act, cfg=-1: ops.conv_tc(x, w, bias, stride, pad, act, cfg), conv_tc_meta),
        "conv_tc_into": (lambda x, w, bias, stride, pad, act, out: ops.conv_tc_into(x, w, bias, stride, pad, act, out), nothing),
        "gconv2": (lambda x, w, bias, stride, pad, groups, act, cfg=-1: ops.gconv2(x, w, bias, stride, pad, groups, act, cfg),
                   gconv2_meta),
        "gconv2_pool": (lambda x, w, bias, stride, pad, groups, act: ops.gconv2_pool(x, w, bias, stride, pad, groups, act),
                        gconv2_pool_meta),
        "dwmult": (lambda x, w_rsk, bias, stride, pad, act: ops.dwmult(x, w_rsk, bias, stride, pad, act), dwmult_meta),
        "se_scale": (ops.se_scale, same_meta),
        "stem_direct": (ops.stem_direct, stem_meta),
        "stem_pool": (ops.stem_pool, stem_pool_meta),
        "bias_act_": (lambda y, bias, res, relu: ops.bias_act_(y, bias, res, relu), lambda y, bias, res, relu: y),
        "segx.dwconv": (ops.segx_dwconv, segx_dw_meta),
        "upsample_bilinear": (lambda x, H, W, sf_h, sf_w, align: ops.upsample_bilinear(x, H, W, sf_h, sf_w, align), up_meta),
        "upsample_like": (ops.upsample_like, lambda x, ref, align: _empty_cl(x, (x.shape[0], x.shape[1], ref.shape[2], ref.shape[3]))),
        "upsample_bilinear_t": (ops.upsample_bilinear_t, None),     # data-dependent output size: no Meta kernel
        "up_argmax": (up_argmax, up_argmax_meta),
        "upsample_add": (ops.upsample_add, lambda base, z, sf, relu: torch.empty_like(base)),
        "upsample_add_": (ops.upsample_add_, lambda base, z, sf, relu: base),
    }


_LIBS: List[torch.library.Library] = []
_REGISTERED = {}


def _defined(ns: str, name: str) -> bool:
    try:
        return hasattr(getattr(torch.ops, ns), name)
    except (AttributeError, RuntimeError):
        return False


def register(prefix: Optional[str] = None) -> dict:
    """Defines the schemas and binds the CUDA (and Meta) kernels; idempotent. Returns {namespace: [op names]}.
    Works without a GPU (the ops then exist but any call raises in the operator layer)."""
    pre = PREFIX if prefix is None else prefix
    if pre in _REGISTERED:
        return _REGISTERED[pre]
    impls = _cuda_impls()
    done = {}
    for ns, defs in SCHEMAS.items():
        full = pre + ns
        names = [d.split("(", 1)[0] for d in defs]
        clash = [n for n in names if _defined(full, n)]
        if clash:
            raise RuntimeError(f"torch.ops.{full}.{clash[0]} is already defined in this process (the reference's extension "
                               f"is loaded?); call register(prefix='b200_') or set FVM_B200_OPS_PREFIX")
        lib = torch.library.Library(full, "FRAGMENT")
        for schema, name in zip(defs, names):
            lib.define(schema)
            cuda_fn, meta_fn = impls.get(f"{ns}.{name}") or impls[name]
            lib.impl(name, cuda_fn, "CUDA")
            if meta_fn is not None:
                lib.impl(name, meta_fn, "Meta")
        _LIBS.append(lib)      # the registrations live as long as the Library objects
        done[full] = names
    _REGISTERED[pre] = done
    return done
