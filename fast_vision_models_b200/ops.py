"""Operator layer: torch tensors in, C-ABI calls out.

Each function mirrors one op schema of the reference's `TORCH_LIBRARY` blocks (same name, argument order and meaning;
classification/fast/csrc/fused_conv.cu:622-631, r3.cu:796-808, segmentation/fast/csrc/segx_conv.cu:619-629,
segx_ops.cu:294-322) and forwards raw device pointers, sizes and the current CUDA stream to libfvm_b200.so.
Activations are NCHW-shaped fp16 tensors in channels-last memory format (NHWC in memory), possibly a channel slice
of a wider channels-last buffer. There is no CPU or aten fallback: a tensor that is not on a CUDA device, or a
library that is missing, raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from . import _lib

ACT_NONE, ACT_RELU, ACT_RELU6, ACT_SILU, ACT_HARDSWISH, ACT_GELU_ERF, ACT_GELU_TANH = range(7)

_initialised_devices = set()


class FvmError(RuntimeError):
    pass


_STATUS_TEXT = {1: "bad argument or unsupported shape", 2: "set-up failed (not an sm_100 device, or driver entry point missing)",
                3: "kernel launch error", 4: "tensor-map encode error"}


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise FvmError(f"fvm_b200.{what}: status {rc} ({_STATUS_TEXT.get(rc, 'unknown')})")


def lib() -> ctypes.CDLL:
    return _lib.load()


def init(device: Optional[torch.device] = None) -> None:
    """Per-device set-up; must run before the first launch on a device and before any CUDA-graph capture."""
    if not torch.cuda.is_available():
        raise FvmError("fvm_b200 needs a CUDA device (sm_100a); there is no CPU path")
    cur = torch.cuda.current_device()
    dev = torch.device("cuda", cur) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else cur
    if idx != cur:
        # the library launches on the current device's stream: a tensor of another device would be a wild pointer there
        raise FvmError(f"fvm_b200: tensor on cuda:{idx} but the current device is cuda:{cur}; "
                       f"wrap the call in torch.cuda.device({idx})")
    if idx in _initialised_devices:
        return
    with torch.cuda.device(idx):
        _check(lib().fvm_init(), "init")
    _initialised_devices.add(idx)


def last_status() -> int:
    """Asynchronous status word of the current device (0 = no fault); synchronises first."""
    torch.cuda.synchronize()
    code = ctypes.c_int(0)
    _check(lib().fvm_last_status(ctypes.byref(code)), "last_status")
    return code.value


def poll_status() -> int:
    """The status word as it stands now, without synchronising (reads and clears it): non-zero means a kernel that has
    already finished reported a fault. Cheap enough to call before every graph replay."""
    code = ctypes.c_int(0)
    _check(lib().fvm_last_status(ctypes.byref(code)), "last_status")
    return code.value


def selftest_wait_expiry(limit_us: int = 1000) -> None:
    """Launches the library's fault-path self-test: a kernel whose bounded wait runs out after `limit_us` microseconds
    and reports 0x1ff through the status word (read it with `last_status()`)."""
    init()
    _check(lib().fvm_selftest_wait_expiry(int(limit_us), _stream()), "selftest_wait_expiry")


def launches() -> int:
    """Number of kernels this library has launched since it was loaded."""
    return int(lib().fvm_query(3))


def query(what: int) -> int:
    """fvm_query: 0 version, 1 SM count, 2 max dynamic shared memory, 3 launches, 4 CTA pairs resident at once."""
    return int(lib().fvm_query(int(what)))


def _stream() -> int:
    # every launch of this module asks for the stream first: convolutions recorded for a chain launch go out before
    # anything else that could read their outputs
    if _chain is not None and _chain.layers:
        _chain.flush()
    return torch.cuda.current_stream().cuda_stream


# ------------------------------------------------------------------------------------------------ layer chains
CHAIN_MAX_LAYERS = 48
CHAINS = os.environ.get("FVM_B200_CHAIN", "1") != "0"


class _Chain:
    """Convolutions recorded between chain_begin() and chain_end(): launched together by fvm_conv_chain_f16 (one kernel
    whose tiles follow the layers' data dependencies), or one by one where the library cannot express the run."""

    def __init__(self):
        self.layers = []      # (argument list of fvm_conv2d_f16, tile code, tensors kept alive)

    def add(self, args, tile_n, keep) -> None:
        self.layers.append((args, int(tile_n), keep))
        if len(self.layers) == CHAIN_MAX_LAYERS:
            self.flush()

    def flush(self) -> None:
        layers, self.layers = self.layers, []
        if not layers:
            return
        L = lib()
        stream = torch.cuda.current_stream().cuda_stream
        if len(layers) > 1:
            arr = (_lib.ChainLayer * len(layers))()
            for c, (a, tile_n, _keep) in zip(arr, layers):
                (c.x, c.w, c.bias, c.res, c.scale, c.y, c.N, c.H, c.W, c.C, c.K, c.R, c.S, c.ph, c.pw, c.sh, c.sw, c.dh,
                 c.dw, c.ldx, c.ldy, c.ldr, c.act) = a
                c.tile_n = (tile_n & 0xffff) if (tile_n >> 30) & 1 else 0     # a width that was chosen for CTA pairs
            rc = L.fvm_conv_chain_f16(arr, len(layers), stream)
            if rc == 0:
                return
            if rc != 1:
                _check(rc, "conv_chain_f16")
        for a, tile_n, _keep in layers:        # not expressible as a chain (or a single layer): stream order
            rc = L.fvm_conv2d_f16_tile(*a, tile_n, stream) if tile_n else L.fvm_conv2d_f16(*a, stream)
            _check(rc, "conv2d_f16")


_chain: Optional[_Chain] = None


def chain_begin() -> bool:
    """Starts recording: conv_fused_into calls with at least 24 input channels are collected instead of launched, until
    chain_end() (or any other launch of this module, or 48 layers) sends them out as one chain launch. Outputs must not
    be read by anything but this module before that. Returns False (and records nothing) when chains are switched off
    (FVM_B200_CHAIN=0), the device cannot run CTA pairs, or a recording is already open."""
    global _chain
    if not CHAINS or _chain is not None or query(4) <= 0:
        return False
    _chain = _Chain()
    return True


def chain_end() -> None:
    global _chain
    c, _chain = _chain, None
    if c is not None:
        c.flush()


def chain_active() -> bool:
    return _chain is not None


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _require_cuda_half(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise FvmError(f"{name}: tensor is not on a CUDA device; fvm_b200 has no CPU path")
    if t.dtype != torch.float16:
        raise FvmError(f"{name}: expected fp16, got {t.dtype}")


def nhwc_view(x: torch.Tensor, name: str = "x"):
    """Returns (tensor, N, C, H, W, ld): `tensor` is NHWC in memory with pixel stride `ld` (a channels-last tensor or a
    channel slice of one); anything else is made channels-last contiguous first (reference: fused_conv.cu:237-244)."""
    _require_cuda_half(x, name)
    if x.dim() != 4:
        raise FvmError(f"{name}: expected a 4-D NCHW-shaped tensor")
    N, C, H, W = x.shape
    sN, sC, sH, sW = x.stride()
    # pixel (n,h,w) must sit at ((n*H + h)*W + w) * ld; ld comes from the innermost dimension that has extent > 1
    if W > 1:
        ld = sW
    elif H > 1:
        ld = sH
    elif N > 1:
        ld = sN
    else:
        ld = C
    ok = (C == 1 or sC == 1) and ld % 8 == 0 and ld >= C and x.data_ptr() % 16 == 0 \
        and (H == 1 or sH == W * ld) and (N == 1 or sN == H * W * ld)
    if not ok:
        x = x.contiguous(memory_format=torch.channels_last)
        if x.data_ptr() % 16 != 0 or C % 8 != 0:
            raise FvmError(f"{name}: channels must be a multiple of 8 and the storage 16-byte aligned")
        ld = C
    return x, N, C, H, W, ld


def empty_nhwc(N: int, C: int, H: int, W: int, device) -> torch.Tensor:
    return torch.empty((N, C, H, W), dtype=torch.float16, device=device, memory_format=torch.channels_last)


def _pair(v) -> tuple:
    if isinstance(v, int):
        return (v, v)
    v = tuple(int(a) for a in v)
    return (v[0], v[0]) if len(v) == 1 else (v[0], v[1])


# ------------------------------------------------------------------------------------------------ dense conv / GEMM
def _krsc(w: torch.Tensor) -> torch.Tensor:
    """[K,C,R,S] weight -> KRSC in memory (a channels-last tensor), as the reference requires (fused_conv.cu:245)."""
    _require_cuda_half(w, "w")
    if w.dim() != 4:
        raise FvmError("w: expected [K,C,R,S]")
    return w.contiguous(memory_format=torch.channels_last)


def conv_fused_into(x, w, bias, res, padding, stride, act: int, out: torch.Tensor, dilation=(1, 1),
                    scale: Optional[torch.Tensor] = None, tile_n: int = 0, pad_hi=None) -> None:
    """clf::conv_fused_into / segx::conv_fused_into: y = act((conv(x,w)+bias)*scale + res) written into `out`.
    `pad_hi` = (bottom, right) padding when it differs from `padding` = (top, left)."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    w = _krsc(w)
    K, Cw, R, S = w.shape
    if Cw != C:
        raise FvmError(f"conv_fused: weight has {Cw} input channels, input has {C}")
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    ph_hi, pw_hi = (ph, pw) if pad_hi is None else _pair(pad_hi)
    P = (H + ph + ph_hi - dh * (R - 1) - 1) // sh + 1
    Q = (W + pw + pw_hi - dw * (S - 1) - 1) // sw + 1
    out_v, No, Ko, Po, Qo, ldy = nhwc_view(out, "out")
    if out_v is not out or (No, Ko, Po, Qo) != (N, K, P, Q):
        raise FvmError(f"conv_fused_into: out must be a channels-last [N,K,P,Q]={N, K, P, Q} tensor or channel slice, "
                       f"got {tuple(out.shape)} strides {out.stride()}")
    ldr = 0
    if res is not None:
        res, Nr, Kr, Pr, Qr, ldr = nhwc_view(res, "res")
        if (Nr, Kr, Pr, Qr) != (N, K, P, Q):
            raise FvmError("conv_fused: residual shape does not match the output")
    if bias is not None:
        _require_cuda_half(bias, "bias")
        bias = bias.contiguous()
    if scale is not None:
        if scale.dtype != torch.float32 or not scale.is_cuda:
            raise FvmError("conv_fused: scale must be an fp32 CUDA tensor")
        scale = scale.contiguous()
    args = [x.data_ptr(), w.data_ptr(), _ptr(bias), _ptr(res), _ptr(scale), out.data_ptr(), N, H, W, C, K, R, S, ph, pw,
            sh, sw, dh, dw, ldx, ldy, ldr, int(act)]
    if _chain is not None and pad_hi is None and C >= 24:
        _chain.add(args, tile_n, (x, w, bias, res, scale, out))
        return
    L = lib()
    if pad_hi is not None:
        rc = L.fvm_conv2d_f16_pad(*args, int(tile_n), ph_hi, pw_hi, _stream())
    elif tile_n:
        rc = L.fvm_conv2d_f16_tile(*args, int(tile_n), _stream())
    else:
        rc = L.fvm_conv2d_f16(*args, _stream())
    _check(rc, "conv2d_f16")


def conv_fused(x, w, bias=None, res=None, padding=(0, 0), stride=(1, 1), act: int = 0, cfg: int = -1,
               dilation=(1, 1), scale=None, tile_n: int = 0) -> torch.Tensor:
    """clf::conv_fused(x, w, bias?, res?, padding, stride, act, cfg=-1) -> Tensor (fused_conv.cu:298-302, schema :624).
    `cfg` (the reference's CUTLASS tile index) is accepted and ignored; `tile_n` forces this library's own N tile."""
    N, C, H, W = x.shape
    K, _, R, S = w.shape
    ph, pw = _pair(padding)
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    P = (H + 2 * ph - dh * (R - 1) - 1) // sh + 1
    Q = (W + 2 * pw - dw * (S - 1) - 1) // sw + 1
    out = empty_nhwc(N, K, P, Q, x.device)
    conv_fused_into(x, w, bias, res, padding, stride, act, out, dilation=dilation, scale=scale, tile_n=tile_n)
    return out


def conv_fused_d(x, w, bias, res, padding, stride, dilation, act: int) -> torch.Tensor:
    """segx::conv_fused_d (segmentation/fast/csrc/segx_conv.cu:295-299)."""
    return conv_fused(x, w, bias, res, padding, stride, act, dilation=dilation)


def pw(x, w, bias=None, res=None, act: int = 0, force: int = 0) -> torch.Tensor:
    """clfr3::pw(x, w, bias?, res?, act, force=0) (classification/fast/csrc/r3.cu:758-761, schema :797): 1x1 stride-1
    conv, y = act(x . w^T + bias + res). The reference runs it as a cublasLt GEMM and uses `force` to pick between that
    and its CUTLASS kernel; here it is the tcgen05 kernel either way and `force` is accepted and ignored."""
    return conv_fused(x, w, bias, res, (0, 0), (1, 1), act)


def pw_into(x, w, bias, res, act: int, out: torch.Tensor, force: int = 0) -> None:
    """clfr3::pw_into(x, w, bias?, res?, act, out, force=0) (r3.cu:762-765): pw written into `out`, which may be a
    channel slice of a wider channels-last buffer."""
    conv_fused_into(x, w, bias, res, (0, 0), (1, 1), act, out)


def pw_dual_ok(C1: int, K1: int, K2: int) -> bool:
    """Shapes fvm_conv_dual_f16 takes: (C1, K1) one of (64, 128), (64, 256), (128, 128) -- both weight tensors stay in
    shared memory -- and K2 a multiple of 16 up to 128."""
    return (C1, K1) in ((64, 128), (64, 256), (128, 128)) and 16 <= K2 <= 128 and K2 % 16 == 0


def pw_dual(x, w1, b1, res, act1: int, w2, b2, act2: int):
    """Two 1x1 stride-1 convolutions as one launch: y = act1(x . w1^T + b1 + res), z = act2(y . w2^T + b2); returns (y, z).
    The last convolution of a bottleneck block with the first of the next one (torchvision Bottleneck.conv3 + identity
    + ReLU -> conv1 + ReLU); the reference runs them as two clf::conv_fused launches (fused_conv.cu:231-306). y is
    written once and the second layer reads it from shared memory; same bits as `pw` twice. Raises FvmError for shapes
    outside pw_dual_ok."""
    init(x.device)
    x, N, C1, H, W, ldx = nhwc_view(x, "x")
    w1, w2 = _krsc(w1), _krsc(w2)
    K1, K2 = w1.shape[0], w2.shape[0]
    if tuple(w1.shape[1:]) != (C1, 1, 1) or tuple(w2.shape[1:]) != (K1, 1, 1):
        raise FvmError("pw_dual: expected 1x1 weights [K1,C1,1,1] and [K2,K1,1,1]")
    if not pw_dual_ok(C1, K1, K2):
        raise FvmError(f"pw_dual: unsupported channel counts {C1} -> {K1} -> {K2}")
    ldr = 0
    if res is not None:
        res, Nr, Kr, Hr, Wr, ldr = nhwc_view(res, "res")
        if (Nr, Kr, Hr, Wr) != (N, K1, H, W):
            raise FvmError("pw_dual: residual shape does not match the first layer's output")
    for b, name in ((b1, "b1"), (b2, "b2")):
        if b is not None:
            _require_cuda_half(b, name)
    b1 = None if b1 is None else b1.contiguous()
    b2 = None if b2 is None else b2.contiguous()
    y = empty_nhwc(N, K1, H, W, x.device)
    z = empty_nhwc(N, K2, H, W, x.device)
    rc = lib().fvm_conv_dual_f16(x.data_ptr(), w1.data_ptr(), _ptr(b1), _ptr(res), y.data_ptr(), w2.data_ptr(), _ptr(b2),
                                 z.data_ptr(), N * H * W, C1, K1, K2, ldx, ldr, K1, K2, int(act1), int(act2), _stream())
    _check(rc, "conv_dual_f16")
    return y, z


_PACKED_GROUPED = {}      # (data_ptr, version, shape, groups) -> (packed weights, gsg, gsk, the source tensor kept alive)


def _packed_grouped(w: torch.Tensor, groups: int):
    from . import fold
    key = (w.data_ptr(), w._version, tuple(w.shape), int(groups))
    hit = _PACKED_GROUPED.get(key)
    if hit is None:
        if len(_PACKED_GROUPED) >= 512:
            _PACKED_GROUPED.clear()
        wp, gsg, gsk = fold.pack_grouped(w, groups)
        hit = _PACKED_GROUPED[key] = (wp, gsg, gsk, w)
    return hit[:3]


def gconv2_packed_into(x, w_sg, bias, res, stride, pad, act: int, gsg: int, gsk: int, out: torch.Tensor, dilation=(1, 1)) -> None:
    """Grouped convolution with weights already in the super-group layout of fold.pack_grouped (fvm_gconv2d_f16)."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    w_sg = _krsc(w_sg)
    K, Cw, R, S = w_sg.shape
    if Cw != gsg:
        raise FvmError(f"gconv2: packed weight has {Cw} input channels per run, expected {gsg}")
    ph, pw = _pair(pad)
    sh, sw = _pair(stride)
    dh, dw = _pair(dilation)
    P = (H + 2 * ph - dh * (R - 1) - 1) // sh + 1
    Q = (W + 2 * pw - dw * (S - 1) - 1) // sw + 1
    out_v, No, Ko, Po, Qo, ldy = nhwc_view(out, "out")
    if out_v is not out or (No, Ko, Po, Qo) != (N, K, P, Q):
        raise FvmError(f"gconv2: out must be a channels-last [N,K,P,Q]={N, K, P, Q} tensor or channel slice")
    ldr = 0
    if res is not None:
        res, Nr, Kr, Pr, Qr, ldr = nhwc_view(res, "res")
        if (Nr, Kr, Pr, Qr) != (N, K, P, Q):
            raise FvmError("gconv2: residual shape does not match the output")
    if bias is not None:
        _require_cuda_half(bias, "bias")
        bias = bias.contiguous()
    _check(lib().fvm_gconv2d_f16(x.data_ptr(), w_sg.data_ptr(), _ptr(bias), _ptr(res), out.data_ptr(), N, H, W, C, K, R, S,
                                 ph, pw, sh, sw, dh, dw, ldx, ldy, ldr, int(act), int(gsg), int(gsk), _stream()), "gconv2d_f16")


def gconv2(x, w, bias=None, stride=(1, 1), pad=(0, 0), groups: int = 1, act: int = 0, cfg: int = -1) -> torch.Tensor:
    """clfr3::gconv2(x, w, bias?, stride, pad, groups, act, cfg=-1) -> Tensor (r3.cu:276-279, schema :800): grouped
    convolution, w [K, C/groups, R, S] channels-last. Runs on the dense tcgen05 kernel over block-diagonal runs of groups
    (the packed weights are built once per weight tensor and kept); `cfg` is accepted and ignored."""
    N, C, H, W = x.shape
    K, GW, R, S = w.shape
    if GW * groups != C:
        raise FvmError(f"gconv2: weight has {GW} channels per group, {groups} groups, input has {C} channels")
    w_sg, gsg, gsk = _packed_grouped(w, groups)
    ph, pw = _pair(pad)
    sh, sw = _pair(stride)
    out = empty_nhwc(N, K, (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1, x.device)
    gconv2_packed_into(x, w_sg, bias, None, stride, pad, act, gsg, gsk, out)
    return out


def gconv2_pool(x, w, bias, stride, pad, groups: int, act: int):
    """clfr3::gconv2_pool -> (y, mean [N, K, 1, 1]) (r3.cu:289-299): the grouped convolution and the global average of its
    output (the squeeze of a squeeze-excite block that follows). Two launches here: gconv2, then the pooling kernel."""
    y = gconv2(x, w, bias, stride, pad, groups, act)
    return y, global_avgpool(y)


def dwmult(x, w_rsk, bias=None, stride=(1, 1), pad=(0, 0), act: int = 0) -> torch.Tensor:
    """clfmb::dwmult(x, w_rsk, bias?, stride, pad, act) (mbconv.cu:776-788, schema :1248): depthwise convolution with a
    channel multiplier, w_rsk [R, S, K] with K = m * C (output channel k reads input channel k // m). A grouped
    convolution with groups = C and one input channel per group."""
    R, S, K = w_rsk.shape
    C = x.shape[1]
    if K % C:
        raise FvmError("dwmult: K must be a multiple of C")
    w = w_rsk.permute(2, 0, 1).reshape(K, 1, R, S)
    key_src = w_rsk
    hit = _PACKED_GROUPED.get((key_src.data_ptr(), key_src._version, tuple(key_src.shape), -C))
    if hit is None:
        from . import fold
        wp, gsg, gsk = fold.pack_grouped(w, C)
        hit = _PACKED_GROUPED[(key_src.data_ptr(), key_src._version, tuple(key_src.shape), -C)] = (wp, gsg, gsk, key_src)
    w_sg, gsg, gsk = hit[:3]
    N, _, H, W = x.shape
    ph, pw = _pair(pad)
    sh, sw = _pair(stride)
    out = empty_nhwc(N, K, (H + 2 * ph - R) // sh + 1, (W + 2 * pw - S) // sw + 1, x.device)
    gconv2_packed_into(x, w_sg, bias, None, stride, pad, act, gsg, gsk, out)
    return out


def conv_tc(x, w, bias=None, stride=(1, 1), pad=(0, 0), act: int = 0, cfg: int = -1) -> torch.Tensor:
    """clfr3::conv_tc(x, w, bias?, stride, pad, act, cfg=-1) (r3.cu:801): dense KxK conv over few input channels
    (C <= 48, C % 16 == 0 in the reference, which runs it on its grouped-conv kernel). Note the argument order: stride
    before pad. Here every dense conv is the same kernel; 8- and 16-channel inputs take its tap-packed mode."""
    return conv_fused(x, w, bias, None, pad, stride, act)


def conv_tc_into(x, w, bias, stride, pad, act: int, out: torch.Tensor) -> None:
    """clfr3::conv_tc_into(x, w, bias?, stride, pad, act, out) (r3.cu:802)."""
    conv_fused_into(x, w, bias, None, pad, stride, act, out)


def linear(x2d: torch.Tensor, w: torch.Tensor, bias=None, res2d=None, act: int = 0, scale=None) -> torch.Tensor:
    """Row-major GEMM y[M,K] = act((x[M,C] @ w[K,C]^T + bias)*scale + res): the reference's `_lin` view
    (classification/fast/vit.py:56-64) without the permutes."""
    _require_cuda_half(x2d, "x")
    M, C = x2d.shape
    K = w.shape[0]
    x4 = x2d.contiguous().view(1, M, 1, C).permute(0, 3, 1, 2)
    y = torch.empty((M, K), dtype=torch.float16, device=x2d.device)
    y4 = y.view(1, M, 1, K).permute(0, 3, 1, 2)
    r4 = None if res2d is None else res2d.contiguous().view(1, M, 1, K).permute(0, 3, 1, 2)
    conv_fused_into(x4, w.reshape(K, C, 1, 1), bias, r4, (0, 0), (1, 1), act, y4, scale=scale)
    return y


# ------------------------------------------------------------------------------------------------ depthwise
def dwconv(x, w_rsc, bias=None, stride=(1, 1), padding=(0, 0), act: int = 0, dilation=(1, 1),
           pool: bool = False):
    """clf::dwconv(x, w_rsc, bias?, stride, padding, act) (fused_conv.cu:480-502) / clfr3::dwconv2 (r3.cu:423-454) /
    segx::dwconv with dilation (segx_ops.cu:45-57). w_rsc is [R,S,C] contiguous.
    With `pool=True` returns (y, partial): `partial` is fp32 [N, slots, C], per-tile sums of the rounded outputs (the
    fused squeeze of a squeeze-excite block, cf. clfr3::gconv2_pool r3.cu:181-203); `se_gate_pooled` consumes it."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    _require_cuda_half(w_rsc, "w_rsc")
    w_rsc = w_rsc.contiguous()
    R, S, Cw = w_rsc.shape
    if Cw != C:
        raise FvmError("dwconv: weight channel count mismatch")
    sh, sw = _pair(stride)
    ph, pw_ = _pair(padding)
    dh, dw = _pair(dilation)
    P = (H + 2 * ph - dh * (R - 1) - 1) // sh + 1
    Q = (W + 2 * pw_ - dw * (S - 1) - 1) // sw + 1
    y = empty_nhwc(N, C, P, Q, x.device)
    if bias is not None:
        bias = bias.contiguous()
    partial = None
    if pool:
        slots = int(lib().fvm_dwconv_pool_slots(N, H, W, C, R, S, ph, pw_, sh, sw, dh, dw))
        if slots <= 0:
            raise FvmError("dwconv: unsupported geometry")
        partial = torch.empty((N, slots, C), dtype=torch.float32, device=x.device)
    _check(lib().fvm_dwconv_f16(x.data_ptr(), w_rsc.data_ptr(), _ptr(bias), y.data_ptr(), _ptr(partial), N, H, W, C,
                                R, S, ph, pw_, sh, sw, dh, dw, ldx, C, int(act), _stream()), "dwconv_f16")
    return (y, partial) if pool else y


dwconv2 = dwconv      # clfr3::dwconv2(x, w_rsc, bias?, stride, padding, act): same schema (r3.cu:803)
dwconv8 = dwconv      # segx::dwconv8(x, w_rsc, bias?, stride, padding, act) (segmentation/fast/csrc/segx_conv.cu:624)


def segx_dwconv(x, wt, bias, kh: int, kw: int, stride, padding, dilation, act: int) -> torch.Tensor:
    """segx::dwconv(x, wt, bias?, kh, kw, stride, padding, dilation, act) (segmentation/fast/csrc/segx_ops.cu:45-57):
    depthwise conv with any kernel size / stride / padding / dilation; `wt` is fp16 [kh*kw, C] tap-major. In this op
    `act` is 0 = none, 1 = GELU (erf) (segmentation/fast/seg_kernels.cu:151-154), not the clf activation table."""
    if act not in (0, 1):
        raise FvmError("segx::dwconv: act is 0 (none) or 1 (erf GELU)")
    C = x.shape[1]
    if wt.dim() != 2 or tuple(wt.shape) != (int(kh) * int(kw), C):
        raise FvmError(f"segx::dwconv: wt must be [kh*kw, C] = {(int(kh) * int(kw), C)}, got {tuple(wt.shape)}")
    return dwconv(x, wt.contiguous().view(int(kh), int(kw), C), bias, stride, padding, ACT_GELU_ERF if act == 1 else ACT_NONE,
                  dilation=dilation)


# ------------------------------------------------------------------------------------------------ pooling
def _pool_out(L: int, k: int, s: int, p: int, ceil: bool) -> int:
    """Output size rule of the reference (fused_conv.cu:363-367)."""
    if not ceil:
        return (L + 2 * p - k) // s + 1
    o = (L + 2 * p - k + s - 1) // s + 1
    if (o - 1) * s >= L + p:
        o -= 1
    return o


def maxpool(x, k, stride, pad, ceil: bool = False) -> torch.Tensor:
    """clf::maxpool(x, k, stride, pad, ceil=False) (fused_conv.cu:358-374)."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    if ldx != C:
        x = x.contiguous(memory_format=torch.channels_last)
    kh, kw = _pair(k)
    sh, sw = _pair(stride)
    ph, pw_ = _pair(pad)
    P, Q = _pool_out(H, kh, sh, ph, ceil), _pool_out(W, kw, sw, pw_, ceil)
    y = empty_nhwc(N, C, P, Q, x.device)
    _check(lib().fvm_maxpool_f16(x.data_ptr(), y.data_ptr(), N, H, W, C, kh, kw, sh, sw, ph, pw_, P, Q, _stream()),
           "maxpool_f16")
    return y


def avgpool(x, k, stride, pad, count_include_pad: bool = True, *, ceil: bool = False) -> torch.Tensor:
    """clf::avgpool(x, k, stride, pad, count_include_pad=True) (fused_conv.cu:584-594, schema :626): the fifth
    positional argument is count_include_pad, as in the reference, whose op always uses the floor rule for the output
    size; `ceil` (keyword only) is this library's extension for ceil-mode pools."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    if ldx != C:
        x = x.contiguous(memory_format=torch.channels_last)
    kh, kw = _pair(k)
    sh, sw = _pair(stride)
    ph, pw_ = _pair(pad)
    P, Q = _pool_out(H, kh, sh, ph, ceil), _pool_out(W, kw, sw, pw_, ceil)
    y = empty_nhwc(N, C, P, Q, x.device)
    _check(lib().fvm_avgpool_f16(x.data_ptr(), y.data_ptr(), N, H, W, C, kh, kw, sh, sw, ph, pw_, P, Q,
                                 int(bool(count_include_pad)), _stream()), "avgpool_f16")
    return y


def gap_scratch(N: int, HW: int, C: int, device) -> torch.Tensor:
    init(device)
    return torch.empty(int(lib().fvm_gap_scratch_floats(N, HW, C)), dtype=torch.float32, device=device)


def global_avgpool(x, scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """AdaptiveAvgPool2d(1) on NHWC fp16 -> [N,C,1,1] fp16; deterministic two-stage fp32 reduction."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    need = int(lib().fvm_gap_scratch_floats(N, H * W, C))
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=x.device)
    elif scratch.numel() < need or scratch.dtype != torch.float32:
        raise FvmError("global_avgpool: scratch too small")
    y = torch.empty((N, C), dtype=torch.float16, device=x.device)
    _check(lib().fvm_global_avgpool_f16(x.data_ptr(), y.data_ptr(), scratch.data_ptr(), N, H * W, C, ldx, _stream()),
           "global_avgpool_f16")
    return y.view(N, C, 1, 1)


# ------------------------------------------------------------------------------------------------ squeeze-excite
def se_gate(g, w1, b1, w2, b2, act: int = ACT_SILU, mean_scale: float = 0.0) -> torch.Tensor:
    """s = W2 act(W1 g + b1) + b2 for g [N,C(,1,1)] -> s [N,C,1,1] fp16 (pre-sigmoid)."""
    init(g.device)
    N = g.shape[0]
    C = g.shape[1]
    w1 = w1.reshape(w1.shape[0], -1).contiguous()
    w2 = w2.reshape(w2.shape[0], -1).contiguous()
    Cs = w1.shape[0]
    if w1.shape[1] != C or tuple(w2.shape) != (C, Cs):
        raise FvmError("se_gate: weight shapes do not match")
    g = g.reshape(N, C).contiguous()
    if mean_scale == 0.0:
        _require_cuda_half(g, "g")
    elif g.dtype != torch.float32:
        raise FvmError("se_gate: with mean_scale the squeeze input must be fp32 sums")
    s = torch.empty((N, C), dtype=torch.float16, device=g.device)
    _check(lib().fvm_se_gate_f16(g.data_ptr(), w1.data_ptr(), _ptr(b1), w2.data_ptr(), _ptr(b2), s.data_ptr(), N, C, Cs,
                                 int(act), float(mean_scale), _stream()), "se_gate_f16")
    return s.view(N, C, 1, 1)


def se_gate_pooled(partial, pixels: int, w1, b1, w2, b2, act: int = ACT_SILU) -> torch.Tensor:
    """The gate fed by the fused squeeze of `dwconv(..., pool=True)`: partial fp32 [N, slots, C] -> s [N,C,1,1] fp16
    with g = half(sum over slots / pixels) (deterministic: the slots are added in order)."""
    init(partial.device)
    if partial.dtype != torch.float32 or partial.dim() != 3 or not partial.is_cuda:
        raise FvmError("se_gate_pooled: partial must be an fp32 CUDA tensor [N, slots, C]")
    partial = partial.contiguous()
    N, slots, C = partial.shape
    w1 = w1.reshape(w1.shape[0], -1).contiguous()
    w2 = w2.reshape(w2.shape[0], -1).contiguous()
    Cs = w1.shape[0]
    if w1.shape[1] != C or tuple(w2.shape) != (C, Cs):
        raise FvmError("se_gate_pooled: weight shapes do not match")
    s = torch.empty((N, C), dtype=torch.float16, device=partial.device)
    _check(lib().fvm_se_gate_pooled_f16(partial.data_ptr(), slots, w1.data_ptr(), _ptr(b1), w2.data_ptr(), _ptr(b2),
                                        s.data_ptr(), N, C, Cs, int(act), 1.0 / float(pixels), _stream()), "se_gate_pooled_f16")
    return s.view(N, C, 1, 1)


def gate_weights(w, s) -> torch.Tensor:
    """Folds a squeeze-excite gate into the 1x1 weights of the conv that follows, per image:
    out[n, k, c] = half(w[k, c] * half(sigmoid(s[n, c]))); w [K, C(,1,1)] fp16, s [N, C(,1,1)] fp16 (pre-sigmoid)."""
    init(w.device)
    _require_cuda_half(w, "w")
    _require_cuda_half(s, "s")
    K = w.shape[0]
    w2 = w.reshape(K, -1).contiguous()
    C = w2.shape[1]
    N = s.shape[0]
    s2 = s.reshape(N, -1).contiguous()
    if s2.shape[1] != C:
        raise FvmError("gate_weights: the gate has another channel count than the weights")
    out = torch.empty((N, K, C), dtype=torch.float16, device=w.device)
    _check(lib().fvm_gate_weights_f16(w2.data_ptr(), s2.data_ptr(), out.data_ptr(), N, K, C, _stream()), "gate_weights_f16")
    return out


def conv1x1_wbatch(x, w_n, bias=None, res=None, act: int = 0) -> torch.Tensor:
    """1x1 stride-1 convolution with per-image weights w_n [N, K, C] (from `gate_weights`): together they are
    se_scale + project conv without the pass that writes and re-reads the scaled tensor."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    _require_cuda_half(w_n, "w_n")
    if w_n.dim() != 3 or w_n.shape[0] != N or w_n.shape[2] != C:
        raise FvmError(f"conv1x1_wbatch: w_n must be [N, K, C] = [{N}, K, {C}], got {tuple(w_n.shape)}")
    w_n = w_n.contiguous()
    K = w_n.shape[1]
    y = empty_nhwc(N, K, H, W, x.device)
    ldr = 0
    if res is not None:
        res, Nr, Kr, Hr, Wr, ldr = nhwc_view(res, "res")
        if (Nr, Kr, Hr, Wr) != (N, K, H, W):
            raise FvmError("conv1x1_wbatch: residual shape does not match the output")
    if bias is not None:
        _require_cuda_half(bias, "bias")
        bias = bias.contiguous()
    _check(lib().fvm_conv1x1_wbatch_f16(x.data_ptr(), w_n.data_ptr(), _ptr(bias), _ptr(res), y.data_ptr(), N, H, W, C, K,
                                        ldx, K, ldr, int(act), _stream()), "conv1x1_wbatch_f16")
    return y


def se_scale(x, s) -> torch.Tensor:
    """clfr3::se_scale(x, s) (classification/fast/csrc/r3.cu:319-329): y = x * sigmoid(s)."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    if ldx != C:
        x = x.contiguous(memory_format=torch.channels_last)
    _require_cuda_half(s, "s")
    s = s.reshape(N, C).contiguous()
    y = empty_nhwc(N, C, H, W, x.device)
    _check(lib().fvm_se_scale_f16(x.data_ptr(), s.data_ptr(), y.data_ptr(), N, H * W, C, _stream()), "se_scale_f16")
    return y


# ------------------------------------------------------------------------------------------------ LayerNorm
def layernorm_cl(x, weight, bias, eps: float = 1e-6) -> torch.Tensor:
    """LayerNorm over the channel dimension of a channels-last tensor ([N,C,H,W] NHWC in memory) or over the last
    dimension of a contiguous [..., C] tensor; same shape and layout out."""
    init(x.device)
    _require_cuda_half(x, "x")
    if x.dim() == 4 and x.stride(1) == 1 and x.shape[1] > 1:
        xv, N, C, H, W, ldx = nhwc_view(x, "x")
        rows = N * H * W
        y = empty_nhwc(N, C, H, W, x.device)
        src = xv
    else:
        src = x.contiguous()
        C = src.shape[-1]
        rows = src.numel() // C
        ldx = C
        y = torch.empty_like(src)
    _check(lib().fvm_layernorm_cl_f16(src.data_ptr(), _ptr(weight), _ptr(bias), y.data_ptr(), rows, C, float(eps), ldx,
                                      C, _stream()), "layernorm_cl_f16")
    return y


# ------------------------------------------------------------------------------------------------ elementwise
def input_nhwc8(x: torch.Tensor) -> torch.Tensor:
    """clf::input_nhwc8(x) (fused_conv.cu:608-620): fp32 or fp16 NCHW (C<=8) -> fp16 channels-last, C padded to 8."""
    init(x.device)
    if not x.is_cuda or x.dtype not in (torch.float32, torch.float16):
        raise FvmError("input_nhwc8: expected an fp32 or fp16 CUDA tensor")
    x = x.contiguous()
    N, C, H, W = x.shape
    y = empty_nhwc(N, 8, H, W, x.device)
    fn = lib().fvm_input_nhwc8_f32 if x.dtype == torch.float32 else lib().fvm_input_nhwc8_f16
    _check(fn(x.data_ptr(), y.data_ptr(), N, C, H, W, _stream()), "input_nhwc8")
    return y


def input_nhwc8_split(x: torch.Tensor) -> torch.Tensor:
    """input_nhwc8 into two column-parity planes per image row: returns fp16 [N, H, 2, W/2, 8] with
    out[n, h, w & 1, w >> 1, c] = x[n, c, h, w] (channels zero-padded to 8). Input layout of `stem_conv_s2`."""
    init(x.device)
    if not x.is_cuda or x.dtype not in (torch.float32, torch.float16):
        raise FvmError("input_nhwc8_split: expected an fp32 or fp16 CUDA tensor")
    x = x.contiguous()
    N, C, H, W = x.shape
    if W % 2:
        raise FvmError("input_nhwc8_split: the width must be even")
    y = torch.empty((N, H, 2, W // 2, 8), dtype=torch.float16, device=x.device)
    fn = lib().fvm_input_nhwc8_split_f32 if x.dtype == torch.float32 else lib().fvm_input_nhwc8_split_f16
    _check(fn(x.data_ptr(), y.data_ptr(), N, C, H, W, _stream()), "input_nhwc8_split")
    return y


def stem_conv_s2(xs: torch.Tensor, w: torch.Tensor, bias, padding, act: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Stride-2 stem on the split input: xs [N, H, 2, W/2, 8] (from `input_nhwc8_split`), w [K, 8, R, S] channels-last
    (the KRSC weights of `conv_fused`), same-sided padding (ph, pw). Returns act(conv + bias) as NHWC fp16."""
    init(xs.device)
    if xs.dim() != 5 or xs.shape[2] != 2 or xs.shape[4] != 8 or xs.dtype != torch.float16 or not xs.is_contiguous():
        raise FvmError("stem_conv_s2: xs must be a contiguous fp16 [N, H, 2, W/2, 8] tensor")
    N, H, _, Wh, _ = xs.shape
    W = 2 * Wh
    K, C, R, S = w.shape
    if C != 8 or w.dtype != torch.float16 or not w.is_contiguous(memory_format=torch.channels_last):
        raise FvmError("stem_conv_s2: w must be a channels-last fp16 [K, 8, R, S] tensor")
    ph, pw = padding
    P, Q = (H + 2 * ph - R) // 2 + 1, (W + 2 * pw - S) // 2 + 1
    if out is None:
        out = empty_nhwc(N, K, P, Q, xs.device)
    ov, oN, oK, oP, oQ, ldy = nhwc_view(out, "out")
    if ov is not out or (oN, oK, oP, oQ) != (N, K, P, Q):
        raise FvmError(f"stem_conv_s2: out must be a channels-last [N,K,P,Q]={N, K, P, Q} tensor or channel slice")
    _check(lib().fvm_stem_conv_s2_f16(xs.data_ptr(), w.data_ptr(), _ptr(bias), ov.data_ptr(), N, H, W, K, R, S, ph, pw,
                                      ldy, int(act), _stream()), "stem_conv_s2_f16")
    return out


_STEM_WEIGHTS = {}


def _stem_weights_from_rsck(w_t: torch.Tensor) -> torch.Tensor:
    """The reference's raw-input stem weights w_t [R, S, C, K] (C <= 4; classification/fast/fused.py:73) as this
    library's KRSC weights with the input channels zero-padded to 8. Re-packed once per weight tensor."""
    key = (w_t.data_ptr(), tuple(w_t.shape), w_t.device.index, w_t._version)
    w = _STEM_WEIGHTS.get(key)
    if w is None:
        R, S, C, K = w_t.shape
        if C > 8:
            raise FvmError("stem: at most 8 input channels")
        w = torch.zeros((K, 8, R, S), dtype=torch.float16, device=w_t.device)
        w[:, :C] = w_t.permute(3, 2, 0, 1)
        w = w.contiguous(memory_format=torch.channels_last)
        if len(_STEM_WEIGHTS) > 64:
            _STEM_WEIGHTS.clear()
        _STEM_WEIGHTS[key] = w
    return w


def stem_direct(x, w_t, bias=None, stride=(2, 2), pad=(1, 1), act: int = 0) -> torch.Tensor:
    """clfmb::stem_direct(x, w_t, bias?, stride, pad, act) (classification/fast/csrc/mbconv.cu:1212-1241): the stem
    convolution straight from the raw fp32 / fp16 NCHW image batch (C <= 4), w_t [R, S, C, K] fp16. Stride-2 stems on
    even-width images run as `input_nhwc8_split` + `stem_conv_s2`, everything else as `input_nhwc8` + `conv_fused`."""
    _require_cuda_half(w_t, "w_t")
    if w_t.dim() != 4 or w_t.shape[2] != x.shape[1] or not w_t.is_contiguous():
        raise FvmError("stem_direct: w_t must be a contiguous [R, S, C, K] tensor matching the image channels")
    w = _stem_weights_from_rsck(w_t)
    K, _, R, S = w.shape
    sh, sw = _pair(stride)
    ph, pw_ = _pair(pad)
    if (sh, sw) == (2, 2) and x.shape[3] % 2 == 0 and R <= 8 and S <= 8 and K <= 256 and K % 8 == 0 and ph < R and pw_ < S \
            and (R + R % 2) * S * ((K + 31) // 32 * 32) * 16 <= 96 * 1024:
        return stem_conv_s2(input_nhwc8_split(x), w, bias, (ph, pw_), act)
    return conv_fused(input_nhwc8(x), w, bias, None, (ph, pw_), (sh, sw), act)


def stem_pool(x, w_t, bias, stride, pad, act: int, pk: int, ps: int, pp: int, ceil: bool = False) -> torch.Tensor:
    """clfr3::stem_pool(x, w_t, bias?, stride, pad, act, pk, ps, pp, ceil) (classification/fast/csrc/r3.cu:584-630): stem
    convolution from the raw image followed by a pk x pk max pool (stride ps, padding pp). The reference runs the pair
    as one kernel; here it is the stem convolution and the pooling kernel back to back (two launches)."""
    return maxpool(stem_direct(x, w_t, bias, stride, pad, act), (pk, pk), (ps, ps), (pp, pp), ceil)


def bias_act_(y, bias=None, res=None, relu: bool = False) -> torch.Tensor:
    """segx::bias_act_(y, bias?, res?, relu) in place (segmentation/fast/csrc/segx_ops.cu:28-42)."""
    init(y.device)
    yv, N, C, H, W, ld = nhwc_view(y, "y")
    if yv is not y or ld != C:
        raise FvmError("bias_act_: y must be channels-last contiguous")
    if res is not None:
        res, *_r, ldr = nhwc_view(res, "res")
        if ldr != C:
            res = res.contiguous(memory_format=torch.channels_last)
    _check(lib().fvm_bias_act_f16(y.data_ptr(), _ptr(bias), _ptr(res), N * H * W, C, int(relu), _stream()),
           "bias_act_f16")
    return y


def affine_act(x, scale, shift, act: int) -> torch.Tensor:
    """clf::affine_act(x, scale, shift, act) (fused_conv.cu:323-335)."""
    init(x.device)
    x, N, C, H, W, ldx = nhwc_view(x, "x")
    y = empty_nhwc(N, C, H, W, x.device)
    _check(lib().fvm_affine_act_f16(x.data_ptr(), scale.float().contiguous().data_ptr(),
                                    shift.float().contiguous().data_ptr(), y.data_ptr(), N * H * W, C, ldx, C, int(act),
                                    _stream()), "affine_act_f16")
    return y


def add_act(a, b, act: int = 0) -> torch.Tensor:
    """y = act(a + b) for two channels-last tensors of the same shape."""
    init(a.device)
    a, N, C, H, W, lda = nhwc_view(a, "a")
    b, *_s, ldb = nhwc_view(b, "b")
    if lda != C:
        a = a.contiguous(memory_format=torch.channels_last)
    if ldb != C:
        b = b.contiguous(memory_format=torch.channels_last)
    y = empty_nhwc(N, C, H, W, a.device)
    _check(lib().fvm_add_act_f16(a.data_ptr(), b.data_ptr(), y.data_ptr(), a.numel(), int(act), _stream()), "add_act_f16")
    return y


# ------------------------------------------------------------------------------------------------ resize / argmax
def upsample_bilinear(x, H: int, W: int, sf_h: Optional[float] = None, sf_w: Optional[float] = None,
                      align: bool = False, base=None, relu: bool = False, out: Optional[torch.Tensor] = None
                      ) -> torch.Tensor:
    """segx::upsample_bilinear(x, H, W, sf_h?, sf_w?, align) and upsample_add (segx_ops.cu:131-217). `out` may be a
    channel slice of a wider channels-last buffer."""
    init(x.device)
    x, N, C, h, w, ldx = nhwc_view(x, "x")
    ldy = C
    if out is None:
        y = empty_nhwc(N, C, H, W, x.device)
    else:
        y, No, Co, Ho, Wo, ldy = nhwc_view(out, "out")
        if y is not out or (No, Co, Ho, Wo) != (N, C, H, W):
            raise FvmError("upsample_bilinear: out must be a channels-last [N,C,H,W] tensor or channel slice")
    if base is not None:
        base, *_s, ldb = nhwc_view(base, "base")
        if ldb != C:
            base = base.contiguous(memory_format=torch.channels_last)
    if base is not None and ldy != C:
        raise FvmError("upsample_bilinear: base and a sliced output cannot be combined")
    _check(lib().fvm_bilinear_f16(x.data_ptr(), _ptr(base), y.data_ptr(), N, h, w, C, H, W, int(align),
                                  float(sf_h or 0.0), float(sf_w or 0.0), int(relu), ldx, ldy, _stream()), "bilinear_f16")
    return y


def upsample_like(x, ref, align: bool = False) -> torch.Tensor:
    """segx::upsample_like(x, ref, align) (segx_ops.cu:160-162): bilinear resize of x to ref's height and width."""
    return upsample_bilinear(x, int(ref.shape[2]), int(ref.shape[3]), None, None, align)


def upsample_bilinear_t(x, size: torch.Tensor, align: bool = False) -> torch.Tensor:
    """segx::upsample_bilinear_t(x, size, align) (segx_ops.cu:166-169): the target size comes as an integer tensor [2]
    (the reference builds it from traced sizes so that a TorchScript trace stays shape-generic)."""
    hw = size.to("cpu", torch.int64).reshape(-1).tolist()
    if len(hw) != 2:
        raise FvmError("upsample_bilinear_t: size must hold (H, W)")
    return upsample_bilinear(x, int(hw[0]), int(hw[1]), None, None, align)


def _upsample_add(base, z, sf: float, relu: bool, inplace: bool) -> torch.Tensor:
    import math
    N, C, H, W = base.shape
    h, w = z.shape[2], z.shape[3]
    if z.shape[1] != C:
        raise FvmError("upsample_add: base and z must have the same channel count")
    bv, *_b, ldb = nhwc_view(base, "base")
    if inplace and (bv is not base or ldb != C):
        raise FvmError("upsample_add_: base must be a contiguous channels-last tensor")
    out = base if inplace else None
    if math.floor(h * sf) == H and math.floor(w * sf) == W:
        # one pass: the resize by `sf` lands exactly on base's size (segx_ops.cu:205-216: source scale 1 / sf)
        return upsample_bilinear(z, H, W, sf, sf, False, base=bv, relu=relu, out=out)
    # composite of the reference (segx_ops.cu:209-214): resize by sf, resize again to base's size, add, ReLU
    u = upsample_bilinear(z, int(math.floor(h * sf)), int(math.floor(w * sf)), sf, sf, False)
    return upsample_bilinear(u, H, W, None, None, False, base=bv, relu=relu, out=out)


def upsample_add(base, z, sf: float, relu: bool = False) -> torch.Tensor:
    """segx::upsample_add(base, z, sf, relu) (segx_ops.cu:200-218): relu?(base + half(bilinear(z, scale_factor sf)))."""
    return _upsample_add(base, z, float(sf), bool(relu), False)


def upsample_add_(base, z, sf: float, relu: bool = False) -> torch.Tensor:
    """segx::upsample_add_(base, z, sf, relu): the same, written into `base`."""
    return _upsample_add(base, z, float(sf), bool(relu), True)


def up_argmax(s, H: int, W: int, align: bool = False, num_classes: Optional[int] = None) -> torch.Tensor:
    """segx::up_argmax(s, H, W, align) (segx_ops.cu:171-195): int32 class map [N,H,W]; first maximum wins.
    `num_classes` restricts the argmax to the first channels of a zero-padded score tensor."""
    init(s.device)
    s, N, C, h, w, ld = nhwc_view(s, "s")
    C_eff = C if num_classes is None else int(num_classes)
    out = torch.empty((N, H, W), dtype=torch.int32, device=s.device)
    _check(lib().fvm_up_argmax_f16(s.data_ptr(), out.data_ptr(), N, h, w, C_eff, ld, H, W, int(align), _stream()),
           "up_argmax_f16")
    return out
