"""GPU parity of every kernel against the CPU oracle, called through the C-ABI (ctypes) operator layer."""
import pytest
import torch

from conftest import rel_l2
from fast_vision_models_b200 import ops
from oracle import ops_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda"
# fp16 outputs of fp32-accumulated ops: the CUDA result and the oracle differ by summation order and one rounding
TOL_REL_L2 = 1e-3
TOL_ULP = 2 ** -9       # |a-b| <= TOL_ULP * max(|b|, 1): about four fp16 ulps


def gen(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).half()


def cl(t):
    return t.to(DEV).contiguous(memory_format=torch.channels_last)


def close(y, ref, tol=TOL_REL_L2):
    y, ref = y.float().cpu(), ref.float().cpu()
    assert y.shape == ref.shape, (y.shape, ref.shape)
    assert torch.isfinite(y).all()
    assert rel_l2(y, ref) < tol, rel_l2(y, ref)
    assert ((y - ref).abs() <= 4 * TOL_ULP * ref.abs().clamp_min(1.0) + 1e-3).all()


CONV_CASES = [
    # N, H, W, C, K, R, S, pad, stride, dil, act, res
    (2, 8, 8, 64, 64, 1, 1, 0, 1, 1, 0, False),
    (2, 56, 56, 64, 256, 1, 1, 0, 1, 1, 1, True),
    (3, 14, 14, 256, 1024, 1, 1, 0, 1, 1, 1, True),
    (2, 7, 7, 2048, 512, 1, 1, 0, 1, 1, 1, False),
    (2, 9, 9, 48, 24, 1, 1, 0, 1, 1, 3, False),        # ragged channels: C and K below one tile
    (2, 9, 9, 144, 40, 1, 1, 0, 1, 1, 0, True),
    (2, 5, 5, 64, 1000, 1, 1, 0, 1, 1, 0, False),       # classifier-head shape: K not a multiple of 64
    (1, 1, 1, 2048, 1000, 1, 1, 0, 1, 1, 0, False),     # one pixel
    (2, 8, 8, 64, 64, 3, 3, 1, 1, 1, 0, False),
    (2, 56, 56, 64, 64, 3, 3, 1, 1, 1, 1, True),
    (2, 28, 28, 128, 128, 3, 3, 1, 2, 1, 1, False),
    (2, 14, 14, 256, 512, 1, 1, 0, 2, 1, 0, False),     # stride-2 1x1 downsample
    (2, 17, 13, 64, 64, 3, 3, 1, 1, 1, 1, False),       # odd sizes: tiles cross rows and images
    (2, 16, 16, 64, 64, 3, 3, 2, 1, 2, 1, False),       # dilation 2
    (1, 32, 32, 64, 64, 3, 3, 12, 1, 12, 1, False),     # ASPP-style dilation 12
    (1, 40, 40, 64, 64, 3, 3, 36, 1, 36, 1, False),     # dilation 36: most taps fall outside the image
    (2, 15, 15, 48, 48, 5, 5, 2, 2, 1, 3, False),
    (2, 32, 32, 8, 64, 7, 7, 3, 2, 1, 1, False),        # ResNet stem on zero-padded RGB
    (2, 32, 32, 8, 96, 4, 4, 0, 4, 1, 0, False),        # ConvNeXt patchify stem
    (2, 37, 41, 8, 48, 3, 3, 1, 2, 1, 3, False),        # EfficientNet-B4 stem shape (tap-packed path, 9 taps)
    (3, 30, 30, 8, 264, 3, 3, 1, 1, 1, 0, False),       # 8-channel input, K too wide for the tap-packed path
    (2, 12, 12, 96, 192, 2, 2, 0, 2, 1, 0, False),      # ConvNeXt downsample
    (2, 14, 14, 96, 384, 1, 1, 0, 1, 1, 5, False),      # fc1 + GELU
    (2, 14, 14, 96, 96, 1, 1, 0, 1, 1, 6, True),
    (2, 6, 6, 64, 64, 1, 1, 0, 1, 1, 4, False),         # hardswish
    (2, 6, 6, 64, 64, 1, 1, 0, 1, 1, 2, False),         # relu6
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_fused_matches_oracle(case):
    N, H, W, C, K, Rr, S, pad, stride, dil, act, res = case
    x = gen((N, C, H, W), 1)
    w = gen((K, C, Rr, S), 2, 0.05)
    b = gen((K,), 3, 0.1)
    P = (H + 2 * pad - dil * (Rr - 1) - 1) // stride + 1
    Q = (W + 2 * pad - dil * (S - 1) - 1) // stride + 1
    r = gen((N, K, P, Q), 4) if res else None
    ref = R.conv_fused_ref(x, w, b, r, (pad, pad), (stride, stride), act, (dil, dil))
    y = ops.conv_fused(cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (stride, stride), act,
                       dilation=(dil, dil))
    assert ops.last_status() == 0
    close(y, ref)


@pytest.mark.parametrize("tile", [64, 128, 192, 256])
def test_conv_every_tile_width(tile):
    x, w, b, r = gen((2, 128, 28, 28), 1), gen((256, 128, 1, 1), 2, 0.05), gen((256,), 3, 0.1), gen((2, 256, 28, 28), 4)
    ref = R.conv_fused_ref(x, w, b, r, act=1)
    y = ops.conv_fused(cl(x), cl(w), b.to(DEV), cl(r), act=1, tile_n=tile)
    assert ops.last_status() == 0
    close(y, ref)


@pytest.mark.parametrize("mt", [1, 2, 4])
@pytest.mark.parametrize("case", [(3, 20, 20, 64, 64, 1, 0, True), (3, 20, 20, 64, 64, 3, 1, False),
                                  (3, 23, 23, 8, 64, 7, 3, False), (5, 9, 9, 128, 128, 1, 0, True),
                                  (1, 5, 5, 64, 32, 1, 0, False)])
def test_conv_tiles_of_several_sub_tiles(case, mt):
    # tiles of 128*mt output pixels (mt sub-tiles share one weight tile and one hand-off): ragged last tiles included
    N, H, W, C, K, Rr, pad, res = case
    if mt * ((K + 31) // 32 * 32) > 256:
        pytest.skip("accumulators would not fit TMEM twice")
    x, w, b = gen((N, C, H, W), 1), gen((K, C, Rr, Rr), 2, 0.05), gen((K,), 3, 0.1)
    stride = 2 if C == 8 else 1
    P = (H + 2 * pad - Rr) // stride + 1
    r = gen((N, K, P, P), 4) if res else None
    ref = R.conv_fused_ref(x, w, b, r, (pad, pad), (stride, stride), 1)
    try:
        y = ops.conv_fused(cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (stride, stride), 1,
                           tile_n=mt << 16)
    except ops.FvmError:
        assert mt == 4      # four sub-tiles may not fit shared memory; the library must say so, not mis-compute
        return
    assert ops.last_status() == 0
    close(y, ref)


@pytest.mark.parametrize("case", [(4, 20, 20, 64, 256, 1, 0, True, 64), (4, 20, 20, 64, 256, 1, 0, True, 128),
                                  (3, 14, 14, 256, 1024, 1, 0, True, 128), (2, 20, 20, 64, 64, 3, 1, False, 64),
                                  (2, 9, 9, 144, 40, 1, 0, True, 0), (64, 14, 14, 256, 64, 1, 0, False, 0)])
def test_conv_weight_resident_mode_matches_streaming_mode(case):
    # each CTA keeps the weight tile of one n-tile in shared memory and walks the m-tiles: same results, bit for bit
    N, H, W, C, K, Rr, pad, res, bn = case
    x, w, b = gen((N, C, H, W), 1), gen((K, C, Rr, Rr), 2, 0.05), gen((K,), 3, 0.1)
    r = gen((N, K, H, W), 4) if res else None
    ref = R.conv_fused_ref(x, w, b, r, (pad, pad), (1, 1), 1)
    args = (cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (1, 1), 1)
    y_on = ops.conv_fused(*args, tile_n=(1 << 24) | bn)
    y_off = ops.conv_fused(*args, tile_n=(2 << 24) | bn)
    assert ops.last_status() == 0
    close(y_on, ref)
    assert torch.equal(y_on, y_off)


STREAMK_CASES = [
    # N, H, W, C, K, R, pad, stride, res, tile width (0 = library's choice)
    (64, 14, 14, 1024, 256, 1, 0, 1, False, 256),    # 98 tiles on 148 SMs: every tile shared by two or three CTAs
    (64, 14, 14, 256, 256, 3, 1, 1, False, 256),     # im2col loads, 36 k-blocks per tile
    (64, 14, 14, 256, 1024, 1, 0, 1, True, 128),     # residual, 784 tiles of 4 k-blocks
    (64, 7, 7, 2048, 512, 1, 0, 1, False, 128),
    (64, 7, 7, 512, 2048, 1, 0, 1, True, 0),
    (64, 7, 7, 512, 512, 3, 1, 1, False, 128),
    (64, 1, 1, 2048, 1000, 1, 0, 1, False, 128),     # classifier GEMM: one row tile, ragged last column tile
    (64, 14, 14, 1024, 512, 1, 0, 2, False, 0),      # stride-2 downsample (im2col map)
    (37, 9, 11, 128, 192, 1, 0, 1, True, 64),        # ragged rows, two k-blocks
    (12, 10, 10, 96, 40, 3, 1, 1, False, 0),         # ragged channels on both sides
]


@pytest.mark.parametrize("case", STREAMK_CASES)
def test_conv_stream_k_matches_oracle_and_plain_schedule(case):
    # the k-blocks of all tiles cut into one run per SM; tiles that straddle runs are summed in fp32 through the
    # library's scratch buffer. Against the oracle (first and last image) and against the plain schedule (all of it);
    # twice in a row: the hand-over counters must be back at zero after every launch.
    N, H, W, C, K, Rr, pad, stride, res, bn = case
    x, w, b = gen((N, C, H, W), 21), gen((K, C, Rr, Rr), 22, 0.02), gen((K,), 23, 0.1)
    P = (H + 2 * pad - Rr) // stride + 1
    r = gen((N, K, P, P if H == W else (W + 2 * pad - Rr) // stride + 1), 24) if res else None
    args = (cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (stride, stride), 1)
    y_sk = ops.conv_fused(*args, tile_n=(1 << 28) | bn)
    assert ops.last_status() == 0
    y_plain = ops.conv_fused(*args, tile_n=(2 << 28) | bn)
    assert ops.last_status() == 0
    for img in (0, N - 1):
        ref = R.conv_fused_ref(x[img:img + 1], w, b, None if r is None else r[img:img + 1], (pad, pad), (stride, stride), 1)
        close(y_sk[img:img + 1], ref)
    close(y_sk, y_plain)
    y_again = ops.conv_fused(*args, tile_n=(1 << 28) | bn)
    assert ops.last_status() == 0
    assert torch.equal(y_again, y_sk)           # fixed order of the partial sums: same bits every time


def test_conv_stream_k_is_refused_where_it_does_not_apply():
    x, w = cl(gen((1, 64, 4, 4), 1)), cl(gen((64, 64, 1, 1), 2, 0.05))
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x, w, None, None, (0, 0), (1, 1), 0, tile_n=1 << 28)          # fewer k-blocks than SMs
    x8, w8 = cl(gen((2, 8, 32, 32), 1)), cl(gen((64, 8, 7, 7), 2, 0.05))
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x8, w8, None, None, (3, 3), (2, 2), 0, tile_n=1 << 28)        # tap-packed stem


def _random_conv_cases(n, seed):
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < n:
        R_ = rng.choice([1, 1, 3, 3, 5])
        stride = rng.choice([1, 1, 2])
        dil = rng.choice([1, 1, 2]) if R_ > 1 else 1
        pad = rng.choice([0, (R_ // 2) * dil, R_ // 2]) if R_ > 1 else 0
        C = 8 * rng.randint(1, 40)
        K = 8 * rng.randint(1, 40)
        N = rng.randint(1, 9)
        H, W = rng.randint(1, 40), rng.randint(1, 40)
        if (H + 2 * pad - dil * (R_ - 1) - 1) // stride + 1 <= 0 or (W + 2 * pad - dil * (R_ - 1) - 1) // stride + 1 <= 0:
            continue
        cases.append((N, H, W, C, K, R_, pad, stride, dil, rng.random() < 0.4, rng.choice([0, 1, 1, 3, 5]), rng.random() < 0.8))
    return cases


@pytest.mark.parametrize("case", _random_conv_cases(40, 2024))
def test_conv_random_shapes_with_the_library_s_own_tile_choice(case):
    # shapes drawn at random (seeded): whatever mode and tile the library picks for them (single CTA or pair, staged
    # patches, resident weights, tap-packed 8 / 16-channel inputs, reverse tile order) must agree with the oracle
    N, H, W, C, K, R_, pad, stride, dil, res, act, has_bias = case
    x, w = gen((N, C, H, W), 61), gen((K, C, R_, R_), 62, 1.0 / (C * R_ * R_) ** 0.5)
    b = gen((K,), 63, 0.1) if has_bias else None
    P = (H + 2 * pad - dil * (R_ - 1) - 1) // stride + 1
    Q = (W + 2 * pad - dil * (R_ - 1) - 1) // stride + 1
    r = gen((N, K, P, Q), 64) if res else None
    y = ops.conv_fused(cl(x), cl(w), None if b is None else b.to(DEV), None if r is None else cl(r), (pad, pad),
                       (stride, stride), act, dilation=(dil, dil))
    assert ops.last_status() == 0
    close(y, R.conv_fused_ref(x, w, b, r, (pad, pad), (stride, stride), act, dilation=(dil, dil)))


PAIR_CASES = [
    # N, H, W, C, K, R, pad, stride, res, act, tile width (0 = library's choice)
    (64, 14, 14, 1024, 256, 1, 0, 1, False, 1, 256),   # 49 tiles of 256 pixels x 256 channels, 16 k-blocks
    (64, 14, 14, 256, 256, 3, 1, 1, False, 1, 256),    # im2col loads in both CTAs, 36 k-blocks
    (64, 14, 14, 256, 1024, 1, 0, 1, True, 1, 128),    # residual, 8 n-tiles
    (64, 7, 7, 2048, 512, 1, 0, 1, False, 1, 256),     # M = 3136 = 12.25 tiles: the last peer CTA has no rows
    (64, 7, 7, 512, 2048, 1, 0, 1, True, 1, 0),
    (64, 7, 7, 512, 512, 3, 1, 1, False, 1, 128),
    (64, 1, 1, 2048, 1000, 1, 0, 1, False, 0, 128),    # classifier GEMM: 64 rows, ragged last column tile
    (64, 14, 14, 1024, 512, 1, 0, 2, False, 0, 256),   # stride-2 downsample (im2col map)
    (37, 9, 11, 128, 192, 1, 0, 1, True, 3, 64),       # ragged rows, SiLU
    (12, 10, 10, 96, 40, 3, 1, 1, False, 5, 0),        # ragged channels on both sides, GELU
    (3, 40, 40, 64, 32, 3, 2, 1, False, 1, 32),        # padding 2, one narrow tile
]


@pytest.mark.parametrize("case", PAIR_CASES)
def test_conv_cta_pairs_match_oracle_and_single_cta_kernel(case):
    # two CTAs per 256-pixel tile, each loading half of the weight tile (tcgen05.mma.cta_group::2). Against the oracle
    # (first and last image) and bit for bit against the single-CTA kernel (same products, same order of the k-blocks).
    ops.init(DEV)
    if ops.query(4) <= 0:
        pytest.skip("this device cannot launch CTA pairs")
    N, H, W, C, K, Rr, pad, stride, res, act, bn = case
    x, w, b = gen((N, C, H, W), 31), gen((K, C, Rr, Rr), 32, 0.02), gen((K,), 33, 0.1)
    P = (H + 2 * pad - Rr) // stride + 1
    Q = (W + 2 * pad - Rr) // stride + 1
    r = gen((N, K, P, Q), 34) if res else None
    args = (cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (stride, stride), act)
    y_pair = ops.conv_fused(*args, tile_n=(1 << 30) | bn)
    assert ops.last_status() == 0
    y_one = ops.conv_fused(*args, tile_n=(2 << 28) | (2 << 26) | (2 << 24) | bn)     # plain schedule, im2col, streamed weights
    assert ops.last_status() == 0
    for img in (0, N - 1):
        ref = R.conv_fused_ref(x[img:img + 1], w, b, None if r is None else r[img:img + 1], (pad, pad), (stride, stride), act)
        close(y_pair[img:img + 1], ref)
    assert torch.equal(y_pair, y_one)


@pytest.mark.parametrize("case", [
    # N, H, W, C, K, R, pad, stride, res, act: shapes whose default tile is a CTA pair of an unusual width
    (8, 14, 14, 64, 72, 1, 0, 1, False, 1),        # one 96-wide tile, 24 columns of padding
    (8, 14, 14, 512, 200, 1, 0, 1, False, 3),      # 224-wide tile, SiLU
    (8, 14, 14, 128, 136, 3, 1, 1, True, 1),       # two 128-wide tiles, the second 8 channels wide, residual
    (4, 28, 28, 96, 80, 3, 1, 2, False, 5),        # stride 2, GELU, 96-wide tile
    (2, 7, 7, 2048, 1000, 1, 0, 1, False, 0),      # eight tiles, ragged last one
    (1, 5, 5, 24, 64, 3, 1, 1, True, 1),           # fewer rows than one CTA's 128: the peer CTA has none
])
def test_conv_default_tiles_with_odd_channel_counts(case):
    N, H, W, C, K, Rr, pad, stride, res, act = case
    x, w, b = gen((N, C, H, W), 41), gen((K, C, Rr, Rr), 42, 0.03), gen((K,), 43, 0.1)
    P = (H + 2 * pad - Rr) // stride + 1
    Q = (W + 2 * pad - Rr) // stride + 1
    r = gen((N, K, P, Q), 44) if res else None
    y = ops.conv_fused(cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (stride, stride), act)
    assert ops.last_status() == 0
    close(y, R.conv_fused_ref(x, w, b, r, (pad, pad), (stride, stride), act))
    y1 = ops.conv_fused(cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (pad, pad), (stride, stride), act,
                        tile_n=(2 << 28) | (2 << 26) | (2 << 24) | 64)            # single-CTA kernel, 64-wide tiles
    assert torch.equal(y, y1)


def test_conv_cta_pairs_are_refused_where_they_do_not_apply():
    x8, w8 = cl(gen((2, 8, 32, 32), 1)), cl(gen((64, 8, 7, 7), 2, 0.05))
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x8, w8, None, None, (3, 3), (2, 2), 0, tile_n=1 << 30)                  # tap-packed stem
    x, w = cl(gen((2, 64, 16, 16), 1)), cl(gen((64, 64, 3, 3), 2, 0.05))
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x, w, None, None, (1, 1), (1, 1), 0, tile_n=(1 << 30) | (1 << 28))      # with stream-K
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x, w, None, None, (1, 1), (1, 1), 0, tile_n=(1 << 30) | (2 << 16))      # with two sub-tiles


def _resnet_stage(N, H, W, cin, mid, blocks, stride, seed):
    """Weights and a runner for a ResNet bottleneck stage (torchvision layout: the stride sits on the 3x3 convolution
    and on the 1x1 downsample of the first block). run() returns every layer's output, in launch order."""
    x = cl(gen((N, cin, H, W), seed))
    ws = []
    c = cin
    for b in range(blocks):
        s_ = stride if b == 0 else 1
        blk = {"c1": (cl(gen((mid, c, 1, 1), seed + 10 * b + 1, 0.05)), gen((mid,), seed + 10 * b + 2, 0.1).to(DEV)),
               "c2": (cl(gen((mid, mid, 3, 3), seed + 10 * b + 3, 0.03)), gen((mid,), seed + 10 * b + 4, 0.1).to(DEV)),
               "c3": (cl(gen((4 * mid, mid, 1, 1), seed + 10 * b + 5, 0.05)), gen((4 * mid,), seed + 10 * b + 6, 0.1).to(DEV)),
               "stride": s_}
        if b == 0:
            blk["ds"] = (cl(gen((4 * mid, c, 1, 1), seed + 7, 0.05)), gen((4 * mid,), seed + 8, 0.1).to(DEV))
        ws.append(blk)
        c = 4 * mid

    def run():
        outs = []
        y = x
        for blk in ws:
            s_ = blk["stride"]
            idn = y
            if "ds" in blk:
                idn = ops.conv_fused(y, blk["ds"][0], blk["ds"][1], None, (0, 0), (s_, s_), 0)
                outs.append(idn)
            a = ops.conv_fused(y, blk["c1"][0], blk["c1"][1], None, (0, 0), (1, 1), 1)
            b_ = ops.conv_fused(a, blk["c2"][0], blk["c2"][1], None, (1, 1), (s_, s_), 1)
            y = ops.conv_fused(b_, blk["c3"][0], blk["c3"][1], idn, (0, 0), (1, 1), 1)
            outs += [a, b_, y]
        return outs
    return run


DUAL_CASES = [
    # N, H, W, C1, K1, K2, act1, act2, residual
    (64, 56, 56, 64, 256, 64, 1, 1, True),     # ResNet-50 stage 1: conv3 + identity + ReLU, then the next block's conv1
    (8, 128, 256, 64, 256, 64, 1, 1, True),    # the same pair inside DeepLabV3 at 512 x 1024, batch 8
    (3, 19, 23, 64, 256, 64, 1, 1, True),      # 1311 pixels: ragged last tile
    (2, 9, 7, 128, 128, 48, 1, 0, True),       # two k-blocks in the first layer, 48 output channels
    (5, 12, 12, 64, 128, 16, 0, 1, True),      # y of one half only, narrowest z
    (4, 30, 30, 128, 128, 32, 3, 5, False),    # no residual, SiLU / GELU through the generic activation code
    (1, 1, 1, 64, 256, 64, 1, 1, False),       # a single pixel
    (64, 28, 28, 128, 128, 64, 1, 1, True),    # more tiles than one wave, fewer than three
    (64, 56, 56, 64, 256, 128, 1, 1, True),    # z wider than 64 channels (y in 64-channel units): stage 1 -> stage 2 of ResNet-50
    (3, 17, 11, 128, 128, 128, 1, 1, True),    # the same mode with two k-blocks, ragged
    (2, 21, 21, 64, 128, 80, 0, 1, False),     # 80 output channels, no residual
]


@pytest.mark.parametrize("case", DUAL_CASES)
def test_pw_dual_matches_two_launches_bit_for_bit(case):
    # y = act1(conv1x1(x) + b1 + res), z = act2(conv1x1(y) + b2) as one launch (the second layer reads y from the shared
    # memory tile it is stored from) against two launches of the single-layer kernel: same bits for y and for z
    N, H, W, C1, K1, K2, act1, act2, has_res = case
    ops.init(DEV)
    x = cl(gen((N, C1, H, W), 70))
    w1, b1 = cl(gen((K1, C1, 1, 1), 71, 0.08)), gen((K1,), 72, 0.1).to(DEV)
    w2, b2 = cl(gen((K2, K1, 1, 1), 73, 0.05)), gen((K2,), 74, 0.1).to(DEV)
    res = cl(gen((N, K1, H, W), 75)) if has_res else None
    y_ref = ops.conv_fused(x, w1, b1, res, (0, 0), (1, 1), act1)
    z_ref = ops.conv_fused(y_ref, w2, b2, None, (0, 0), (1, 1), act2)
    for _ in range(2):
        before = ops.launches()
        y, z = ops.pw_dual(x, w1, b1, res, act1, w2, b2, act2)
        assert ops.launches() - before == 1
        assert ops.last_status() == 0
        assert torch.equal(y, y_ref), (y.float() - y_ref.float()).abs().max().item()
        assert torch.equal(z, z_ref), (z.float() - z_ref.float()).abs().max().item()


def test_pw_dual_against_the_oracle_and_refusals():
    ops.init(DEV)
    N, H, W = 2, 11, 13
    x, w1, b1 = gen((N, 64, H, W), 80), gen((256, 64, 1, 1), 81, 0.08), gen((256,), 82, 0.1)
    w2, b2, res = gen((64, 256, 1, 1), 83, 0.05), gen((64,), 84, 0.1), gen((N, 256, H, W), 85)
    y, z = ops.pw_dual(cl(x), cl(w1), b1.to(DEV), cl(res), 1, cl(w2), b2.to(DEV), 1)
    assert ops.last_status() == 0
    close(y, R.conv_fused_ref(x, w1, b1, res, (0, 0), (1, 1), 1))
    close(z, R.conv_fused_ref(y.float().cpu(), w2, b2, None, (0, 0), (1, 1), 1))
    # shapes outside the kernel's range are refused by the host layer and by the C entry point (status 1, no launch)
    with pytest.raises(ops.FvmError):
        ops.pw_dual(cl(gen((1, 96, 4, 4), 86)), cl(gen((256, 96, 1, 1), 87)), None, None, 1, cl(w2), None, 1)
    L = ops.lib()
    xd, w1d, w2d = cl(x), cl(w1), cl(w2)
    yd, zd = ops.empty_nhwc(N, 256, H, W, DEV), ops.empty_nhwc(N, 64, H, W, DEV)
    before = ops.launches()
    args = lambda y_ptr, K2: (xd.data_ptr(), w1d.data_ptr(), None, None, y_ptr, w2d.data_ptr(), None, zd.data_ptr(),
                              N * H * W, 64, 256, K2, 64, 0, 256, 64, 1, 1, None)
    assert L.fvm_conv_dual_f16(*args(yd.data_ptr(), 40)) == 1           # K2 not a multiple of 16
    assert L.fvm_conv_dual_f16(*args(yd.data_ptr(), 144)) == 1          # K2 above 128
    assert L.fvm_conv_dual_f16(*args(xd.data_ptr(), 64)) == 1           # y overlaps x
    assert L.fvm_conv_dual_f16(*args(yd.data_ptr() + 8, 64)) == 1       # misaligned y
    assert ops.launches() == before


CHAIN_CASES = [
    # N, H, W, input channels, bottleneck width, blocks, stride of the first block
    (64, 28, 28, 512, 256, 3, 2),      # ResNet-50 stage 3 (first three blocks): 28x28 -> 14x14
    (64, 14, 14, 1024, 512, 3, 2),     # stage 4: 14x14 -> 7x7, 2048 output channels
    (64, 56, 56, 256, 128, 2, 2),      # stage 2: 56x56 -> 28x28
    (5, 20, 12, 96, 40, 2, 1),         # ragged rows and channels, no stride
    (3, 9, 9, 64, 32, 17, 1),          # 52 layers: sent out as two chain launches
]


@pytest.mark.parametrize("case", CHAIN_CASES)
def test_conv_chain_matches_layer_by_layer_launches(case):
    # the same convolutions recorded and sent out as chain launches (tiles ordered by their data dependencies inside
    # one kernel) against one launch per layer in stream order: same bits for every layer's output, twice in a row
    # (the completion counters are zeroed before every chain launch)
    ops.init(DEV)
    if ops.query(4) <= 0:
        pytest.skip("this device cannot launch CTA pairs")
    run = _resnet_stage(*case, seed=40)
    ref = run()
    assert ops.last_status() == 0
    for _ in range(2):
        before = ops.launches()
        assert ops.chain_begin()
        try:
            got = run()
        finally:
            ops.chain_end()
        assert ops.last_status() == 0
        n_launch = ops.launches() - before
        assert n_launch == (len(ref) + ops.CHAIN_MAX_LAYERS - 1) // ops.CHAIN_MAX_LAYERS, n_launch
        for i, (a, b) in enumerate(zip(got, ref)):
            assert torch.equal(a, b), f"layer {i}: {(a.float() - b.float()).abs().max().item()}"


def test_conv_chain_against_the_oracle():
    ops.init(DEV)
    if ops.query(4) <= 0:
        pytest.skip("this device cannot launch CTA pairs")
    N, C, H, W = 2, 64, 12, 10
    x, w1, b1 = gen((N, C, H, W), 51), gen((96, C, 3, 3), 52, 0.04), gen((96,), 53, 0.1)
    w2, b2 = gen((64, 96, 1, 1), 54, 0.08), gen((64,), 55, 0.1)
    assert ops.chain_begin()
    try:
        y1 = ops.conv_fused(cl(x), cl(w1), b1.to(DEV), None, (1, 1), (1, 1), 1)
        y2 = ops.conv_fused(y1, cl(w2), b2.to(DEV), cl(x), (0, 0), (1, 1), 3)       # residual from outside the chain
        y3 = ops.conv_fused(y2, cl(w2[:, :64]), b2.to(DEV), y2, (0, 0), (1, 1), 1)   # residual from inside
    finally:
        ops.chain_end()
    assert ops.last_status() == 0
    r1 = R.conv_fused_ref(x, w1, b1, None, (1, 1), (1, 1), 1)
    close(y1, r1)
    r2 = R.conv_fused_ref(y1.float().cpu(), w2, b2, x, (0, 0), (1, 1), 3)
    close(y2, r2)
    r3 = R.conv_fused_ref(y2.float().cpu(), w2[:, :64], b2, y2.float().cpu(), (0, 0), (1, 1), 1)
    close(y3, r3)


def test_conv_chain_with_aliased_buffers_falls_back_to_stream_order():
    # the second layer writes into the first layer's input buffer: not expressible as a chain, so the recorded layers
    # go out one by one and the result is that of stream order
    ops.init(DEV)
    if ops.query(4) <= 0:
        pytest.skip("this device cannot launch CTA pairs")
    x = cl(gen((4, 64, 16, 16), 61))
    w1, w2 = cl(gen((64, 64, 1, 1), 62, 0.1)), cl(gen((64, 64, 1, 1), 63, 0.1))
    y1_ref = ops.conv_fused(x, w1, None, None, (0, 0), (1, 1), 1)
    y2_ref = ops.conv_fused(y1_ref, w2, None, None, (0, 0), (1, 1), 1)
    xin = x.clone(memory_format=torch.channels_last)
    before = ops.launches()
    assert ops.chain_begin()
    try:
        y1 = ops.conv_fused(xin, w1, None, None, (0, 0), (1, 1), 1)
        ops.conv_fused_into(y1, w2, None, None, (0, 0), (1, 1), 1, xin)
    finally:
        ops.chain_end()
    assert ops.last_status() == 0
    assert ops.launches() - before == 2
    assert torch.equal(y1, y1_ref) and torch.equal(xin, y2_ref)


@pytest.mark.parametrize("M,C,K,act,res,scale", [(197 * 4, 384, 1536, 5, False, False), (197 * 4, 1536, 384, 0, True, True),
                                                  (64, 2048, 1000, 0, False, False), (1000, 96, 40, 3, True, False)])
def test_linear_gemm_matches_oracle(M, C, K, act, res, scale):
    # ops.linear: the row-major GEMM view the reference's transformer blocks use (`_lin`, classification/fast/vit.py:56-64):
    # y[M,K] = act((x[M,C] @ w[K,C]^T + bias) * scale + res), on the convolution kernel as a 1x1 convolution over M pixels
    x, w, b = gen((M, C), 91), gen((K, C), 92, 0.05), gen((K,), 93, 0.1)
    r = gen((M, K), 94) if res else None
    sc = (torch.rand(K, generator=torch.Generator().manual_seed(95)) + 0.5) if scale else None
    y = ops.linear(x.to(DEV), w.to(DEV), b.to(DEV), None if r is None else r.to(DEV), act,
                   None if sc is None else sc.to(DEV))
    assert ops.last_status() == 0
    v = x.float() @ w.float().t() + b.float()
    if sc is not None:
        v = v * sc
    if r is not None:
        v = v + r.float()
    close(y, R.act_ref(v, act).half())


GCONV_CASES = [
    # N, H, W, C, K, groups, R, pad, stride, act
    (4, 28, 28, 128, 128, 32, 3, 1, 1, 1),      # ResNeXt-50 32x4d stage 1: 4 channels per group, 16 groups per run
    (4, 14, 14, 256, 256, 16, 3, 1, 2, 1),      # 16 per group, stride 2
    (3, 20, 20, 96, 96, 2, 3, 1, 1, 3),         # RegNet-like 48 per group: one run over everything
    (2, 17, 13, 432, 432, 9, 3, 1, 1, 1),       # 48 per group, 9 groups: runs of 192 with a short last run
    (2, 12, 12, 448, 448, 4, 3, 1, 2, 1),       # 112 per group: one run of 448
    (5, 9, 9, 64, 128, 8, 1, 0, 1, 0),          # 1x1, more output than input channels per group (8 -> 16)
    (2, 16, 16, 224, 224, 28, 3, 1, 1, 1),      # 8 per group: runs of 64, 3.5 runs
]


@pytest.mark.parametrize("case", GCONV_CASES)
def test_gconv2_matches_oracle(case):
    N, H, W, C, K, G, Rr, pad, stride, act = case
    x, w, b = gen((N, C, H, W), 71), gen((K, C // G, Rr, Rr), 72, 0.08), gen((K,), 73, 0.1)
    y = ops.gconv2(cl(x), cl(w), b.to(DEV), (stride, stride), (pad, pad), G, act)
    assert ops.last_status() == 0
    close(y, R.gconv2_ref(x, w, b, (stride, stride), (pad, pad), G, act))
    y2, mean = ops.gconv2_pool(cl(x), cl(w), b.to(DEV), (stride, stride), (pad, pad), G, act)
    assert torch.equal(y2, y)
    close(mean, y.float().mean((2, 3), keepdim=True).half().cpu(), 2e-3)


def test_dwmult_matches_oracle():
    # depthwise with channel multiplier 2 and 4: output channel k reads input channel k // m
    for C, m, Rr in ((32, 2, 3), (16, 4, 5)):
        K = C * m
        x, w, b = gen((3, C, 15, 11), 81), gen((K, 1, Rr, Rr), 82, 0.2), gen((K,), 83, 0.1)
        w_rsk = w[:, 0].permute(1, 2, 0).contiguous().half().to(DEV)
        y = ops.dwmult(cl(x), w_rsk, b.to(DEV), (1, 1), (Rr // 2, Rr // 2), 3)
        assert ops.last_status() == 0
        close(y, R.gconv2_ref(x, w, b, (1, 1), (Rr // 2, Rr // 2), C, 3))


HALO_CASES = [
    # N, H, W, C, K, dil, res, tile, weight-resident (0 choose / 1 on / 2 off)
    (2, 16, 8, 64, 64, 1, False, 0, 2),        # exactly one patch per image
    (2, 56, 56, 64, 64, 1, True, 0, 1),        # ResNet layer1 shape: bottom patches half outside the image
    (3, 17, 13, 64, 64, 1, False, 0, 2),       # ragged: patches clipped on both borders
    (2, 28, 28, 128, 128, 1, True, 0, 2),      # two 64-channel chunks, weights streamed
    (2, 20, 24, 256, 256, 2, False, 256, 2),   # dilation 2, four chunks, 256-channel tile
    (1, 32, 32, 128, 512, 4, True, 128, 2),    # dilation 4, several n-tiles
    (2, 24, 16, 96, 40, 1, False, 0, 0),       # ragged channels on both sides
    (64, 14, 14, 64, 64, 1, False, 0, 0),      # many small images
]


@pytest.mark.parametrize("case", HALO_CASES)
def test_conv_halo_mode_matches_oracle_and_im2col_mode(case):
    # 3x3 stride-1 convolutions over staged input patches (each input pixel read once per tile) against the oracle
    # and against the same convolution through im2col loads (above 64 input channels the fp32 summation order differs)
    N, H, W, C, K, d, res, bn, wr = case
    x, w, b = gen((N, C, H, W), 11), gen((K, C, 3, 3), 12, 0.05), gen((K,), 13, 0.1)
    r = gen((N, K, H, W), 14) if res else None
    ref = R.conv_fused_ref(x, w, b, r, (d, d), (1, 1), 1, dilation=(d, d))
    args = (cl(x), cl(w), b.to(DEV), None if r is None else cl(r), (d, d), (1, 1), 1)
    y_halo = ops.conv_fused(*args, dilation=(d, d), tile_n=(1 << 26) | (wr << 24) | bn)
    assert ops.last_status() == 0
    y_plain = ops.conv_fused(*args, dilation=(d, d), tile_n=(2 << 26) | (wr << 24) | bn)
    assert ops.last_status() == 0
    close(y_halo, ref)
    close(y_halo, y_plain)
    if C <= 64:
        assert torch.equal(y_halo, y_plain)     # one 64-channel chunk: the taps are added in the same order


def test_conv_halo_mode_is_refused_where_it_does_not_apply():
    x, w = cl(gen((1, 64, 16, 16), 1)), cl(gen((64, 64, 3, 3), 2, 0.05))
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x, w, None, None, (1, 1), (2, 2), 0, tile_n=1 << 26)          # stride 2
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x, w, None, None, (8, 8), (1, 1), 0, dilation=(8, 8), tile_n=1 << 26)   # dilation above 4


@pytest.mark.parametrize("case", [(2, 20, 22, 16, 64, 3, 3, 1, 1), (2, 17, 19, 16, 48, 7, 4, 3, 1), (3, 12, 12, 16, 96, 2, 2, 0, 2),
                                  (1, 9, 40, 16, 256, 1, 5, 0, 1)])
def test_conv_sixteen_channel_taps(case):
    # 16-channel inputs take the tap-packed path with one MMA per filter tap (32-byte-swizzled rows)
    N, H, W, C, K, Rr, S, pad, stride = case
    x, w, b = gen((N, C, H, W), 1), gen((K, C, Rr, S), 2, 0.05), gen((K,), 3, 0.1)
    ref = R.conv_fused_ref(x, w, b, None, (pad, pad), (stride, stride), 1)
    y = ops.conv_fused(cl(x), cl(w), b.to(DEV), None, (pad, pad), (stride, stride), 1)
    assert ops.last_status() == 0
    close(y, ref)


@pytest.mark.parametrize("C", [16, 64])
def test_conv_separate_low_and_high_padding(C):
    x, w, b = gen((2, C, 11, 14), 1), gen((64, C, 3, 4), 2, 0.05), gen((64,), 3, 0.1)
    lo, hi = (1, 2), (0, 1)            # (top, left), (bottom, right)
    xp = torch.nn.functional.pad(x.float(), (lo[1], hi[1], lo[0], hi[0])).half()
    ref = R.conv_fused_ref(xp, w, b, None, (0, 0), (1, 1), 1)
    out = ops.empty_nhwc(2, 64, ref.shape[2], ref.shape[3], DEV)
    ops.conv_fused_into(cl(x), cl(w), b.to(DEV), None, lo, (1, 1), 1, out, pad_hi=hi)
    assert ops.last_status() == 0
    close(out, ref)


@pytest.mark.parametrize("case", [(2, 64, 64, 64, 7, 2, 3), (2, 38, 46, 48, 3, 2, 1), (2, 32, 48, 96, 4, 4, 0)])
def test_rgb_stem_over_column_pairs_matches_the_plain_stem(case):
    # FusedConv re-expresses an even-stride RGB stem over pairs of input columns; both ways must agree with the oracle
    from fast_vision_models_b200 import layers
    N, H, W, K, k, stride, pad = case
    conv = torch.nn.Conv2d(3, K, k, stride=stride, padding=pad, bias=True)
    x32 = torch.randn(N, 3, H, W, generator=torch.Generator().manual_seed(5))
    x8 = ops.input_nhwc8(x32.to(DEV))
    fc = layers.FusedConv.from_conv_bn(conv, None, 1).to(DEV)
    assert fc._pair is not None
    y_pair = fc(x8)
    fc._pair = None
    y_plain = fc(x8)
    w8 = torch.zeros(K, 8, k, k)
    w8[:, :3] = conv.weight.detach()
    ref = R.conv_fused_ref(R.input_nhwc8_ref(x32), w8.half(), conv.bias.detach().half(), None, (pad, pad), (stride, stride), 1)
    assert ops.last_status() == 0
    close(y_pair, ref)
    close(y_plain, ref)


STEM_CASES = [
    # N, H, W, K, R, S, pad, act
    (2, 64, 64, 64, 7, 7, 3, 1),        # ResNet stem
    (1, 224, 224, 64, 7, 7, 3, 1),      # full-size image: 7 x 14 patches
    (2, 38, 46, 48, 3, 3, 1, 3),        # EfficientNet stem shape: ragged patches, K below one tile
    (2, 37, 42, 32, 3, 3, 1, 0),        # odd height
    (2, 30, 34, 32, 5, 5, 2, 1),
    (2, 32, 32, 96, 7, 7, 3, 5),        # two 64-channel output boxes
    (3, 20, 24, 64, 4, 4, 1, 1),        # even filter: no zero-weight tap row
    (2, 16, 16, 256, 3, 3, 1, 1),       # widest tile
    (2, 18, 20, 64, 7, 7, 0, 0),        # no padding
]


@pytest.mark.parametrize("case", STEM_CASES)
def test_stem_conv_on_split_input_matches_oracle_and_plain_conv(case):
    # the stride-2 stem over column-parity planes: same products and sums as the convolution on the NHWC8 tensor
    N, H, W, K, Rr, S, pad, act = case
    g = torch.Generator().manual_seed(5)
    x = torch.randn((N, 3, H, W), generator=g)
    w = torch.zeros((K, 8, Rr, S))
    w[:, :3] = torch.randn((K, 3, Rr, S), generator=g) * 0.1
    w, b = w.half(), gen((K,), 6, 0.1)
    x8 = ops.input_nhwc8(x.to(DEV))
    ref = R.conv_fused_ref(x8.cpu(), w, b, None, (pad, pad), (2, 2), act)
    xs = ops.input_nhwc8_split(x.to(DEV))
    # the split tensor holds the NHWC8 pixels, even columns first
    assert torch.equal(xs[:, :, 0], x8.permute(0, 2, 3, 1)[:, :, 0::2]) and torch.equal(xs[:, :, 1], x8.permute(0, 2, 3, 1)[:, :, 1::2])
    y = ops.stem_conv_s2(xs, cl(w), b.to(DEV), (pad, pad), act)
    assert ops.last_status() == 0
    close(y, ref)
    y_plain = ops.conv_fused(x8, cl(w), b.to(DEV), None, (pad, pad), (2, 2), act)
    close(y, y_plain)


def test_stem_conv_without_bias_into_a_channel_slice_and_bad_arguments():
    g = torch.Generator().manual_seed(7)
    x = torch.randn((2, 3, 24, 24), generator=g).to(DEV)
    w = torch.zeros((32, 8, 3, 3))
    w[:, :3] = torch.randn((32, 3, 3, 3), generator=g) * 0.1
    w = cl(w.half())
    xs = ops.input_nhwc8_split(x)
    big = ops.empty_nhwc(2, 64, 12, 12, DEV).fill_(7.0)
    ops.stem_conv_s2(xs, w, None, (1, 1), 0, out=big[:, 16:48])
    ref = R.conv_fused_ref(ops.input_nhwc8(x).cpu(), w.cpu(), None, None, (1, 1), (2, 2), 0)
    close(big[:, 16:48], ref)
    assert (big[:, :16] == 7.0).all() and (big[:, 48:] == 7.0).all()
    with pytest.raises(ops.FvmError):
        ops.input_nhwc8_split(torch.randn(1, 3, 8, 9, device=DEV))          # odd width
    with pytest.raises(ops.FvmError):
        ops.stem_conv_s2(xs, cl(torch.zeros(32, 8, 9, 9).half()), None, (4, 4), 0)   # filter too large
    with pytest.raises(ops.FvmError):
        ops.stem_conv_s2(xs.float(), w, None, (1, 1), 0)


def test_conv_no_bias_scale_and_sliced_io():
    # input read from a channel slice, output written into a channel slice of a wider buffer (concat-free ASPP),
    # un-folded LayerScale as an fp32 epilogue scale
    x_wide = gen((2, 128, 10, 10), 1)
    w = gen((64, 64, 3, 3), 2, 0.05)
    scale = torch.rand(64, generator=torch.Generator().manual_seed(5)) + 0.5
    r = gen((2, 64, 10, 10), 4)
    ref = R.conv_fused_ref(x_wide[:, 64:], w, None, r, (1, 1), (1, 1), 0, scale=scale)
    xd = cl(x_wide)
    out_wide = torch.zeros((2, 192, 10, 10), dtype=torch.float16, device=DEV).contiguous(memory_format=torch.channels_last)
    ops.conv_fused_into(xd[:, 64:], cl(w), None, cl(r), (1, 1), (1, 1), 0, out_wide[:, 64:128], scale=scale.to(DEV))
    assert ops.last_status() == 0
    close(out_wide[:, 64:128], ref)
    assert out_wide[:, :64].abs().sum() == 0 and out_wide[:, 128:].abs().sum() == 0   # neighbours untouched


def test_conv_linearity_at_full_size():
    # size-independent property at a BASELINE-sized layer: conv(x1 + x2) == conv(x1) + conv(x2) up to fp16 rounding
    N, C, K, H = 64, 256, 256, 14
    x1, x2 = cl(gen((N, C, H, H), 1, 0.5)), cl(gen((N, C, H, H), 2, 0.5))
    w = cl(gen((K, C, 3, 3), 3, 0.02))
    y12 = ops.conv_fused((x1.float() + x2.float()).half(), w, None, None, (1, 1), (1, 1), 0)
    y1 = ops.conv_fused(x1, w, None, None, (1, 1), (1, 1), 0)
    y2 = ops.conv_fused(x2, w, None, None, (1, 1), (1, 1), 0)
    assert ops.last_status() == 0
    assert rel_l2(y12, y1.float() + y2.float()) < 2e-3


SWEEP_CASES = [(r, c, h) for r in (1, 3) for c in (64, 128, 256, 512) for h in (56, 28, 14, 7)]


@pytest.mark.parametrize("r,c,h", SWEEP_CASES)
def test_conv_sweep_at_batch_64(r, c, h):
    # The single-op sweep at its real size: N = 64, C_in = C_out = c, H = W = h, 1x1 (pad 0) and 3x3 (pad 1), stride 1,
    # input N(0,1), weights N(0,0.02), epilogue = folded-BatchNorm bias + residual N(0,1) + ReLU. The kernel flattens
    # the output pixels of all images into one row dimension, so tiles straddle image boundaries: the CPU oracle
    # checks the first, a middle and the last image, an fp32 convolution on the device checks the whole tensor.
    N, pad = 64, r // 2
    i = SWEEP_CASES.index((r, c, h))
    g = torch.Generator().manual_seed(10 + i)
    x = torch.randn((N, c, h, h), generator=g).half()
    w = (torch.randn((c, c, r, r), generator=g) * 0.02).half()
    res = torch.randn((N, c, h, h), generator=g).half()
    # bias of a BatchNorm folded with gamma ~ U(0.5,1.5), beta ~ N(0,0.1), mean ~ N(0,0.1), var ~ U(0.5,1.5)
    gamma, beta = torch.rand(c, generator=g) + 0.5, torch.randn(c, generator=g) * 0.1
    mean, var = torch.randn(c, generator=g) * 0.1, torch.rand(c, generator=g) + 0.5
    b = (beta - mean * gamma / torch.sqrt(var + 1e-5)).half()
    xd, wd, rd, bd = cl(x), cl(w), cl(res), b.to(DEV)
    y = ops.conv_fused(xd, wd, bd, rd, (pad, pad), (1, 1), ops.ACT_RELU)
    assert ops.last_status() == 0
    for img in (0, 31, 63):
        ref = R.conv_fused_ref(x[img:img + 1], w, b, res[img:img + 1], (pad, pad), (1, 1), 1)
        close(y[img:img + 1], ref)
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        full = torch.nn.functional.conv2d(xd.float(), wd.float(), bd.float(), 1, pad) + rd.float()
    finally:
        torch.backends.cudnn.allow_tf32 = old
    full = full.clamp_min(0)
    assert rel_l2(y, full) < TOL_REL_L2
    assert float((y.float() - full).abs().max()) <= 4 * TOL_ULP * float(full.abs().max()) + 1e-3


def test_conv_rejects_bad_arguments():
    x = cl(gen((1, 12, 4, 4), 1))        # C not a multiple of 8
    w = cl(gen((8, 12, 1, 1), 2))
    with pytest.raises(ops.FvmError):
        ops.conv_fused(x, w)
    with pytest.raises(ops.FvmError):
        ops.conv_fused(gen((1, 8, 4, 4), 1), gen((8, 8, 1, 1), 2))   # CPU tensors


DW_CASES = [
    # N, H, W, C, k, stride, pad, dil, act
    (2, 20, 20, 48, 3, 1, 1, 1, 3), (2, 21, 19, 144, 3, 2, 1, 1, 3), (2, 17, 17, 192, 5, 1, 2, 1, 3),
    (2, 16, 16, 336, 5, 2, 2, 1, 3), (2, 14, 14, 96, 7, 1, 3, 1, 0), (2, 7, 7, 768, 7, 1, 3, 1, 0),
    (1, 40, 40, 64, 3, 1, 1, 1, 1), (1, 12, 12, 32, 3, 1, 2, 2, 5), (3, 5, 5, 8, 3, 1, 1, 1, 0),
]


@pytest.mark.parametrize("case", DW_CASES)
def test_dwconv_matches_oracle(case):
    N, H, W, C, k, stride, pad, dil, act = case
    x, w, b = gen((N, C, H, W), 1), gen((k, k, C), 2, 0.2), gen((C,), 3, 0.1)
    ref = R.dwconv_ref(x, w, b, (stride, stride), (pad, pad), act, (dil, dil))
    y = ops.dwconv(cl(x), w.to(DEV), b.to(DEV), (stride, stride), (pad, pad), act, dilation=(dil, dil))
    close(y, ref)


def _random_dw_cases(n, seed):
    import random
    rng = random.Random(seed)
    cases = []
    while len(cases) < n:
        k = rng.choice([3, 3, 5, 7, rng.choice([1, 2, 4, 9])])
        stride = rng.choice([1, 1, 2])
        dil = rng.choice([1, 1, 1, 2])
        pad = rng.choice([(k // 2) * dil, k // 2, 0])
        C = 8 * rng.randint(1, 50)
        N, H, W = rng.randint(1, 5), rng.randint(1, 45), rng.randint(1, 45)
        if (H + 2 * pad - dil * (k - 1) - 1) // stride + 1 <= 0 or (W + 2 * pad - dil * (k - 1) - 1) // stride + 1 <= 0:
            continue
        cases.append((N, H, W, C, k, stride, pad, dil, rng.choice([0, 1, 3, 3, 5]), rng.random() < 0.8))
    return cases


@pytest.mark.parametrize("case", _random_dw_cases(30, 7))
def test_dwconv_random_shapes(case):
    # seeded random depthwise shapes: whichever kernel the library routes them to (tiled 3 / 5 / 7, general) vs the oracle
    N, H, W, C, k, stride, pad, dil, act, has_bias = case
    x, w = gen((N, C, H, W), 1), gen((k, k, C), 2, 1.0 / k)
    b = gen((C,), 3, 0.1) if has_bias else None
    ref = R.dwconv_ref(x, w, b, (stride, stride), (pad, pad), act, (dil, dil))
    y = ops.dwconv(cl(x), w.to(DEV), None if b is None else b.to(DEV), (stride, stride), (pad, pad), act, dilation=(dil, dil))
    assert ops.last_status() == 0
    close(y, ref)


DW_ANY_CASES = [
    # N, H, W, C, R, S, stride, pad, dil, act: every shape the tiled 3/5/7 kernel does not take
    (2, 20, 24, 64, 3, 3, 1, 2, 2, 5), (1, 40, 40, 32, 3, 3, 1, 12, 12, 0), (2, 9, 9, 24, 1, 5, 1, 2, 1, 1),
    (2, 16, 16, 48, 2, 2, 2, 0, 1, 0), (2, 3, 3, 72, 3, 3, 1, 1, 1, 3), (2, 30, 30, 16, 9, 9, 1, 4, 1, 0),
    (2, 21, 17, 40, 3, 3, 3, 1, 1, 4), (1, 2, 2, 8, 7, 7, 1, 3, 1, 0),
]


@pytest.mark.parametrize("case", DW_ANY_CASES)
def test_dwconv_any_shape_matches_oracle(case):
    N, H, W, C, Rr, S, stride, pad, dil, act = case
    pw_ = pad if Rr == S else (S // 2) * dil
    ph_ = pad if Rr == S else (Rr // 2) * dil
    x, w, b = gen((N, C, H, W), 1), gen((Rr, S, C), 2, 0.2), gen((C,), 3, 0.1)
    ref = R.dwconv_ref(x, w, b, (stride, stride), (ph_, pw_), act, (dil, dil))
    y = ops.dwconv(cl(x), w.to(DEV), b.to(DEV), (stride, stride), (ph_, pw_), act, dilation=(dil, dil))
    assert ops.last_status() == 0
    close(y, ref)


@pytest.mark.parametrize("case", [(3, 144, 19, 19, 3, 1, 3), (2, 96, 30, 30, 7, 1, 0), (2, 336, 17, 23, 5, 2, 3),
                                  (2, 48, 40, 40, 3, 1, 3), (2, 64, 12, 12, 3, 1, 1)])
def test_dwconv_fused_squeeze_is_exact_and_deterministic(case):
    N, C, H, W, k, stride, act = case
    x, w, b = gen((N, C, H, W), 1), gen((k, k, C), 2, 0.2), gen((C,), 3, 0.1)
    ref = R.dwconv_ref(x, w, b, (stride, stride), (k // 2, k // 2), act)
    y, partial = ops.dwconv(cl(x), w.to(DEV), b.to(DEV), (stride, stride), (k // 2, k // 2), act, pool=True)
    assert ops.last_status() == 0
    close(y, ref)
    assert partial.dtype == torch.float32 and partial.shape[0] == N and partial.shape[2] == C
    # the partial sums are sums of the kernel's own fp16 outputs: compare with those, not with the oracle's
    want = y.float().sum(dim=(2, 3))
    got = partial.sum(dim=1)
    assert (got - want).abs().max() <= 2e-4 * want.abs().max() + 1e-3
    y2, partial2 = ops.dwconv(cl(x), w.to(DEV), b.to(DEV), (stride, stride), (k // 2, k // 2), act, pool=True)
    assert torch.equal(partial, partial2) and torch.equal(y, y2)            # no atomics: same bits every time
    # the gate fed by the partial sums equals the gate fed by the global average pool of y
    Cs = 16
    w1, b1, w2, b2 = gen((Cs, C), 4, 0.1).to(DEV), gen((Cs,), 5, 0.1).to(DEV), gen((C, Cs), 6, 0.1).to(DEV), gen((C,), 7, 0.1).to(DEV)
    s_fused = ops.se_gate_pooled(partial, y.shape[2] * y.shape[3], w1, b1, w2, b2, 3)
    s_plain = ops.se_gate(ops.global_avgpool(y), w1, b1, w2, b2, 3)
    close(s_fused, s_plain, 2e-3)


@pytest.mark.parametrize("shape,k,s,p,ceil", [((2, 64, 112, 112), 3, 2, 1, False), ((2, 16, 9, 9), 2, 2, 0, True),
                                              ((1, 8, 7, 5), 3, 1, 1, False), ((2, 24, 8, 8), 3, 2, 0, True)])
def test_pools_match_oracle(shape, k, s, p, ceil):
    x = gen(shape, 1)
    y = ops.maxpool(cl(x), k, s, p, ceil)
    assert torch.equal(y.cpu().float(), R.maxpool_ref(x, k, s, p, ceil).float())    # max is exact
    for cip in (True, False):
        close(ops.avgpool(cl(x), k, s, p, cip, ceil=ceil), R.avgpool_ref(x, k, s, p, ceil, cip))


@pytest.mark.parametrize("shape", [(64, 2048, 7, 7), (2, 144, 95, 95), (3, 8, 1, 1), (2, 1792, 12, 12), (1, 48, 190, 190)])
def test_global_avgpool_matches_oracle_and_is_deterministic(shape):
    x = gen(shape, 1)
    xd = cl(x)
    y = ops.global_avgpool(xd)
    close(y, R.global_avgpool_ref(x))
    assert torch.equal(y, ops.global_avgpool(xd))


@pytest.mark.parametrize("N,C,Cs,act", [(4, 144, 8, 3), (2, 2688, 112, 3), (3, 48, 16, 1), (64, 672, 32, 3)])
def test_se_gate_and_scale_match_oracle(N, C, Cs, act):
    g, w1, b1 = gen((N, C, 1, 1), 1), gen((Cs, C), 2, 0.1), gen((Cs,), 3, 0.1)
    w2, b2 = gen((C, Cs), 4, 0.1), gen((C,), 5, 0.1)
    ref_s = R.se_gate_ref(g, w1, b1, w2, b2, act)
    s = ops.se_gate(g.to(DEV), w1.to(DEV), b1.to(DEV), w2.to(DEV), b2.to(DEV), act)
    close(s, ref_s, 2e-3)
    x = gen((N, C, 6, 5), 6)
    close(ops.se_scale(cl(x), ref_s.to(DEV)), R.se_scale_ref(x, ref_s))


@pytest.mark.parametrize("case", [(3, 144, 19, 19, 24, False), (4, 672, 24, 24, 112, True), (2, 48, 7, 5, 40, True),
                                  (64, 960, 12, 12, 272, False), (5, 96, 1, 1, 32, False)])
def test_gate_folded_into_project_weights_matches_scale_then_conv(case):
    # squeeze-excite scale + project conv without the scaled tensor: the rounded gate multiplies the 1x1 weights (per
    # image) instead of the activations; same products, the gate's fp16 rounding falls on the other operand
    N, C, H, W, K, res = case
    x, s = gen((N, C, H, W), 31), gen((N, C, 1, 1), 32)
    w, b = gen((K, C, 1, 1), 33, 0.05), gen((K,), 34, 0.1)
    r = gen((N, K, H, W), 35) if res else None
    ref = R.conv_fused_ref(R.se_scale_ref(x, s), w, b, r, act=0)
    w_n = ops.gate_weights(cl(w), s.to(DEV))
    assert w_n.shape == (N, K, C)
    want_w = (w.float().view(1, K, C) * torch.sigmoid(s.float()).half().float().view(N, 1, C)).half()
    assert rel_l2(w_n, want_w) < 1e-3
    y = ops.conv1x1_wbatch(cl(x), w_n, b.to(DEV), None if r is None else cl(r), 0)
    assert ops.last_status() == 0
    close(y, ref, 2e-3)
    # and it is exactly the plain convolution of each image with that image's weights
    for n in (0, N - 1):
        one = ops.conv_fused(cl(x[n:n + 1]), cl(w_n[n].view(K, C, 1, 1)), b.to(DEV), None if r is None else cl(r[n:n + 1]))
        assert torch.equal(one, y[n:n + 1])


@pytest.mark.parametrize("shape", [(2, 96, 14, 14), (2, 192, 9, 7), (1, 384, 5, 5), (3, 768, 7, 7), (2, 8, 3, 3),
                                   (2, 1536, 2, 2), (5, 768, 1, 1)])
def test_layernorm_matches_oracle(shape):
    x, w, b = gen(shape, 1), (gen((shape[1],), 2, 0.2) + 1).half(), gen((shape[1],), 3, 0.1)
    y = ops.layernorm_cl(cl(x), w.to(DEV), b.to(DEV), 1e-6)
    close(y, R.layernorm_cl_ref(x, w, b, 1e-6), 2e-3)


def test_layernorm_idempotent_on_normalised_rows():
    # size-independent property at a BASELINE-sized tensor: LN(LN(x)) == LN(x) for unit gamma, zero beta
    x = cl(gen((64, 96, 56, 56), 1))
    one, zero = torch.ones(96, dtype=torch.float16, device=DEV), torch.zeros(96, dtype=torch.float16, device=DEV)
    y1 = ops.layernorm_cl(x, one, zero, 1e-6)
    y2 = ops.layernorm_cl(y1, one, zero, 1e-6)
    assert rel_l2(y2, y1) < 2e-3


def test_input_and_elementwise_ops_match_oracle():
    x32 = torch.randn(2, 3, 17, 19, generator=torch.Generator().manual_seed(1))
    assert torch.equal(ops.input_nhwc8(x32.to(DEV)).cpu(), R.input_nhwc8_ref(x32))
    y, b, r = gen((2, 24, 6, 7), 1), gen((24,), 2), gen((2, 24, 6, 7), 3)
    yd = cl(y).clone(memory_format=torch.channels_last)
    close(ops.bias_act_(yd, b.to(DEV), cl(r), True), R.bias_act_ref(y, b, r, True))
    sc, sh = torch.rand(24) + 0.5, torch.randn(24) * 0.1
    close(ops.affine_act(cl(y), sc.to(DEV), sh.to(DEV), 1), R.affine_act_ref(y, sc, sh, 1))
    close(ops.add_act(cl(y), cl(r), 1), R.add_act_ref(y, r, 1))


@pytest.mark.parametrize("case", [(2, 19, 9, 13, 2), (1, 21, 5, 7, 4), (2, 24, 11, 6, 8), (1, 19, 3, 5, 16), (3, 8, 1, 1, 8),
                                  (1, 150, 6, 1, 4)])
def test_up_argmax_power_of_two_factors(case):
    # upsample by 2 / 4 / 8 / 16 without corner alignment: one thread per group of output pixels between two source
    # columns (vertical lerp first); against the oracle, and with duplicated channels the first maximum must win
    N, classes, h, w, sf = case
    C = (classes + 7) // 8 * 8
    x = gen((N, C, h, w), 90 + sf)
    am = ops.up_argmax(cl(x), h * sf, w * sf, False, num_classes=classes).cpu()
    ref = R.up_argmax_ref(x, h * sf, w * sf, False, num_classes=classes)
    assert am.dtype == torch.int32 and am.shape == ref.shape
    assert (am == ref).float().mean() >= 0.999
    assert int(am.max()) < classes
    if classes >= 4:
        x2 = x.clone()
        x2[:, 3] = x2[:, 1]                    # channel 3 ties with channel 1 everywhere: 3 must never be reported
        am2 = ops.up_argmax(cl(x2), h * sf, w * sf, False, num_classes=classes).cpu()
        assert not bool((am2 == 3).any())


@pytest.mark.parametrize("align", [False, True])
def test_bilinear_and_up_argmax_match_oracle(align):
    x = gen((2, 256, 1, 1), 1)
    close(ops.upsample_bilinear(cl(x), 8, 16, align=align), R.bilinear_ref(x, 8, 16, align))
    x = gen((2, 24, 9, 13), 2)
    close(ops.upsample_bilinear(cl(x), 33, 41, align=align), R.bilinear_ref(x, 33, 41, align))
    base = gen((2, 24, 33, 41), 3)
    close(ops.upsample_bilinear(cl(x), 33, 41, align=align, base=cl(base), relu=True),
          R.bilinear_ref(x, 33, 41, align, base=base, relu=True))
    am = ops.up_argmax(cl(x), 72, 104, align, num_classes=19).cpu()
    ref = R.up_argmax_ref(x, 72, 104, align, num_classes=19)
    assert am.dtype == torch.int32 and am.shape == ref.shape
    # near-ties between channels may resolve differently where the fp32 lerp is contracted into FMAs
    assert (am == ref).float().mean() >= 0.999


def _random_misc_cases(n, seed):
    import random
    rng = random.Random(seed)
    return [(rng.randint(1, 4), 8 * rng.randint(1, 60), rng.randint(1, 33), rng.randint(1, 33), rng.choice([2, 3, 3, 5]),
             rng.choice([1, 2, 2, 3]), rng.random() < 0.5, rng.random() < 0.5, rng.randint(1, 70), rng.randint(1, 70),
             rng.random() < 0.5) for _ in range(n)]


@pytest.mark.parametrize("case", _random_misc_cases(20, 5))
def test_pools_layernorm_resize_random_shapes(case):
    # seeded random shapes for the bandwidth-bound operators: max / average pool (both divisor rules, ceil mode),
    # channels-last LayerNorm, bilinear resize and the fused upsample + argmax, each against the oracle
    N, C, H, W, k, st, ceil, cip, OH, OW, align = case
    x = gen((N, C, H, W), 17)
    pad = (k // 2) if H + 2 * (k // 2) >= k and W + 2 * (k // 2) >= k else 0
    if H + 2 * pad >= k and W + 2 * pad >= k:
        assert torch.equal(ops.maxpool(cl(x), k, st, pad, ceil).cpu().float(), R.maxpool_ref(x, k, st, pad, ceil).float())
        close(ops.avgpool(cl(x), k, st, pad, cip, ceil=ceil), R.avgpool_ref(x, k, st, pad, ceil, cip))
    g, b = gen((C,), 18, 0.5) + 1.0, gen((C,), 19, 0.2)
    close(ops.layernorm_cl(cl(x), g.to(DEV), b.to(DEV), 1e-6), R.layernorm_cl_ref(x, g, b, 1e-6), 2e-3)
    close(ops.upsample_bilinear(cl(x), OH, OW, align=align), R.bilinear_ref(x, OH, OW, align))
    am = ops.up_argmax(cl(x), OH, OW, align, num_classes=C).cpu()
    assert (am == R.up_argmax_ref(x, OH, OW, align, num_classes=C)).float().mean() >= 0.999
    assert ops.last_status() == 0


def _random_group_cases(n, seed):
    import random
    rng = random.Random(seed)
    return [(rng.randint(1, 4), rng.randint(3, 30), rng.randint(3, 30), rng.randint(2, 12), 8 * rng.randint(1, 4),
             8 * rng.randint(1, 4), rng.choice([1, 3, 3]), rng.choice([1, 1, 2]), rng.choice([0, 1, 3])) for _ in range(n)]


@pytest.mark.parametrize("case", _random_group_cases(16, 11))
def test_gconv2_random_shapes(case):
    # seeded random grouped convolutions (2-12 groups of 8-32 channels on either side) against the oracle
    N, H, W, G, cg, kg, Rr, stride, act = case
    C, K, pad = G * cg, G * kg, Rr // 2
    x, w, b = gen((N, C, H, W), 21), gen((K, cg, Rr, Rr), 22, 1.0 / (cg * Rr * Rr) ** 0.5), gen((K,), 23, 0.1)
    y = ops.gconv2(cl(x), cl(w), b.to(DEV), (stride, stride), (pad, pad), G, act)
    assert ops.last_status() == 0
    close(y, R.gconv2_ref(x, w, b, (stride, stride), (pad, pad), G, act))
