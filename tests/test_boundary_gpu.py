"""The operator boundary on the GPU: the `torch.ops` registrations (reference schemas), the thin schema aliases, the
generic graph pass, fp16 image input, argument refusal before launch, and the bounded-wait fault path."""
import ctypes

import pytest
import torch

from conftest import rel_l2
from fast_vision_models_b200 import ops, torch_ops
from oracle import ops_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def gen(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).half()


def cl(t):
    return t.to(DEV).contiguous(memory_format=torch.channels_last)


def close(y, ref, tol=1e-3):
    y, ref = y.float().cpu(), ref.float().cpu()
    assert y.shape == ref.shape, (y.shape, ref.shape)
    assert torch.isfinite(y).all()
    assert rel_l2(y, ref) < tol, rel_l2(y, ref)


def test_torch_ops_follow_the_reference_schemas_and_match_the_oracle():
    torch_ops.register()
    x, w, b, r = gen((2, 64, 14, 14), 1), gen((128, 64, 3, 3), 2, 0.05), gen((128,), 3, 0.1), gen((2, 128, 14, 14), 4)
    # clf::conv_fused(x, w, bias?, res?, padding, stride, act, cfg=-1)
    y = torch.ops.clf.conv_fused(cl(x), cl(w), b.to(DEV), cl(r), [1, 1], [1, 1], 1)
    close(y, R.conv_fused_ref(x, w, b, r, (1, 1), (1, 1), 1))
    out = ops.empty_nhwc(2, 128, 14, 14, DEV)
    assert torch.ops.clf.conv_fused_into(cl(x), cl(w), b.to(DEV), None, [1, 1], [1, 1], 0, out) is None
    close(out, R.conv_fused_ref(x, w, b, None, (1, 1), (1, 1), 0))
    # clfr3::pw(x, w, bias?, res?, act, force=0) and pw_into(..., out, force=0)
    w1 = gen((128, 64, 1, 1), 5, 0.05)
    close(torch.ops.clfr3.pw(cl(x), cl(w1), b.to(DEV), cl(r), 1), R.conv_fused_ref(x, w1, b, r, act=1))
    wide = torch.zeros((2, 256, 14, 14), dtype=torch.float16, device=DEV).contiguous(memory_format=torch.channels_last)
    torch.ops.clfr3.pw_into(cl(x), cl(w1), b.to(DEV), None, 1, wide[:, 128:], 0)
    close(wide[:, 128:], R.conv_fused_ref(x, w1, b, None, act=1))
    assert wide[:, :128].abs().sum() == 0
    # clfr3::conv_tc(x, w, bias?, stride, pad, act, cfg=-1): stride comes before pad
    x16, w16 = gen((2, 16, 20, 20), 6), gen((32, 16, 3, 3), 7, 0.1)
    close(torch.ops.clfr3.conv_tc(cl(x16), cl(w16), None, [2, 2], [1, 1], 1), R.conv_fused_ref(x16, w16, None, None, (1, 1), (2, 2), 1))
    # clfr3::se_scale(x, s), clf::avgpool(x, k, stride, pad, count_include_pad=True): 5th positional = count_include_pad
    s = gen((2, 64, 1, 1), 8)
    close(torch.ops.clfr3.se_scale(cl(x), s.to(DEV)), R.se_scale_ref(x, s))
    close(torch.ops.clf.avgpool(cl(x), [3, 3], [2, 2], [1, 1], False), R.avgpool_ref(x, 3, 2, 1, False, False))
    close(torch.ops.clf.avgpool(cl(x), [3, 3], [2, 2], [1, 1]), R.avgpool_ref(x, 3, 2, 1, False, True))
    assert torch.equal(torch.ops.clf.maxpool(cl(x), [3, 3], [2, 2], [1, 1], False).cpu().float(), R.maxpool_ref(x, 3, 2, 1, False).float())
    # segx::conv_fused_d(..., dilation, act), segx::dwconv(x, wt [kh*kw, C], bias?, kh, kw, stride, padding, dilation, act: 1 = GELU)
    close(torch.ops.segx.conv_fused_d(cl(x), cl(w), b.to(DEV), None, [2, 2], [1, 1], [2, 2], 1),
          R.conv_fused_ref(x, w, b, None, (2, 2), (1, 1), 1, (2, 2)))
    wt, bd = gen((9, 64), 9, 0.2), gen((64,), 10, 0.1)
    close(torch.ops.segx.dwconv(cl(x), wt.to(DEV), bd.to(DEV), 3, 3, [1, 1], [2, 2], [2, 2], 1),
          R.dwconv_ref(x, wt.view(3, 3, 64), bd, (1, 1), (2, 2), 5, (2, 2)))
    close(torch.ops.segx.dwconv8(cl(x), wt.view(3, 3, 64).to(DEV), bd.to(DEV), [1, 1], [1, 1], 3),
          R.dwconv_ref(x, wt.view(3, 3, 64), bd, (1, 1), (1, 1), 3))
    # segx::up_argmax(s [B, h, w, C], H, W, align) and the resize family
    sc = gen((2, 24, 9, 13), 11)
    am = torch.ops.segx.up_argmax(cl(sc).permute(0, 2, 3, 1), 72, 104, False).cpu()
    assert am.dtype == torch.int32 and (am == R.up_argmax_ref(sc, 72, 104, False)).float().mean() >= 0.999
    close(torch.ops.segx.upsample_bilinear(cl(sc), 33, 41, None, None, False), R.bilinear_ref(sc, 33, 41, False))
    ref_t = torch.empty((2, 24, 20, 30), dtype=torch.float16, device=DEV)
    close(torch.ops.segx.upsample_like(cl(sc), ref_t, True), R.bilinear_ref(sc, 20, 30, True))
    close(torch.ops.segx.upsample_bilinear_t(cl(sc), torch.tensor([18, 26]), False), R.bilinear_ref(sc, 18, 26, False))
    base = gen((2, 24, 18, 26), 12)
    want = R.bilinear_ref(sc, 18, 26, False, sf_h=2.0, sf_w=2.0, base=base, relu=True)
    close(torch.ops.segx.upsample_add(cl(base), cl(sc), 2.0, True), want)
    bdev = cl(base).clone(memory_format=torch.channels_last)
    assert torch.ops.segx.upsample_add_(bdev, cl(sc), 2.0, True).data_ptr() == bdev.data_ptr()
    close(bdev, want)
    yb = cl(gen((2, 24, 6, 7), 13)).clone(memory_format=torch.channels_last)
    want_b = R.bias_act_ref(yb.cpu(), gen((24,), 14), None, True)
    close(torch.ops.segx.bias_act_(yb, gen((24,), 14).to(DEV), None, True), want_b)
    # clfmb::stem_direct(x raw NCHW, w_t [R,S,C,K], bias?, stride, pad, act) and clfr3::stem_pool(..., pk, ps, pp, ceil)
    img = torch.randn(2, 3, 38, 46, generator=torch.Generator().manual_seed(15))
    wk = gen((48, 3, 3, 3), 16, 0.1)
    w_t = wk.permute(2, 3, 1, 0).contiguous().to(DEV)
    w8 = torch.zeros(48, 8, 3, 3, dtype=torch.float16)
    w8[:, :3] = wk
    want_stem = R.conv_fused_ref(R.input_nhwc8_ref(img), w8, gen((48,), 17, 0.1), None, (1, 1), (2, 2), 3)
    close(torch.ops.clfmb.stem_direct(img.to(DEV), w_t, gen((48,), 17, 0.1).to(DEV), [2, 2], [1, 1], 3), want_stem)
    got = torch.ops.clfr3.stem_pool(img.to(DEV), w_t, gen((48,), 17, 0.1).to(DEV), [2, 2], [1, 1], 3, 3, 2, 1, False)
    close(got, R.maxpool_ref(want_stem, 3, 2, 1, False), 2e-3)
    assert ops.last_status() == 0
    with pytest.raises((NotImplementedError, RuntimeError)):       # only the CUDA key is bound, as in the reference
        torch.ops.clf.conv_fused(x, w, None, None, [1, 1], [1, 1], 0)


def test_fx_graph_of_registered_ops_replays_under_cuda_graph_capture():
    import torch.fx as fx
    torch_ops.register()

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.register_buffer("w1", cl(gen((64, 64, 3, 3), 1, 0.05)))
            self.register_buffer("b1", gen((64,), 2, 0.1).to(DEV))
            self.register_buffer("w2", cl(gen((24, 64, 1, 1), 3, 0.05)))

        def forward(self, x, gate):
            y = torch.ops.clf.conv_fused(x, self.w1, self.b1, x, [1, 1], [1, 1], 1)
            y = torch.ops.clfr3.se_scale(y, gate)
            s = torch.ops.clf.conv_fused(y, self.w2, None, None, [0, 0], [1, 1], 0)
            return torch.ops.segx.up_argmax(s.permute(0, 2, 3, 1), 48, 64, False)

    gm = fx.symbolic_trace(Block())
    targets = [n.target for n in gm.graph.nodes if n.op == "call_function"]
    assert torch.ops.clf.conv_fused in targets and torch.ops.clfr3.se_scale in targets and torch.ops.segx.up_argmax in targets
    x, gate = cl(gen((2, 64, 12, 16), 4)), gen((2, 64, 1, 1), 5).to(DEV)
    eager = gm(x, gate)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        gm(x, gate)                      # warm-up on the capture stream
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=side):
            captured = gm(x, gate)
    captured.fill_(-1)
    graph.replay()
    torch.cuda.synchronize()
    assert ops.last_status() == 0
    assert torch.equal(captured, eager)
    y = R.conv_fused_ref(x.cpu(), gm.w1.cpu(), gm.b1.cpu(), x.cpu(), (1, 1), (1, 1), 1)
    y = R.se_scale_ref(y, gate.cpu())
    s = R.conv_fused_ref(y, gm.w2.cpu(), None, None, (0, 0), (1, 1), 0)
    assert (captured.cpu() == R.up_argmax_ref(s, 48, 64, False)).float().mean() >= 0.995


@pytest.mark.parametrize("name", ["resnet18", "mobilenet_v2", "densenet121", "regnet_y_400mf", "squeezenet1_1", "resnext50_32x4d"])
def test_generic_graph_pass_matches_upstream_fp32(name):
    # architectures without a hand-built compiler go through the pattern pass (conv -> [add] -> [act] chains,
    # depthwise, pools, unfoldable BatchNorm, squeeze-excite scale); what it cannot place stays on aten in fp16
    import torchvision
    from fast_vision_models_b200.classification.fast import Fast
    from fast_vision_models_b200.classification.fused import fuse_graph
    from fast_vision_models_b200.weights import seeded_init, seeded_input
    model = torchvision.models.get_model(name, weights=None).eval()
    if name != "densenet121":      # 120 concatenating layers with randomised BatchNorm statistics leave the fp16 range
        model = seeded_init(model, seed=1)          # (plain fp16 PyTorch overflows too); DenseNet keeps torchvision's init
    net = Fast(fuse_graph(model)).to(DEV)          # what optimize() builds for a family without a hand-built compiler
    stats = net.net.gm.fvm_stats
    assert stats["conv_fused"] >= 10 and stats["stem_pad"] == 1
    if name in ("regnet_y_400mf", "resnext50_32x4d"):
        assert stats.get("gconv", 0) >= 10          # grouped convolutions go to clfr3.gconv2, not to aten
    x = seeded_input((4, 3, 96, 96), seed=0).to(DEV)
    y = net(x)
    with torch.inference_mode():
        y32 = model.to(DEV)(x)
    assert ops.last_status() == 0
    from fast_vision_models_b200.classification.fast import Portable
    port = Portable(model.cpu()).to(DEV)(x)
    print(name, stats, "rel-L2 vs fp32", rel_l2(y, y32), "vs portable fp16", rel_l2(y, port), "portable vs fp32", rel_l2(port, y32))
    # fp16 through 50+ layers of a random-init network: the b200 graph must be as close to fp32 as plain fp16 PyTorch is
    assert rel_l2(y, y32) < max(1e-2, 1.5 * rel_l2(port, y32))
    assert torch.equal(net(x), y)            # graph replay


def test_fp16_image_input_matches_fp32_input_rounded():
    x32 = torch.randn(2, 3, 18, 20, generator=torch.Generator().manual_seed(1)).to(DEV)
    x16 = x32.half()
    assert torch.equal(ops.input_nhwc8(x16), ops.input_nhwc8(x16.float()))
    assert torch.equal(ops.input_nhwc8_split(x16), ops.input_nhwc8_split(x16.float()))
    assert torch.equal(ops.input_nhwc8(x16).cpu(), R.input_nhwc8_ref(x16.float().cpu()))
    from fast_vision_models_b200.classification import zoo
    from fast_vision_models_b200.weights import seeded_input
    m = zoo.load("resnet18", "b200", device=DEV, seed=1)
    x = seeded_input((2, 3, 64, 64), seed=0).to(DEV).half()
    assert torch.equal(m.model(x), m.model(x.float()))      # an fp16 batch is the fp32 batch rounded once, either way


def test_misaligned_scale_pointer_is_refused_before_launch():
    # the un-folded LayerScale vector is read as float4: a 4-byte-aligned pointer must come back as status 1 (bad
    # argument), not reach the kernel
    L = ops.lib()
    ops.init()
    x, w = cl(gen((1, 64, 4, 4), 1)), cl(gen((64, 64, 1, 1), 2))
    y = ops.empty_nhwc(1, 64, 4, 4, DEV)
    scale = torch.ones(72, dtype=torch.float32, device=DEV)
    n0 = ops.launches()
    args = [x.data_ptr(), w.data_ptr(), None, None]
    tail = [y.data_ptr(), 1, 4, 4, 64, 64, 1, 1, 0, 0, 1, 1, 1, 1, 64, 64, 0, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)]
    assert L.fvm_conv2d_f16(*args, scale.data_ptr() + 4, *tail) == 1
    assert ops.launches() == n0
    assert L.fvm_conv2d_f16(*args, scale.data_ptr(), *tail) == 0
    assert ops.last_status() == 0


def test_bounded_wait_runs_out_reports_and_leaves_the_device_usable():
    # the fault path of every kernel role: a wait with a limit on a barrier nothing arrives at gives up, the kernel
    # writes its code to the status word and returns by itself; the next launch works as before
    ops.init()
    assert ops.last_status() == 0
    ops.selftest_wait_expiry(1000)          # 1 ms
    assert ops.last_status() == 0x1FF
    assert ops.last_status() == 0            # reading clears the word
    x, w = gen((2, 64, 9, 9), 1), gen((64, 64, 3, 3), 2, 0.05)
    close(ops.conv_fused(cl(x), cl(w), None, None, (1, 1), (1, 1), 1), R.conv_fused_ref(x, w, None, None, (1, 1), (1, 1), 1))
    assert ops.last_status() == 0
    # the graph runner turns a reported fault into an exception at its next call
    from fast_vision_models_b200.runtime import GraphRunner
    runner = GraphRunner(lambda t: t * 2)
    t = torch.ones(4, device=DEV)
    runner(t)
    ops.selftest_wait_expiry(200)
    torch.cuda.synchronize()
    with pytest.raises(ops.FvmError):
        runner(t)
    assert ops.last_status() == 0


def test_two_devices_in_one_process():
    # per-device set-up (kernel attributes, status word, scratch, cluster capacity) and launches on a second GPU of the
    # same process; a tensor of a device that is not current is refused before anything is launched
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    x, w, b = gen((4, 64, 28, 28), 1), gen((128, 64, 3, 3), 2, 0.05), gen((128,), 3, 0.1)
    wd, bd = gen((64, 1, 3, 3), 4, 0.2), gen((64,), 5, 0.1)
    ref = R.conv_fused_ref(x, w, b, None, (1, 1), (1, 1), 1)
    ref_dw = R.dwconv_ref(x, wd[:, 0].permute(1, 2, 0).contiguous(), bd, (1, 1), (1, 1), 3)
    for _round in range(2):
        for d in (0, 1):
            dev = f"cuda:{d}"
            with torch.cuda.device(d):
                xd = x.to(dev).contiguous(memory_format=torch.channels_last)
                wdev = w.to(dev).contiguous(memory_format=torch.channels_last)
                y = ops.conv_fused(xd, wdev, b.to(dev), None, (1, 1), (1, 1), 1)
                close(y, ref)
                if ops.query(4) > 0:
                    yp = ops.conv_fused(xd, wdev, b.to(dev), None, (1, 1), (1, 1), 1, tile_n=(1 << 30) | 128)
                    assert torch.equal(yp, y)
                ydw = ops.dwconv(xd, wd[:, 0].permute(1, 2, 0).contiguous().to(dev), bd.to(dev), (1, 1), (1, 1), 3)
                close(ydw, ref_dw)
                assert ops.last_status() == 0
    with torch.cuda.device(0):
        with pytest.raises(ops.FvmError):
            ops.conv_fused(x.to("cuda:1").contiguous(memory_format=torch.channels_last),
                           w.to("cuda:1").contiguous(memory_format=torch.channels_last), None, None, (1, 1), (1, 1), 1)
