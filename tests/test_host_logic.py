"""Host-side logic that needs no GPU: folding arithmetic, layout helpers, registries, compiled-module construction."""
import pytest
import torch
from torch import nn

from fast_vision_models_b200 import fold, ops
from fast_vision_models_b200.classification import zoo
from fast_vision_models_b200.weights import seeded_init, seeded_input
from oracle import models_ref, ops_ref


def test_fold_conv_bn_matches_unfolded_fp32():
    torch.manual_seed(0)
    conv = nn.Conv2d(8, 16, 3, padding=1, bias=True)
    bn = nn.BatchNorm2d(16)
    seeded_init(nn.Sequential(conv, bn), seed=3)
    x = torch.randn(2, 8, 9, 9)
    ref = bn.eval()(conv(x))
    w, b = fold.fold_conv_bn(conv, bn)
    y = torch.nn.functional.conv2d(x, w, b, padding=1)
    assert (y - ref).abs().max() <= 1e-4 * (ref.abs().max() + 1e-6)   # the reference's own fold check is 1e-3
    wr, br = models_ref.fold_bn_ref(conv, bn)
    assert torch.equal(wr, w.half()) and torch.equal(br, b.half())    # product and oracle fold identically


def test_layer_scale_fold_and_padding():
    w = torch.randn(6, 4)
    b = torch.randn(6)
    g = torch.rand(6)
    wf, bf = fold.fold_layer_scale(w, b, g)
    assert torch.allclose(wf, w * g[:, None]) and torch.allclose(bf, b * g)
    w4 = torch.randn(5, 3, 2, 2)
    assert fold.pad_in_channels(w4, 8).shape == (5, 8, 2, 2)
    assert fold.pad_in_channels(w4, 8)[:, 3:].abs().sum() == 0
    wo, bo = fold.pad_out_channels(w4, torch.ones(5), 8)
    assert wo.shape[0] == 8 and bo[5:].abs().sum() == 0
    assert fold.dw_to_rsc_half(torch.randn(16, 1, 3, 5)).shape == (3, 5, 16)


@pytest.mark.parametrize("L,k,s,p,ceil", [(112, 3, 2, 1, False), (7, 2, 2, 0, True), (8, 3, 2, 0, True),
                                          (5, 3, 2, 1, True), (13, 3, 3, 1, True)])
def test_pool_output_rule_matches_torch(L, k, s, p, ceil):
    x = torch.zeros(1, 1, L, L)
    want = torch.nn.functional.max_pool2d(x, k, s, p, ceil_mode=ceil).shape[-1]
    assert ops._pool_out(L, k, s, p, ceil) == want
    assert ops_ref.pool_out_ref(L, k, s, p, ceil) == want


def test_registry_and_aliases():
    assert zoo.ALIASES["cuda-kernels"] == "opt" and zoo.ALIASES["b200"] == "opt" and zoo.ALIASES["upstream"] == "base"
    assert {"resnet50", "efficientnet_b4", "convnext_tiny"} <= set(zoo.names())
    with pytest.raises(KeyError):
        zoo.load("vit_b16", "b200", device="cpu")


def test_compiled_modules_build_on_cpu_and_refuse_to_run_there():
    m = zoo.load("resnet50", "b200", device="cpu")
    assert m.input_size == (3, 224, 224)
    n_convs = sum(1 for mod in m.model.modules() if type(mod).__name__ == "FusedConv")
    assert n_convs == 54          # 53 folded conv+BN pairs + the FC head as a GEMM (reference graph: 39 + 14 + Linear)
    with pytest.raises(ops.FvmError):
        m.model(torch.zeros(1, 3, 64, 64))


def test_seeded_init_is_deterministic():
    a = zoo.build_upstream("resnet18", seed=1)
    b = zoo.build_upstream("resnet18", seed=1)
    for pa, pb in zip(a.state_dict().values(), b.state_dict().values()):
        assert torch.equal(pa, pb)
    assert torch.equal(seeded_input((1, 3, 8, 8), 0), seeded_input((1, 3, 8, 8), 0))


def test_bilinear_oracle_matches_torch_interpolate():
    x = torch.randn(2, 8, 5, 7).half()
    for align in (False, True):
        y = ops_ref.bilinear_ref(x, 11, 13, align=align).float()
        ref = torch.nn.functional.interpolate(x.float(), size=(11, 13), mode="bilinear", align_corners=align)
        assert (y - ref).abs().max() < 2e-3
    am = ops_ref.up_argmax_ref(x, 20, 28)
    ref = torch.nn.functional.interpolate(x.float(), size=(20, 28), mode="bilinear", align_corners=False).argmax(1)
    assert (am.long() == ref).float().mean() > 0.999


def test_stem_entry_points_refuse_cpu_tensors_and_opbench_parses():
    # the split-input stem has no CPU path either: it raises instead of falling back
    with pytest.raises(ops.FvmError):
        ops.input_nhwc8_split(torch.zeros(1, 3, 8, 8))
    with pytest.raises(ops.FvmError):
        ops.stem_conv_s2(torch.zeros(1, 8, 2, 4, 8, dtype=torch.float16), torch.zeros(8, 8, 3, 3, dtype=torch.float16),
                         None, (1, 1), 0)
    import importlib
    mod = importlib.import_module("fast_vision_models_b200.opbench")
    assert callable(mod.main)


def test_torch_ops_registration_defines_the_reference_schemas():
    from fast_vision_models_b200 import torch_ops
    done = torch_ops.register()
    assert torch_ops.register() is done                     # idempotent
    assert set(done) == {"clf", "clfr3", "clfmb", "segx"}
    want = {
        "clf::conv_fused": "clf::conv_fused(Tensor x, Tensor w, Tensor? bias, Tensor? res, int[] padding, int[] stride, int act, int cfg=-1) -> Tensor",
        "clf::avgpool": "clf::avgpool(Tensor x, int[] k, int[] stride, int[] pad, bool count_include_pad=True) -> Tensor",
        "clfr3::pw": "clfr3::pw(Tensor x, Tensor w, Tensor? bias, Tensor? res, int act, int force=0) -> Tensor",
        "clfr3::pw_into": "clfr3::pw_into(Tensor x, Tensor w, Tensor? bias, Tensor? res, int act, Tensor(a!) out, int force=0) -> ()",
        "segx::dwconv": "segx::dwconv(Tensor x, Tensor wt, Tensor? bias, int kh, int kw, int[] stride, int[] padding, int[] dilation, int act) -> Tensor",
        "segx::up_argmax": "segx::up_argmax(Tensor s, int H, int W, bool align) -> Tensor",
    }
    for qual, schema in want.items():
        ns, name = qual.split("::")
        assert str(getattr(getattr(torch.ops, ns), name).default._schema) == schema
    # shapes under fake (meta) tensors; only the CUDA key has a kernel, so a CPU tensor raises instead of falling back
    x = torch.empty(2, 64, 8, 8, dtype=torch.float16, device="meta")
    w = torch.empty(128, 64, 3, 3, dtype=torch.float16, device="meta")
    assert torch.ops.clf.conv_fused(x, w, None, None, [1, 1], [2, 2], 1).shape == (2, 128, 4, 4)
    assert torch.ops.clfr3.conv_tc(x, w, None, [2, 2], [1, 1], 1).shape == (2, 128, 4, 4)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.clfr3.se_scale(torch.zeros(1, 8, 2, 2, dtype=torch.float16), torch.zeros(1, 8, 1, 1, dtype=torch.float16))


def test_op_signatures_keep_the_reference_argument_order():
    import inspect
    assert list(inspect.signature(ops.avgpool).parameters)[:5] == ["x", "k", "stride", "pad", "count_include_pad"]
    assert list(inspect.signature(ops.pw).parameters) == ["x", "w", "bias", "res", "act", "force"]
    assert list(inspect.signature(ops.pw_into).parameters) == ["x", "w", "bias", "res", "act", "out", "force"]
    assert list(inspect.signature(ops.conv_tc).parameters) == ["x", "w", "bias", "stride", "pad", "act", "cfg"]
    assert list(inspect.signature(ops.segx_dwconv).parameters) == ["x", "wt", "bias", "kh", "kw", "stride", "padding", "dilation", "act"]


def test_generic_graph_pass_rewrites_other_architectures():
    import torchvision
    from fast_vision_models_b200.classification.fused import fuse_graph
    net = fuse_graph(torchvision.models.resnet18(weights=None).eval())
    assert net.gm.fvm_stats["conv_fused"] == 20 and net.gm.fvm_stats["stem_pad"] == 1 and net.gm.fvm_stats["left_to_aten"] == 0
    targets = [n.target for n in net.gm.graph.nodes if n.op == "call_function"]
    assert targets.count(torch.ops.clf.conv_fused) == 20 and torch.ops.clf.maxpool in targets
    # residual add and ReLU ride in the conv's epilogue: no add is left in the graph
    import operator
    assert operator.iadd not in targets and operator.add not in targets
    net = fuse_graph(torchvision.models.mobilenet_v2(weights=None).eval())
    assert net.gm.fvm_stats["dwconv"] == 17 and net.gm.fvm_stats["conv_fused"] == 35
    with pytest.raises(ops.FvmError):
        net(torch.zeros(1, 3, 32, 32))           # no CPU path behind the graph either


def test_loader_never_loads_a_stale_library(tmp_path, monkeypatch):
    from fast_vision_models_b200 import _lib
    fake = tmp_path / "libfvm_b200.so"
    fake.write_bytes(b"not a library")
    (tmp_path / "libfvm_b200.so.sha1").write_text("0" * 40)        # stamp of other sources
    monkeypatch.setattr(_lib, "_HERE", str(tmp_path))
    monkeypatch.setattr(_lib, "LIB_PATH", str(fake))
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.delenv("FVM_CACHE", raising=False)

    def no_nvcc():
        raise _lib.NvccMissing("nvcc not found")
    monkeypatch.setattr(_lib, "nvcc_path", no_nvcc)
    with pytest.raises(RuntimeError, match="stale library is never loaded"):
        _lib.load()
    # a compile error is never swallowed either
    monkeypatch.setattr(_lib, "nvcc_path", lambda: "/bin/false")
    with pytest.raises(RuntimeError, match="nvcc failed"):
        _lib.load()
    assert fake.read_bytes() == b"not a library"                   # the failed build left the old file alone


def test_loader_honours_the_cache_directory(tmp_path, monkeypatch):
    from fast_vision_models_b200 import _lib
    want = _lib.source_hash()
    monkeypatch.setenv("FVM_CACHE", str(tmp_path))
    path, stamp = _lib.lib_location(want)
    assert path == str(tmp_path / "fvm_b200" / f"libfvm_b200-{want[:16]}.so") and stamp is None
    monkeypatch.delenv("FVM_CACHE")
    path, stamp = _lib.lib_location(want)
    assert path == _lib.LIB_PATH and stamp == _lib.LIB_PATH + ".sha1"     # writable package directory: in-tree
    monkeypatch.setattr(_lib.os, "access", lambda p, mode: False)          # a read-only install
    monkeypatch.setattr(_lib, "_stamp_of", lambda p: "0" * 40)
    path, stamp = _lib.lib_location(want)
    assert ".cache/fvm_b200/libfvm_b200-" in path and stamp is None
