"""CPU-side checks of the C-ABI library: it builds for sm_100a, loads without a GPU, exports every declared symbol."""
import ctypes
import os
import re

import torch

from fast_vision_models_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    with open(os.path.join(ROOT, "include", "fvm_b200.h")) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(fvm_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_hot_path_entry_points():
    syms = declared_symbols()
    for want in ("fvm_init", "fvm_conv2d_f16", "fvm_dwconv_f16", "fvm_global_avgpool_f16", "fvm_se_gate_f16",
                 "fvm_se_scale_f16", "fvm_layernorm_cl_f16", "fvm_input_nhwc8_f32", "fvm_maxpool_f16",
                 "fvm_bilinear_f16", "fvm_up_argmax_f16"):
        assert want in syms


def test_library_builds_and_exports_every_declared_symbol():
    path = _lib.build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    for name in declared_symbols():
        assert hasattr(lib, name), name
    for name in _lib.EXPORTED:
        assert hasattr(lib, name), name


def test_version_query_needs_no_gpu():
    lib = _lib.load()
    assert lib.fvm_query(0) >= 100


def test_no_gpu_means_loud_failure_not_fallback():
    if torch.cuda.is_available():
        return
    from fast_vision_models_b200 import ops
    x = torch.zeros(1, 8, 4, 4, dtype=torch.float16)
    w = torch.zeros(8, 8, 1, 1, dtype=torch.float16)
    try:
        ops.conv_fused(x, w)
    except ops.FvmError:
        return
    raise AssertionError("conv_fused on a CPU tensor must raise")
