"""Builds (nvcc, sm_100a) and loads libfvm_b200.so, the C-ABI library behind every op of this package.

Stands where the reference's JIT loader sits (fast_vision_models/_build.py:71-93): sources are compiled once, the
result is reused while a hash of the sources matches. Unlike the reference there is no per-user cache: the library is
built in-tree next to this file so that it travels with the package. There is no fallback: if the library cannot be
built or loaded, importing an op raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(_HERE), "include")
LIB_PATH = os.path.join(_HERE, "libfvm_b200.so")
_STAMP = LIB_PATH + ".sha1"
SOURCES = ["abi.cu", "conv_tcgen05.cu", "bandwidth.cu", "dwconv.cu"]
HEADERS = ["fvm_internal.h", "ptx_sm100.cuh"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]

_lock = threading.Lock()
_lib = None


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def source_hash() -> str:
    h = hashlib.sha1()
    for name in _sources() + HEADERS:
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    with open(os.path.join(INCLUDE, "fvm_b200.h"), "rb") as f:
        h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def nvcc_path() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("fvm_b200: nvcc not found (set CUDA_HOME); the CUDA library cannot be built")
    return found


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library for sm_100a if the sources changed. Returns the path of the shared object."""
    want = source_hash()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(_STAMP):
        with open(_STAMP) as f:
            if f.read().strip() == want:
                return LIB_PATH
    cmd = [nvcc_path()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH] + _sources()
    proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("fvm_b200: nvcc failed\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stdout + proc.stderr)
    with open(_STAMP, "w") as f:
        f.write(want)
    return LIB_PATH


def load() -> ctypes.CDLL:
    """Load the library (building it first when nvcc is present and the sources changed). Raises if impossible."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            build()
        except RuntimeError:
            if not os.path.exists(LIB_PATH):
                raise
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("fvm_b200: libfvm_b200.so is missing and could not be built; there is no fallback path")
        lib = ctypes.CDLL(LIB_PATH)
        _declare(lib)
        _lib = lib
        return lib


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float


def _declare(lib: ctypes.CDLL) -> None:
    sig = {
        "fvm_init": ([], _I),
        "fvm_query": ([_I], _L),
        "fvm_last_status": ([ctypes.POINTER(_I)], _I),
        "fvm_conv2d_f16": ([_P] * 6 + [_I] * 13 + [_L] * 3 + [_I, _P], _I),
        "fvm_conv2d_f16_tile": ([_P] * 6 + [_I] * 13 + [_L] * 3 + [_I, _I, _P], _I),
        "fvm_conv2d_f16_pad": ([_P] * 6 + [_I] * 13 + [_L] * 3 + [_I, _I, _I, _I, _P], _I),
        "fvm_dwconv_f16": ([_P] * 5 + [_I] * 12 + [_L] * 2 + [_I, _P], _I),
        "fvm_maxpool_f16": ([_P] * 2 + [_I] * 12 + [_P], _I),
        "fvm_avgpool_f16": ([_P] * 2 + [_I] * 13 + [_P], _I),
        "fvm_gap_scratch_floats": ([_I] * 3, _L),
        "fvm_global_avgpool_f16": ([_P] * 3 + [_I] * 3 + [_L, _P], _I),
        "fvm_global_avgpool_f16_noalloc": ([_P] * 2 + [_I] * 3 + [_L, _P], _I),
        "fvm_global_avgpool_f16_noalloc_max_floats": ([], _L),
        "fvm_se_gate_f16": ([_P] * 6 + [_I] * 4 + [_F, _P], _I),
        "fvm_se_scale_f16": ([_P] * 3 + [_I] * 3 + [_P], _I),
        "fvm_layernorm_cl_f16": ([_P] * 4 + [_L, _I, _F, _L, _L, _P], _I),
        "fvm_input_nhwc8_f32": ([_P] * 2 + [_I] * 4 + [_P], _I),
        "fvm_input_nhwc8_split_f32": ([_P] * 2 + [_I] * 4 + [_P], _I),
        "fvm_stem_conv_s2_f16": ([_P] * 4 + [_I] * 8 + [_L, _I, _P], _I),
        "fvm_bias_act_f16": ([_P] * 3 + [_L, _I, _I, _P], _I),
        "fvm_affine_act_f16": ([_P] * 4 + [_L, _I, _L, _L, _I, _P], _I),
        "fvm_add_act_f16": ([_P] * 3 + [_L, _I, _P], _I),
        "fvm_bilinear_f16": ([_P] * 3 + [_I] * 7 + [_F, _F, _I, _L, _L, _P], _I),
        "fvm_up_argmax_f16": ([_P] * 2 + [_I] * 4 + [_L, _I, _I, _I, _P], _I),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    for name, (argtypes, restype) in OPTIONAL_SIGNATURES.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype


OPTIONAL_SIGNATURES: dict = {}

EXPORTED = ["fvm_init", "fvm_query", "fvm_last_status", "fvm_conv2d_f16", "fvm_conv2d_f16_tile", "fvm_conv2d_f16_pad", "fvm_dwconv_f16", "fvm_maxpool_f16",
            "fvm_avgpool_f16", "fvm_gap_scratch_floats", "fvm_global_avgpool_f16", "fvm_global_avgpool_f16_noalloc",
            "fvm_global_avgpool_f16_noalloc_max_floats", "fvm_se_gate_f16",
            "fvm_se_scale_f16", "fvm_layernorm_cl_f16", "fvm_input_nhwc8_f32", "fvm_input_nhwc8_split_f32",
            "fvm_stem_conv_s2_f16", "fvm_bias_act_f16",
            "fvm_affine_act_f16", "fvm_add_act_f16", "fvm_bilinear_f16", "fvm_up_argmax_f16"]
