"""Builds (nvcc, sm_100a) and loads libfvm_b200.so, the C-ABI library behind every op of this package.

Stands where the reference's JIT loader sits (fast_vision_models/_build.py:71-93): sources are compiled once and the
result is reused while a hash of the sources (and compiler flags) matches. Where the result lives:
  * by default in-tree, next to this file (`libfvm_b200.so` + a `.sha1` stamp), so that it travels with the package;
  * in `$FVM_CACHE/fvm_b200/` when FVM_CACHE is set -- the reference's variable (_build.py:23-28) -- or in
    `~/.cache/fvm_b200/` when the package directory is read-only (a site-packages install); files there carry the
    source hash in their name, so several versions coexist.
A library whose stamp does not match the sources is never loaded: if it cannot be rebuilt (no nvcc, or a compile
error) loading raises with both hashes. Concurrent builders (one process per GPU under torchrun) serialise on a file
lock and the result is moved into place atomically. There is no fallback: no library, no ops.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(_HERE), "include")
LIB_NAME = "libfvm_b200.so"
LIB_PATH = os.path.join(_HERE, LIB_NAME)          # the in-tree location
SOURCES = ["abi.cu", "conv_tcgen05.cu", "bandwidth.cu", "dwconv.cu"]
HEADERS = ["fvm_internal.h", "ptx_sm100.cuh"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]

_lock = threading.Lock()
_lib = None


class NvccMissing(RuntimeError):
    pass


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
        raise NvccMissing("fvm_b200: nvcc not found (set CUDA_HOME); the CUDA library cannot be built")
    return found


def lib_location(want: str):
    """(path of the shared object, path of its stamp file or None) for sources hashing to `want`."""
    cache = os.environ.get("FVM_CACHE")
    if cache:
        d = os.path.join(cache, "fvm_b200")
    elif os.access(_HERE, os.W_OK):
        return LIB_PATH, LIB_PATH + ".sha1"
    elif os.path.exists(LIB_PATH) and _stamp_of(LIB_PATH + ".sha1") == want:
        return LIB_PATH, LIB_PATH + ".sha1"         # read-only install that ships a current library
    else:
        d = os.path.join(os.path.expanduser("~"), ".cache", "fvm_b200")
    return os.path.join(d, f"libfvm_b200-{want[:16]}.so"), None


def _stamp_of(stamp_path: str):
    try:
        with open(stamp_path) as f:
            return f.read().strip()
    except OSError:
        return None


def _is_current(path: str, stamp, want: str) -> bool:
    if not os.path.exists(path):
        return False
    return True if stamp is None else _stamp_of(stamp) == want      # cache files carry the hash in their name


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library for sm_100a unless a current one exists. Returns the path of the shared object."""
    want = source_hash()
    path, stamp = lib_location(want)
    if not force and _is_current(path, stamp, want):
        return path
    os.makedirs(os.path.dirname(path), exist_ok=True)
    nvcc = nvcc_path()
    with open(path + ".lock", "w") as lockf:
        fcntl.flock(lockf, fcntl.LOCK_EX)               # one builder at a time; the others find the result afterwards
        try:
            if not force and _is_current(path, stamp, want):
                return path
            tmp = f"{path}.tmp{os.getpid()}"
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", tmp] + _sources()
            proc = subprocess.run(cmd, cwd=CSRC, capture_output=True, text=True)
            if proc.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("fvm_b200: nvcc failed\n" + proc.stdout + proc.stderr)
            if verbose:
                print(proc.stdout + proc.stderr)
            if stamp is not None and os.path.exists(stamp):
                os.remove(stamp)                         # never leave a new stamp beside an old library or vice versa
            os.replace(tmp, path)
            if stamp is not None:
                with open(stamp + ".tmp", "w") as f:
                    f.write(want)
                os.replace(stamp + ".tmp", stamp)
        finally:
            fcntl.flock(lockf, fcntl.LOCK_UN)
    return path


def load() -> ctypes.CDLL:
    """Load the library, building it first when the sources changed. Raises if no current library can be had."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        want = source_hash()
        path, stamp = lib_location(want)
        if not _is_current(path, stamp, want):
            try:
                path = build()
            except NvccMissing as e:
                have = _stamp_of(stamp) if stamp else None
                raise RuntimeError(f"fvm_b200: no library matches the sources (sources {want[:12]}, library "
                                   f"{have[:12] if have else 'absent'}) and it cannot be rebuilt: {e}. A stale library "
                                   f"is never loaded; there is no fallback path") from e
        lib = ctypes.CDLL(path)
        _declare(lib)
        _lib = lib
        return lib


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float


class ChainLayer(ctypes.Structure):
    """fvm_chain_layer of include/fvm_b200.h: one convolution of a chain launch."""
    _fields_ = ([(n, _P) for n in ("x", "w", "bias", "res", "scale", "y")] +
                [(n, _I) for n in ("N", "H", "W", "C", "K", "R", "S", "ph", "pw", "sh", "sw", "dh", "dw")] +
                [(n, _L) for n in ("ldx", "ldy", "ldr")] + [("act", _I), ("tile_n", _I)])


def _declare(lib: ctypes.CDLL) -> None:
    sig = {
        "fvm_init": ([], _I),
        "fvm_query": ([_I], _L),
        "fvm_last_status": ([ctypes.POINTER(_I)], _I),
        "fvm_selftest_wait_expiry": ([_I, _P], _I),
        "fvm_conv2d_f16": ([_P] * 6 + [_I] * 13 + [_L] * 3 + [_I, _P], _I),
        "fvm_conv2d_f16_tile": ([_P] * 6 + [_I] * 13 + [_L] * 3 + [_I, _I, _P], _I),
        "fvm_conv2d_f16_pad": ([_P] * 6 + [_I] * 13 + [_L] * 3 + [_I, _I, _I, _I, _P], _I),
        "fvm_conv_chain_f16": ([ctypes.POINTER(ChainLayer), _I, _P], _I),
        "fvm_conv_dual_f16": ([_P] * 8 + [_L] + [_I] * 3 + [_L] * 4 + [_I, _I, _P], _I),
        "fvm_gconv2d_f16": ([_P] * 5 + [_I] * 13 + [_L] * 3 + [_I, _I, _I, _P], _I),
        "fvm_dwconv_f16": ([_P] * 5 + [_I] * 12 + [_L] * 2 + [_I, _P], _I),
        "fvm_dwconv_pool_slots": ([_I] * 12, _I),
        "fvm_se_gate_pooled_f16": ([_P, _I] + [_P] * 5 + [_I] * 4 + [_F, _P], _I),
        "fvm_maxpool_f16": ([_P] * 2 + [_I] * 12 + [_P], _I),
        "fvm_avgpool_f16": ([_P] * 2 + [_I] * 13 + [_P], _I),
        "fvm_gap_scratch_floats": ([_I] * 3, _L),
        "fvm_global_avgpool_f16": ([_P] * 3 + [_I] * 3 + [_L, _P], _I),
        "fvm_global_avgpool_f16_noalloc": ([_P] * 2 + [_I] * 3 + [_L, _P], _I),
        "fvm_global_avgpool_f16_noalloc_max_floats": ([], _L),
        "fvm_se_gate_f16": ([_P] * 6 + [_I] * 4 + [_F, _P], _I),
        "fvm_se_scale_f16": ([_P] * 3 + [_I] * 3 + [_P], _I),
        "fvm_gate_weights_f16": ([_P] * 3 + [_I] * 3 + [_P], _I),
        "fvm_conv1x1_wbatch_f16": ([_P] * 5 + [_I] * 5 + [_L] * 3 + [_I, _P], _I),
        "fvm_layernorm_cl_f16": ([_P] * 4 + [_L, _I, _F, _L, _L, _P], _I),
        "fvm_input_nhwc8_f32": ([_P] * 2 + [_I] * 4 + [_P], _I),
        "fvm_input_nhwc8_split_f32": ([_P] * 2 + [_I] * 4 + [_P], _I),
        "fvm_input_nhwc8_f16": ([_P] * 2 + [_I] * 4 + [_P], _I),
        "fvm_input_nhwc8_split_f16": ([_P] * 2 + [_I] * 4 + [_P], _I),
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

EXPORTED = ["fvm_init", "fvm_query", "fvm_last_status", "fvm_selftest_wait_expiry", "fvm_conv2d_f16", "fvm_conv2d_f16_tile", "fvm_conv2d_f16_pad", "fvm_conv_chain_f16", "fvm_conv_dual_f16", "fvm_gconv2d_f16", "fvm_dwconv_f16", "fvm_dwconv_pool_slots", "fvm_se_gate_pooled_f16", "fvm_maxpool_f16",
            "fvm_avgpool_f16", "fvm_gap_scratch_floats", "fvm_global_avgpool_f16", "fvm_global_avgpool_f16_noalloc",
            "fvm_global_avgpool_f16_noalloc_max_floats", "fvm_se_gate_f16",
            "fvm_se_scale_f16", "fvm_gate_weights_f16", "fvm_conv1x1_wbatch_f16", "fvm_layernorm_cl_f16", "fvm_input_nhwc8_f32", "fvm_input_nhwc8_split_f32",
            "fvm_input_nhwc8_f16", "fvm_input_nhwc8_split_f16",
            "fvm_stem_conv_s2_f16", "fvm_bias_act_f16",
            "fvm_affine_act_f16", "fvm_add_act_f16", "fvm_bilinear_f16", "fvm_up_argmax_f16"]
