"""Synthetic models: named shapes from the benchmark configurations and a ctypes front end to the
GGUF writer / quantizers in csrc/synth.cpp."""
import ctypes
import os

import numpy as np

from . import _build

Q8_0, Q4_K, Q6_K, F32 = 8, 12, 14, 0
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q6_K: 256, F32: 1}
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q6_K: 210, F32: 4}

# scheme: 0 = every linear Q8_0; 1 = Q4_K with Q6_K for attn_v / ffn_down / output ("Q4_K_M-style");
#         2 = every linear Q6_K; 3 = every linear Q4_K
SHAPES = {
    "tiny": dict(hidden=256, ffn=512, n_heads=4, n_kv_heads=2, n_layers=2, vocab=512, max_pos=128, theta=10000.0),
    "tiny_mha": dict(hidden=512, ffn=768, n_heads=4, n_kv_heads=4, n_layers=2, vocab=1024, max_pos=256, theta=10000.0),
    "tinyllama-1.1b": dict(hidden=2048, ffn=5632, n_heads=32, n_kv_heads=4, n_layers=22, vocab=32000, max_pos=2048, theta=10000.0),
    "llama2-7b": dict(hidden=4096, ffn=11008, n_heads=32, n_kv_heads=32, n_layers=32, vocab=32000, max_pos=4096, theta=10000.0),
    "llama3-8b": dict(hidden=4096, ffn=14336, n_heads=32, n_kv_heads=8, n_layers=32, vocab=128256, max_pos=8192, theta=500000.0),
    "llama2-70b": dict(hidden=8192, ffn=28672, n_heads=64, n_kv_heads=8, n_layers=80, vocab=32000, max_pos=8192, theta=10000.0),
}


class _Cfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in "hidden ffn n_heads n_kv_heads n_layers vocab max_pos".split()] + [
        ("eps", ctypes.c_float), ("theta", ctypes.c_float), ("scheme", ctypes.c_int32),
        ("norm_random", ctypes.c_int32), ("seed", ctypes.c_uint64), ("sigma", ctypes.c_float)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build_synth())
        _lib.b200_synth_write_gguf.argtypes = [ctypes.c_char_p, ctypes.POINTER(_Cfg)]
        _lib.b200_synth_quantize.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        _lib.b200_synth_fill_normal.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float]
        _lib.b200_synth_fill_normal.restype = None
        _lib.b200_synth_set_threads.argtypes = [ctypes.c_int]
        _lib.b200_synth_set_threads.restype = None
        # a launcher (torchrun) may have pinned OMP_NUM_THREADS to 1 for the process: the writer uses the cores it may run on
        try:
            _lib.b200_synth_set_threads(len(os.sched_getaffinity(0)))
        except AttributeError:
            _lib.b200_synth_set_threads(os.cpu_count() or 1)
    return _lib


def write_gguf(path, shape, scheme, seed=1234, sigma=0.02, norm_random=False, eps=1e-5, embd_quant=False, **overrides):
    """Writes a synthetic model file. `shape` is a key of SHAPES or a dict with the same fields.
    embd_quant: token_embd is quantised like attn_q (what real checkpoints ship) instead of F32."""
    s = dict(SHAPES[shape]) if isinstance(shape, str) else dict(shape)
    s.update(overrides)
    cfg = _Cfg(s["hidden"], s["ffn"], s["n_heads"], s["n_kv_heads"], s["n_layers"], s["vocab"], s["max_pos"],
               eps, s["theta"], scheme, int(bool(norm_random)) | (2 if embd_quant else 0), seed, sigma)
    rc = lib().b200_synth_write_gguf(os.fsencode(path), ctypes.byref(cfg))
    if rc:
        raise RuntimeError(f"b200_synth_write_gguf failed with status {rc}")
    return path


def fill_normal(n, seed, stream=1, sigma=0.02):
    out = np.empty(n, np.float32)
    lib().b200_synth_fill_normal(out.ctypes.data, n, seed, stream, sigma)
    return out


def quantize(ggml_type, x):
    """Quantizes a float32 array (size a multiple of the block size) into packed blocks (uint8 array)."""
    x = np.ascontiguousarray(x, np.float32).ravel()
    out = np.empty(x.size // BLOCK_ELEMS[ggml_type] * BLOCK_BYTES[ggml_type], np.uint8)
    rc = lib().b200_synth_quantize(ggml_type, x.ctypes.data, x.size, out.ctypes.data)
    if rc:
        raise RuntimeError(f"b200_synth_quantize failed with status {rc}")
    return out
