"""TEST INFRASTRUCTURE: ctypes front ends to the CPU checkers in oracle/ —
liboracle.so (plain-C restatement) and _ref/libref_cpu.so (the reference's own CPU sources).
Never imported by the product package."""
import ctypes
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ODIR = os.path.join(ROOT, "oracle")
sys.path.insert(0, ROOT)
import __graft_entry__  # noqa: E402

pkg = __graft_entry__.load_package()
_vp, _i, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
BLOCK_ELEMS = {8: 32, 12: 256, 14: 256}
BLOCK_BYTES = {8: 34, 12: 144, 14: 210}

_orc = None
_ref = None


def _p(a):
    return a.ctypes.data_as(_vp) if a is not None else None


def oracle():
    global _orc
    if _orc is None:
        so = os.path.join(ODIR, "liboracle.so")
        src = [os.path.join(ODIR, f) for f in ("oracle.c", "oracle.h")]
        if not os.path.exists(so) or any(os.path.getmtime(s) > os.path.getmtime(so) for s in src):
            subprocess.run(["make", "-s", "-C", ODIR, "liboracle.so"], check=True)
        L = ctypes.CDLL(so)
        L.orc_fp16_to_fp32.restype = ctypes.c_float
        L.orc_fp16_to_fp32.argtypes = [ctypes.c_uint16, _i]
        L.orc_dequant.argtypes = [_i, _vp, ctypes.c_size_t, _vp]
        L.orc_matvec_f32.argtypes = [_vp, _vp, _vp, _i64, _i64]
        L.orc_matvec_f32.restype = None
        L.orc_rmsnorm_vector.argtypes = [_vp, _vp, _vp, _i, ctypes.c_float]
        L.orc_rmsnorm_batch.argtypes = [_vp, _vp, _vp, _i, _i, ctypes.c_float]
        L.orc_softmax.argtypes = [_vp, _vp, _i]
        L.orc_silu.argtypes = [_vp, _vp, _i]
        L.orc_rope_table.argtypes = [ctypes.c_float, _i, _i, _vp]
        L.orc_rope_vector.argtypes = [_vp, _i, _i, _i, _vp, _i]
        L.orc_kv_quantize_i8.argtypes = [_vp, _i, _vp, _vp]
        L.orc_attention_decode.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp]
        L.orc_attention_decode.restype = None
        L.orc_model_create.restype = _vp
        L.orc_model_create.argtypes = [_i] * 7 + [ctypes.c_float, ctypes.c_float, _i, _i]
        L.orc_model_destroy.argtypes = [_vp]
        L.orc_model_set_tensor.argtypes = [_vp, ctypes.c_char_p, _i, _vp, _i64, _i64]
        L.orc_model_reset.argtypes = [_vp, _i]
        L.orc_model_decode.argtypes = [_vp, _i, _i, _i, _vp]
        L.orc_model_prefill.argtypes = [_vp, _i, _vp, _i, _vp]
        L.orc_model_layer_trace.restype = ctypes.POINTER(ctypes.c_float)
        L.orc_model_layer_trace.argtypes = [_vp]
        _orc = L
    return _orc


def have_ref():
    return os.path.exists(os.path.join(ODIR, "_ref", "libref_cpu.so"))


def ref():
    global _ref
    if _ref is None:
        L = ctypes.CDLL(os.path.join(ODIR, "_ref", "libref_cpu.so"))
        L.ref_last_error.restype = ctypes.c_char_p
        L.ref_fp16_to_fp32.restype = ctypes.c_float
        L.ref_fp16_to_fp32.argtypes = [ctypes.c_uint16, _i]
        L.ref_dequant.argtypes = [_i, _vp, ctypes.c_size_t, _vp]
        L.ref_matvec_f32.argtypes = [_vp, _vp, _vp, _i, _i]
        L.ref_rmsnorm_vector.argtypes = [_vp, _vp, _vp, _i, ctypes.c_float]
        L.ref_rmsnorm_batch.argtypes = [_vp, _vp, _vp, _i, _i, ctypes.c_float]
        L.ref_softmax.argtypes = [_vp, _vp, _i]
        L.ref_silu.argtypes = [_vp, _vp, _i]
        L.ref_rope_vector.argtypes = [_vp, _i, _i, _i, _vp, _i, _i]
        L.ref_model_open.restype = _vp
        L.ref_model_open.argtypes = [ctypes.c_char_p, _i]
        L.ref_model_close.argtypes = [_vp]
        L.ref_model_config.argtypes = [_vp, _vp]
        L.ref_model_reset.argtypes = [_vp]
        L.ref_model_embedding.argtypes = [_vp, _i, _vp]
        L.ref_model_decode.argtypes = [_vp, _i, _i, _vp]
        L.ref_model_prefill.argtypes = [_vp, _vp, _i, _vp, _vp]
        L.ref_model_kv.argtypes = [_vp, _i, _i, _i, _vp]
        L.ref_logger_off()
        if hasattr(L, "ref_set_threads"):
            L.ref_set_threads.argtypes = [_i]
            L.ref_set_threads.restype = None
        _ref = L
    return _ref


# ---- op helpers on either checker ----
def dequant(which, ggml_type, blocks):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    n = blocks.size // BLOCK_BYTES[ggml_type]
    out = np.empty(n * BLOCK_ELEMS[ggml_type], np.float32)
    fn = oracle().orc_dequant if which == "oracle" else ref().ref_dequant
    assert fn(ggml_type, _p(blocks), n, _p(out)) == 0
    return out


def matvec_f32(which, w, x):
    w, x = np.ascontiguousarray(w, np.float32), np.ascontiguousarray(x, np.float32)
    rows, cols = w.shape
    y = np.empty(rows, np.float32)
    if which == "oracle":
        oracle().orc_matvec_f32(_p(w), _p(x), _p(y), rows, cols)
    else:
        ref().ref_matvec_f32(_p(w), _p(x), _p(y), rows, cols)
    return y


def attention_decode(q, kc, vc, nq, nkv, hd, kv_int8=False):
    q, kc, vc = (np.ascontiguousarray(a, np.float32) for a in (q, kc, vc))
    T = kc.size // (nkv * hd)
    out = np.empty(nq * hd, np.float32)
    oracle().orc_attention_decode(_p(q), _p(kc), _p(vc), T, nq, nkv, hd, int(kv_int8), _p(out))
    return out


def rope_table(theta, head_dim, max_pos):
    t = np.empty((max_pos, head_dim // 2, 2), np.float32)
    oracle().orc_rope_table(theta, head_dim, max_pos, _p(t))
    return t


class OracleModel:
    """The restated CPU forward (oracle.c) fed tensor by tensor from a GGUF file."""

    def __init__(self, cfg, kv_int8=False, max_seqs=1):
        self.cfg = cfg
        self.V = cfg["vocab"]
        self.h = _vp(oracle().orc_model_create(cfg["hidden"], cfg["ffn"], cfg["n_heads"], cfg["n_kv_heads"],
                                               cfg["n_layers"], cfg["vocab"], cfg["max_pos"], cfg["eps"], cfg["theta"],
                                               int(kv_int8), max_seqs))

    @classmethod
    def from_gguf(cls, path, kv_int8=False, max_seqs=1):
        g = pkg.gguf.GGUF(path)
        m = cls(g.config(), kv_int8, max_seqs)
        for name in g.order:
            t = g.tensors[name]
            data = np.ascontiguousarray(t["data"])
            rc = oracle().orc_model_set_tensor(m.h, name.encode(), t["type"], _p(data), t["rows"], t["cols"])
            assert rc == 0, (name, rc)
        return m

    def reset(self, seq=0):
        oracle().orc_model_reset(self.h, seq)

    def decode(self, token, pos, seq=0):
        out = np.empty(self.V, np.float32)
        rc = oracle().orc_model_decode(self.h, seq, int(token), int(pos), _p(out))
        assert rc == 0, rc
        return out

    def prefill(self, ids, seq=0):
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty(self.V, np.float32)
        rc = oracle().orc_model_prefill(self.h, seq, _p(ids), len(ids), _p(out))
        assert rc == 0, rc
        return out

    def layer_trace(self):
        n = self.cfg["n_layers"] * self.cfg["hidden"]
        return np.ctypeslib.as_array(oracle().orc_model_layer_trace(self.h), shape=(n,)).reshape(
            self.cfg["n_layers"], self.cfg["hidden"]).copy()

    def __del__(self):
        try:
            oracle().orc_model_destroy(self.h)
        except Exception:
            pass


class RefModel:
    """The reference's own TinyLlamaModel on the CPU, loaded from a GGUF file."""

    def __init__(self, path):
        self.h = _vp(ref().ref_model_open(os.fsencode(path), 1))
        if not self.h:
            raise RuntimeError(ref().ref_last_error().decode())
        cfg = np.zeros(10, np.int32)
        ref().ref_model_config(self.h, _p(cfg))
        self.V, self.H = int(cfg[5]), int(cfg[0])

    def reset(self):
        ref().ref_model_reset(self.h)

    def decode(self, token, pos):
        out = np.empty(self.V, np.float32)
        rc = ref().ref_model_decode(self.h, int(token), int(pos), _p(out))
        assert rc == 0, ref().ref_last_error()
        return out

    def prefill(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty(self.V, np.float32)
        rc = ref().ref_model_prefill(self.h, _p(ids), len(ids), _p(out), None)
        assert rc == 0, ref().ref_last_error()
        return out

    def __del__(self):
        try:
            ref().ref_model_close(self.h)
        except Exception:
            pass
