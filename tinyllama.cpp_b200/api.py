"""ctypes mirror of include/b200llama.h. Every call goes through the C ABI of libb200llama.so;
there is no Python or CPU fallback — without the CUDA library the calls raise."""
import ctypes
import os

import numpy as np

from . import _build

KV_F32, KV_I8 = 0, 1


class B200Error(RuntimeError):
    pass


class ModelDesc(ctypes.Structure):
    _fields_ = [
        ("hidden_size", ctypes.c_int32), ("intermediate_size", ctypes.c_int32),
        ("num_attention_heads", ctypes.c_int32), ("num_key_value_heads", ctypes.c_int32),
        ("num_hidden_layers", ctypes.c_int32), ("vocab_size", ctypes.c_int32),
        ("max_position_embeddings", ctypes.c_int32), ("rms_norm_eps", ctypes.c_float),
        ("rope_theta", ctypes.c_float), ("kv_dtype", ctypes.c_int32), ("max_seqs", ctypes.c_int32),
        ("max_ctx", ctypes.c_int32), ("act_planes", ctypes.c_int32), ("device", ctypes.c_int32),
        ("tp_rank", ctypes.c_int32), ("tp_size", ctypes.c_int32), ("nccl_id", ctypes.c_uint8 * 128)]


EXPORTS = [
    "b200_last_error", "b200_device_count", "b200_engine_create", "b200_engine_upload_tensor",
    "b200_engine_finalize", "b200_engine_load_gguf", "b200_engine_get_desc", "b200_engine_destroy",
    "b200_kv_reset", "b200_lookup_embedding", "b200_forward", "b200_prefill", "b200_prefill_batch", "b200_prefill_plan", "b200_decode",
    "b200_generate_greedy", "b200_generate_greedy_penalized", "b200_dequant", "b200_matvec", "b200_matmul", "b200_rmsnorm", "b200_rmsnorm_batch",
    "b200_fused_qkv_rope", "b200_fused_gate_up_swiglu", "b200_attention_decode", "b200_attention_prefill",
    "b200_attention_decode_noalloc", "b200_engine_stats", "b200_engine_time_kernel", "b200_engine_read_trace",
    "b200_nccl_unique_id", "b200_tp_share", "b200_selftest_exchange_timeout"]

_lib = None
_vp, _i, _i64, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t


def lib():
    """Loads (building first if the sources are newer) the engine library and declares its ABI."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.build_engine()
    if not os.path.exists(path):
        raise B200Error("libb200llama.so is missing: run __graft_entry__.build()")
    L = ctypes.CDLL(path)
    L.b200_last_error.restype = ctypes.c_char_p
    L.b200_device_count.argtypes = [ctypes.POINTER(_i)]
    L.b200_engine_create.argtypes = [ctypes.POINTER(ModelDesc), ctypes.POINTER(_vp)]
    L.b200_engine_upload_tensor.argtypes = [_vp, ctypes.c_char_p, _i, _vp, _sz, _i64, _i64]
    L.b200_engine_finalize.argtypes = [_vp]
    L.b200_engine_load_gguf.argtypes = [ctypes.c_char_p, ctypes.POINTER(ModelDesc), ctypes.POINTER(_vp)]
    L.b200_engine_get_desc.argtypes = [_vp, ctypes.POINTER(ModelDesc)]
    L.b200_engine_destroy.argtypes = [_vp]
    L.b200_kv_reset.argtypes = [_vp, _i]
    L.b200_lookup_embedding.argtypes = [_vp, _i, _vp]
    L.b200_forward.argtypes = [_vp, _i, _vp, _i, _vp]
    L.b200_prefill.argtypes = [_vp, _i, _vp, _i, _i, _vp]
    L.b200_decode.argtypes = [_vp, _i, _vp, _vp, _vp, _vp, _vp]
    L.b200_prefill_batch.argtypes = [_vp, _i, _vp, _vp, _vp, _vp, _vp]
    L.b200_prefill_plan.argtypes = [_i, _vp, _i, _vp, _i, ctypes.POINTER(_i)]
    L.b200_generate_greedy.argtypes = [_vp, _i, _vp, _vp, _vp, _i, _vp, ctypes.POINTER(ctypes.c_float)]
    L.b200_generate_greedy_penalized.argtypes = [_vp, _i, _vp, _vp, _vp, _i, ctypes.c_float, _vp, _vp, _vp, ctypes.POINTER(ctypes.c_float)]
    L.b200_dequant.argtypes = [_i, _vp, _sz, _vp]
    L.b200_matvec.argtypes = [_i, _vp, _i64, _i64, _vp, _i, _i, _vp]
    L.b200_rmsnorm.argtypes = [_vp, _vp, _i, ctypes.c_float, _vp]
    L.b200_rmsnorm_batch.argtypes = [_vp, _vp, _i, _i, ctypes.c_float, _vp]
    L.b200_fused_qkv_rope.argtypes = [_i, _vp, _i, _vp, _i, _vp, _i, _i, _i, _vp, _vp, ctypes.c_float, _i, ctypes.c_float, _i, _vp, _vp, _vp]
    L.b200_fused_gate_up_swiglu.argtypes = [_i, _vp, _vp, _i, _i, _vp, _vp, ctypes.c_float, _i, _vp]
    L.b200_attention_decode.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]
    L.b200_attention_prefill.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]
    L.b200_attention_decode_noalloc.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp]
    L.b200_engine_stats.argtypes = [_vp, ctypes.POINTER(_i64), ctypes.POINTER(_i64), ctypes.POINTER(_i64)]
    L.b200_engine_time_kernel.argtypes = [_vp, _i, _i, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(_i64)]
    L.b200_matmul.argtypes = [_i, _vp, _i64, _i64, _vp, _i, _vp]
    L.b200_engine_read_trace.argtypes = [_vp, _vp, _i, ctypes.POINTER(_i)]
    L.b200_nccl_unique_id.argtypes = [_vp]
    L.b200_tp_share.argtypes = [_i64, _i, _i, ctypes.POINTER(_i64), ctypes.POINTER(_i64)]
    _lib = L
    return L


def _check(rc):
    if rc:
        raise B200Error(f"status {rc}: {lib().b200_last_error().decode()}")


def device_count():
    n = _i(0)
    _check(lib().b200_device_count(ctypes.byref(n)))
    return n.value


def _f32(a):
    return np.ascontiguousarray(a, np.float32)


def _i32(a):
    return np.ascontiguousarray(a, np.int32)


def _ptr(a):
    return a.ctypes.data_as(_vp) if a is not None else None


class Engine:
    """One model on one GPU (the host-side counterpart of TinyLlamaModel + KVCache)."""

    def __init__(self, handle):
        self._h = _vp(handle)
        d = ModelDesc()
        _check(lib().b200_engine_get_desc(self._h, ctypes.byref(d)))
        self.desc = d
        self.vocab, self.hidden = d.vocab_size, d.hidden_size

    @classmethod
    def from_gguf(cls, path, kv_dtype=KV_F32, max_seqs=1, max_ctx=0, act_planes=3, device=0, tp_rank=0, tp_size=1,
                  nccl_id=None):
        ov = ModelDesc(kv_dtype=kv_dtype, max_seqs=max_seqs, max_ctx=max_ctx, act_planes=act_planes, device=device,
                       tp_rank=tp_rank, tp_size=tp_size)
        if nccl_id is not None:
            ctypes.memmove(ov.nccl_id, bytes(nccl_id), 128)
        h = _vp()
        _check(lib().b200_engine_load_gguf(os.fsencode(path), ctypes.byref(ov), ctypes.byref(h)))
        return cls(h.value)

    @classmethod
    def create(cls, cfg, kv_dtype=KV_F32, max_seqs=1, max_ctx=0, act_planes=3, device=0):
        d = ModelDesc(cfg["hidden"], cfg["ffn"], cfg["n_heads"], cfg["n_kv_heads"], cfg["n_layers"], cfg["vocab"],
                      cfg["max_pos"], cfg.get("eps", 1e-5), cfg["theta"], kv_dtype, max_seqs, max_ctx, act_planes,
                      device, 0, 1)
        h = _vp()
        _check(lib().b200_engine_create(ctypes.byref(d), ctypes.byref(h)))
        return cls(h.value)

    def upload_tensor(self, name, ggml_type, data, rows, cols):
        data = np.ascontiguousarray(data)
        _check(lib().b200_engine_upload_tensor(self._h, name.encode(), ggml_type, _ptr(data), data.nbytes, rows, cols))

    def finalize(self):
        _check(lib().b200_engine_finalize(self._h))
        _check(lib().b200_engine_get_desc(self._h, ctypes.byref(self.desc)))

    def close(self):
        if self._h:
            lib().b200_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def kv_reset(self, slot=0):
        _check(lib().b200_kv_reset(self._h, slot))

    def lookup_embedding(self, token):
        out = np.empty(self.hidden, np.float32)
        _check(lib().b200_lookup_embedding(self._h, token, _ptr(out)))
        return out

    def forward(self, x, pos, slot=0):
        """x [hidden] is updated in place (like the reference's `input`); returns logits [vocab]."""
        assert x.dtype == np.float32 and x.flags.c_contiguous
        logits = np.empty(self.vocab, np.float32)
        _check(lib().b200_forward(self._h, slot, _ptr(x), pos, _ptr(logits)))
        return logits

    def prefill(self, ids, slot=0, start_pos=0, want_logits=True):
        ids = _i32(ids)
        logits = np.empty(self.vocab, np.float32) if want_logits else None
        _check(lib().b200_prefill(self._h, slot, _ptr(ids), len(ids), start_pos, _ptr(logits)))
        return logits

    def prefill_batch(self, prompts, slots=None, start_pos=None, want_logits=True):
        """Ingests several prompts in one call (sequence-aware chunks of 512 tokens); returns logits [n][vocab] or None."""
        n = len(prompts)
        lens = _i32([len(p) for p in prompts])
        ids = _i32(np.concatenate([np.asarray(p, np.int32) for p in prompts]))
        slots = _i32(slots if slots is not None else np.arange(n))
        start = _i32(start_pos if start_pos is not None else np.zeros(n))
        logits = np.empty((n, self.vocab), np.float32) if want_logits else None
        _check(lib().b200_prefill_batch(self._h, n, _ptr(slots), _ptr(ids), _ptr(lens), _ptr(start), _ptr(logits)))
        return logits

    def decode(self, tokens, positions, slots=None, want_logits=True, want_argmax=True):
        tokens, positions = _i32(np.atleast_1d(tokens)), _i32(np.atleast_1d(positions))
        b = len(tokens)
        slots = _i32(slots) if slots is not None else None
        logits = np.empty((b, self.vocab), np.float32) if want_logits else None
        amax = np.empty(b, np.int32) if want_argmax else None
        _check(lib().b200_decode(self._h, b, _ptr(tokens), _ptr(positions), _ptr(slots), _ptr(logits), _ptr(amax)))
        return logits, amax

    def generate_greedy(self, first_tokens, start_positions, steps, slots=None):
        first_tokens, start_positions = _i32(np.atleast_1d(first_tokens)), _i32(np.atleast_1d(start_positions))
        b = len(first_tokens)
        slots = _i32(slots) if slots is not None else None
        out = np.empty((steps, b), np.int32)
        ms = ctypes.c_float(0)
        _check(lib().b200_generate_greedy(self._h, b, _ptr(first_tokens), _ptr(start_positions), _ptr(slots), steps,
                                          _ptr(out), ctypes.byref(ms)))
        return out, ms.value

    def generate_greedy_penalized(self, first_tokens, start_positions, steps, penalty, histories=None, slots=None):
        """Greedy loop with the reference's repetition penalty on the device; histories: per sequence, the ids generated so far."""
        first_tokens, start_positions = _i32(np.atleast_1d(first_tokens)), _i32(np.atleast_1d(start_positions))
        b = len(first_tokens)
        slots = _i32(slots) if slots is not None else None
        hist = lens = None
        if histories is not None:
            lens = _i32([len(h) for h in histories])
            hist = _i32(np.concatenate([np.asarray(h, np.int32) for h in histories])) if int(lens.sum()) else _i32(np.zeros(1))
        out = np.empty((steps, b), np.int32)
        ms = ctypes.c_float(0)
        _check(lib().b200_generate_greedy_penalized(self._h, b, _ptr(first_tokens), _ptr(start_positions), _ptr(slots), steps, penalty,
                                                    _ptr(hist), _ptr(lens), _ptr(out), ctypes.byref(ms)))
        return out, ms.value

    def stats(self):
        a, b, c = _i64(0), _i64(0), _i64(0)
        _check(lib().b200_engine_stats(self._h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
        return dict(launches_per_step=a.value, weight_bytes=b.value, kv_bytes_per_position=c.value)

    def read_trace(self, max_records=4096):
        """Device timestamps (ns) of the last step's launches, [n][8]; needs B200_TRACE=1 at engine creation."""
        out = np.zeros((max_records, 8), np.uint64)
        n = _i(0)
        _check(lib().b200_engine_read_trace(self._h, out.ctypes.data_as(_vp), max_records, ctypes.byref(n)))
        return out[:n.value].copy()

    def time_kernel(self, which, iters):
        us, nbytes = ctypes.c_float(0), _i64(0)
        _check(lib().b200_engine_time_kernel(self._h, which, iters, ctypes.byref(us), ctypes.byref(nbytes)))
        return us.value, nbytes.value


def prefill_plan(lens, chunk=512):
    """Runs of the sequence-aware chunk plan: rows of (chunk, row0, tokens, first position, ending sequence or -1)."""
    lens = _i32(lens)
    cap = int(lens.sum() // chunk + 2 * len(lens) + 2)
    out = np.zeros((cap, 5), np.int32)
    n = _i(0)
    _check(lib().b200_prefill_plan(len(lens), _ptr(lens), chunk, _ptr(out), cap, ctypes.byref(n)))
    return out[:n.value].copy()


def dequant(ggml_type, blocks, n_blocks):
    blocks = np.ascontiguousarray(blocks, np.uint8)
    out = np.empty(n_blocks * (32 if ggml_type == 8 else 256), np.float32)
    _check(lib().b200_dequant(ggml_type, _ptr(blocks), n_blocks, _ptr(out)))
    return out


def matvec(ggml_type, blocks, rows, cols, x, act_planes=3):
    blocks, x = np.ascontiguousarray(blocks, np.uint8), _f32(x)
    batch = 1 if x.ndim == 1 else x.shape[0]
    y = np.empty((batch, rows), np.float32)
    _check(lib().b200_matvec(ggml_type, _ptr(blocks), rows, cols, _ptr(x), batch, act_planes, _ptr(y)))
    return y[0] if x.ndim == 1 else y


def matmul(ggml_type, blocks, rows, cols, x):
    """Tensor-core path: x [n_tokens][cols] -> y [n_tokens][rows]."""
    blocks, x = np.ascontiguousarray(blocks, np.uint8), _f32(x)
    assert x.ndim == 2 and x.shape[1] == cols
    y = np.empty((x.shape[0], rows), np.float32)
    _check(lib().b200_matmul(ggml_type, _ptr(blocks), rows, cols, _ptr(x), x.shape[0], _ptr(y)))
    return y


def rmsnorm(x, w, eps):
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    _check(lib().b200_rmsnorm(_ptr(x), _ptr(w), x.size, eps, _ptr(out)))
    return out


def rmsnorm_batch(x, w, eps):
    """x [n_tokens][n] -> normalised rows as the tensor-core path sees them (fp16-rounded)."""
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    _check(lib().b200_rmsnorm_batch(_ptr(x), _ptr(w), x.shape[0], x.shape[1], eps, _ptr(out)))
    return out


def fused_qkv_rope(types, blocks, hidden, n_heads, n_kv_heads, x, norm_w, eps, pos, theta, act_planes=3):
    """types / blocks: (q, k, v) ggml types and packed blocks. Returns rotated q [hidden], rotated k and v [n_kv*hd]."""
    bq, bk, bv = (np.ascontiguousarray(b, np.uint8) for b in blocks)
    x = _f32(x)
    norm_w = _f32(norm_w) if norm_w is not None else None
    kvd = hidden // n_heads * n_kv_heads
    q, k, v = np.empty(hidden, np.float32), np.empty(kvd, np.float32), np.empty(kvd, np.float32)
    _check(lib().b200_fused_qkv_rope(types[0], _ptr(bq), types[1], _ptr(bk), types[2], _ptr(bv), hidden, n_heads, n_kv_heads,
                                     _ptr(x), _ptr(norm_w), eps, pos, theta, act_planes, _ptr(q), _ptr(k), _ptr(v)))
    return q, k, v


def fused_gate_up_swiglu(ggml_type, gate_blocks, up_blocks, ffn, hidden, x, norm_w, eps, act_planes=3):
    bg, bu = np.ascontiguousarray(gate_blocks, np.uint8), np.ascontiguousarray(up_blocks, np.uint8)
    x = _f32(x)
    norm_w = _f32(norm_w) if norm_w is not None else None
    out = np.empty(ffn, np.float32)
    _check(lib().b200_fused_gate_up_swiglu(ggml_type, _ptr(bg), _ptr(bu), ffn, hidden, _ptr(x), _ptr(norm_w), eps, act_planes,
                                           _ptr(out)))
    return out


def attention_decode(q, k_new, v_new, k_cache, v_cache, n_heads, n_kv_heads, head_dim, kv_dtype=KV_F32, n_splits=4):
    q, k_new, v_new = _f32(q), _f32(k_new), _f32(v_new)
    k_cache, v_cache = _f32(k_cache), _f32(v_cache)
    n_ctx = k_cache.size // (n_kv_heads * head_dim)
    out = np.empty(n_heads * head_dim, np.float32)
    _check(lib().b200_attention_decode(_ptr(q), _ptr(k_new), _ptr(v_new), _ptr(k_cache), _ptr(v_cache), n_ctx, n_heads,
                                       n_kv_heads, head_dim, kv_dtype, n_splits, _ptr(out)))
    return out


def attention_prefill(q, k_rows, v_rows, n_heads, n_kv_heads, head_dim, kv_dtype=KV_F32):
    """Causal attention of the last len(q) positions over all rows of k_rows / v_rows (prompt form)."""
    q, k_rows, v_rows = _f32(q), _f32(k_rows), _f32(v_rows)
    n_tokens = q.size // (n_heads * head_dim)
    n_ctx = k_rows.size // (n_kv_heads * head_dim)
    out = np.empty((n_tokens, n_heads * head_dim), np.float32)
    _check(lib().b200_attention_prefill(_ptr(q), _ptr(k_rows), _ptr(v_rows), n_ctx, n_tokens, n_heads, n_kv_heads, head_dim,
                                        kv_dtype, _ptr(out)))
    return out


def attention_decode_noalloc(d_q, d_kv_new, d_k_cache, d_v_cache, d_k_scale, d_v_scale, d_position, n_heads, n_kv_heads,
                             head_dim, max_ctx, kv_dtype, n_splits, d_out, stream=None):
    """Allocation-free decode attention on caller-owned DEVICE buffers (integers = device addresses)."""
    _check(lib().b200_attention_decode_noalloc(d_q, d_kv_new, d_k_cache, d_v_cache, d_k_scale, d_v_scale, d_position, n_heads,
                                               n_kv_heads, head_dim, max_ctx, kv_dtype, n_splits, d_out, stream))


def selftest_exchange_timeout():
    """Returns the status of the failure-path self-test (4 = the bounded wait ran out and was reported)."""
    return lib().b200_selftest_exchange_timeout()


def nccl_unique_id():
    """128 bytes identifying a new NCCL communicator (rank 0 creates it and shares it with the other ranks)."""
    buf = (ctypes.c_uint8 * 128)()
    _check(lib().b200_nccl_unique_id(buf))
    return bytes(buf)


def tp_share(units, tp_size, tp_rank):
    b, e = _i64(0), _i64(0)
    _check(lib().b200_tp_share(units, tp_size, tp_rank, ctypes.byref(b), ctypes.byref(e)))
    return b.value, e.value
