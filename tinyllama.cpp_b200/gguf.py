"""Small GGUF reader (numpy): metadata scalars/strings and zero-copy views of the tensor data.
Same format facts as csrc/gguf.cpp; used by tests and tools that feed tensors one by one."""
import struct

import numpy as np

_SCALAR = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "B", 10: "Q", 11: "q", 12: "d"}
_TYPE_BYTES = {0: (1, 4), 1: (1, 2), 8: (32, 34), 12: (256, 144), 14: (256, 210), 30: (1, 2)}


class GGUF:
    def __init__(self, path):
        self.data = np.memmap(path, dtype=np.uint8, mode="r")
        buf = self.data
        self._p = 0

        def get(fmt):
            size = struct.calcsize("<" + fmt)
            v = struct.unpack_from("<" + fmt, buf, self._p)[0]
            self._p += size
            return v

        def string():
            n = get("Q")
            s = bytes(buf[self._p:self._p + n]).decode("utf-8", "replace")
            self._p += n
            return s

        if get("I") != 0x46554747:
            raise ValueError("not a GGUF file")
        self.version = get("I")
        n_tensors, n_kv = get("Q"), get("Q")
        self.meta = {}
        for _ in range(n_kv):
            key, t = string(), get("I")
            if t == 8:
                self.meta[key] = string()
            elif t == 9:
                et, n = get("I"), get("Q")
                self.meta[key] = [string() if et == 8 else get(_SCALAR[et]) for _ in range(n)]
            else:
                self.meta[key] = get(_SCALAR[t])
        infos = []
        for _ in range(n_tensors):
            name, nd = string(), get("I")
            shape = [get("Q") for _ in range(nd)]
            infos.append((name, shape, get("I"), get("Q")))
        align = int(self.meta.get("general.alignment", 32))
        start = (self._p + align - 1) // align * align
        self.tensors = {}
        self.order = []
        for name, shape, typ, off in infos:
            n = int(np.prod(shape)) if shape else 1
            be, bb = _TYPE_BYTES[typ]
            nbytes = n // be * bb
            cols = shape[0] if shape else 1
            rows = shape[1] if len(shape) > 1 else 1
            self.tensors[name] = dict(type=typ, rows=rows, cols=cols, data=buf[start + off:start + off + nbytes])
            self.order.append(name)

    def config(self):
        m = self.meta
        max_pos = int(m.get("llama.context_length", 4096))
        if max_pos == 0 or max_pos > 8192:
            max_pos = 2048
        return dict(hidden=int(m["llama.embedding_length"]), ffn=int(m["llama.feed_forward_length"]),
                    n_heads=int(m["llama.attention.head_count"]),
                    n_kv_heads=int(m.get("llama.attention.head_count_kv", m["llama.attention.head_count"])),
                    n_layers=int(m["llama.block_count"]),
                    vocab=int(m.get("tokenizer.ggml.vocab_size", m.get("llama.vocab_size", 32000))),
                    max_pos=max_pos, eps=float(m.get("llama.attention.layer_norm_rms_epsilon", 1e-5)),
                    theta=float(m.get("llama.rope.freq_base", 10000.0)))
