"""Generates the golden fixtures in this folder by running the REFERENCE's own CPU code
(oracle/_ref/libref_cpu.so, built from the unmodified reference sources by oracle/Makefile).
Run where the reference tree is available:  python tests/golden/make_golden.py
The fixtures are small .npz files; the tests compare both the C oracle and the CUDA path with them.
"""
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402

pkg = ol.pkg


def f16(x):
    return np.array([x], np.float16).view(np.uint16)[0]


def known_answer_blocks():
    """Hand-packed blocks that exercise the dequantizers' corner cases."""
    rng = np.random.default_rng(7)
    out = {}
    # Q8_0: negative scale (abs() quirk), subnormal scale, zero scale, extreme quants
    blocks = []
    for d_bits, qs in [(f16(-0.0123), np.arange(-16, 16)), (np.uint16(0x0001), np.full(32, 127)),
                       (np.uint16(0x8000), rng.integers(-128, 128, 32)), (f16(0.5), np.full(32, -128)),
                       (np.uint16(0x03ff), rng.integers(-128, 128, 32)), (f16(65504.0), np.full(32, 1))]:
        blocks.append(struct.pack("<H", int(d_bits)) + qs.astype(np.int8).tobytes())
    out["q8_0"] = np.frombuffer(b"".join(blocks), np.uint8)
    # Q4_K: all-ones / all-zeros nibbles, maximal 6-bit scales and mins, subnormal d, negative dmin
    blocks = []
    for d_bits, m_bits, scales, qs in [
            (f16(0.01), f16(0.02), np.full(12, 0xFF), np.full(128, 0xFF)),
            (f16(0.01), f16(0.02), np.zeros(12), np.zeros(128)),
            (np.uint16(0x0002), f16(-0.5), rng.integers(0, 256, 12), rng.integers(0, 256, 128)),
            (f16(-1.5), np.uint16(0x0001), rng.integers(0, 256, 12), rng.integers(0, 256, 128)),
            (f16(3.0e-5), f16(1.0e-4), np.arange(12) * 21, np.arange(128) * 2 % 256)]:
        blocks.append(struct.pack("<HH", int(d_bits), int(m_bits)) + np.asarray(scales).astype(np.uint8).tobytes()
                      + np.asarray(qs).astype(np.uint8).tobytes())
    out["q4_k"] = np.frombuffer(b"".join(blocks), np.uint8)
    # Q6_K: sub-scales -128 / 127, all-ones and all-zeros bit planes, subnormal d
    blocks = []
    for ql, qh, sc, d_bits in [
            (np.full(128, 0xFF), np.full(64, 0xFF), np.full(16, 127), f16(0.002)),
            (np.zeros(128), np.zeros(64), np.full(16, -128), f16(0.002)),
            (rng.integers(0, 256, 128), rng.integers(0, 256, 64), rng.integers(-128, 128, 16), np.uint16(0x0003)),
            (rng.integers(0, 256, 128), rng.integers(0, 256, 64), np.array([-128, 127] * 8), f16(-0.75))]:
        blocks.append(np.asarray(ql).astype(np.uint8).tobytes() + np.asarray(qh).astype(np.uint8).tobytes()
                      + np.asarray(sc).astype(np.int8).tobytes() + struct.pack("<H", int(d_bits)))
    out["q6_k"] = np.frombuffer(b"".join(blocks), np.uint8)
    return out


def main():
    fx = {}
    ka = known_answer_blocks()
    rng = np.random.default_rng(11)
    for name, typ in (("q8_0", 8), ("q4_k", 12), ("q6_k", 14)):
        rnd = rng.integers(0, 256, 8 * ol.BLOCK_BYTES[typ], dtype=np.uint8)
        # keep the fp16 scale fields of the random blocks finite
        bb = ol.BLOCK_BYTES[typ]
        for b in range(8):
            for off in ({8: [0], 12: [0, 2], 14: [208]}[typ]):
                rnd[b * bb + off + 1] &= 0x7B | 0x80
                if (rnd[b * bb + off + 1] & 0x7C) == 0x7C:
                    rnd[b * bb + off + 1] &= 0xBF
        blocks = np.concatenate([ka[name], rnd])
        fx[f"{name}_blocks"] = blocks
        fx[f"{name}_out"] = ol.dequant("ref", typ, blocks)
    # fp16 conversion table for every bit pattern, both flavours
    allh = np.arange(65536, dtype=np.uint32)
    fx["fp16_plain"] = np.array([ol.ref().ref_fp16_to_fp32(int(h), 0) for h in allh], np.float32).view(np.uint32)
    fx["fp16_scale"] = np.array([ol.ref().ref_fp16_to_fp32(int(h), 1) for h in allh], np.float32).view(np.uint32)
    # Kahan matvec on a seeded matrix
    w = pkg.synth.fill_normal(64 * 512, 5, 1, 0.02).reshape(64, 512)
    x = pkg.synth.fill_normal(512, 5, 2, 1.0)
    fx["matvec_w_seed"] = np.array([5, 1, 64, 512])
    fx["matvec_y"] = ol.matvec_f32("ref", w, x)
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **fx)

    # tiny models, every scheme: logits of 3 decode steps and of a 40-token prefill + the greedy ids
    mfx = {}
    for scheme in (0, 1, 2, 3):
        path = pkg.synth.write_gguf(f"/tmp/golden_tiny_s{scheme}.gguf", "tiny", scheme=scheme, norm_random=True)
        r = ol.RefModel(path)
        tok, ids, lg = 7, [], []
        for pos in range(24):
            out = r.decode(tok, pos)
            if pos < 3:
                lg.append(out)
            tok = int(out.argmax())
            ids.append(tok)
        mfx[f"s{scheme}_decode_ids"] = np.array(ids, np.int32)
        mfx[f"s{scheme}_decode_logits"] = np.stack(lg)
        r.reset()
        prompt = np.random.default_rng(4321).integers(0, 512, 40).astype(np.int32)
        out = r.prefill(prompt)
        mfx[f"s{scheme}_prompt"] = prompt
        mfx[f"s{scheme}_prefill_logits"] = out
        tok, ids = int(out.argmax()), []
        for pos in range(40, 56):
            ids.append(tok)
            tok = int(r.decode(tok, pos).argmax())
        mfx[f"s{scheme}_after_prefill_ids"] = np.array(ids, np.int32)
        with open(path, "rb") as f:
            import hashlib
            mfx[f"s{scheme}_sha256"] = np.frombuffer(hashlib.sha256(f.read()).digest(), np.uint8)
    np.savez_compressed(os.path.join(HERE, "tiny_models.npz"), **mfx)
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()
