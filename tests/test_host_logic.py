"""CPU-only checks of the host-side pieces: synthetic model writer, GGUF readers, layout helpers."""
import numpy as np
import pytest

import oracle_lib as ol


def test_gguf_roundtrip_and_shapes(pkg, tiny_models):
    g = pkg.gguf.GGUF(tiny_models[1])
    cfg = g.config()
    assert cfg["hidden"] == 256 and cfg["n_layers"] == 2 and cfg["vocab"] == 512
    t = g.tensors["blk.1.ffn_down.weight"]
    assert (t["type"], t["rows"], t["cols"]) == (14, 256, 512)
    assert t["data"].size == 256 * 512 // 256 * 210
    assert g.tensors["blk.0.attn_q.weight"]["type"] == 12
    assert g.tensors["output.weight"]["type"] == 14
    assert g.tensors["token_embd.weight"]["type"] == 0
    assert len(g.order) == 3 + 9 * 2


def test_synth_is_deterministic(pkg, tmp_path):
    a = pkg.synth.write_gguf(str(tmp_path / "a.gguf"), "tiny", scheme=1)
    b = pkg.synth.write_gguf(str(tmp_path / "b.gguf"), "tiny", scheme=1)
    assert open(a, "rb").read() == open(b, "rb").read()
    c = pkg.synth.write_gguf(str(tmp_path / "c.gguf"), "tiny", scheme=1, seed=99)
    assert open(a, "rb").read() != open(c, "rb").read()


def test_weights_are_n_0_002(pkg):
    x = pkg.synth.fill_normal(1 << 18, 1234, 3, 0.02)
    assert abs(float(x.mean())) < 2e-4 and abs(float(x.std()) - 0.02) < 2e-4


@pytest.mark.parametrize("typ,tol", [(8, 0.01), (12, 0.12), (14, 0.04)])
def test_quantizers_fit_the_dequantizer_layout(pkg, typ, tol):
    """Quantize -> (oracle) dequantize stays within the format's resolution of the source."""
    w = pkg.synth.fill_normal(256 * 40, 5, typ, 0.02)
    back = ol.dequant("oracle", typ, pkg.synth.quantize(typ, w))
    assert np.abs(back - w).max() / np.abs(w).max() < tol


def test_activation_slot_swizzle_is_conflict_free():
    """Restates act_slot() of csrc/gemv.cuh: a bijection on 0..31 whose images of 8 consecutive
    chunks, and of 8 consecutive even (or odd) chunks, fall in 8 distinct 16-byte bank groups."""
    slot = lambda s: (s & 24) | ((s + ((s >> 3) & 1)) & 7)  # noqa: E731
    assert sorted(slot(s) for s in range(32)) == list(range(32))
    for base in range(0, 32, 8):
        assert len({slot(base + i) % 8 for i in range(8)}) == 8
    for base in (0, 16):
        for parity in (0, 1):
            assert len({slot(base + 2 * i + parity) % 8 for i in range(8)}) == 8
