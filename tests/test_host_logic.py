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


def test_quantised_embedding_table_option(pkg, tmp_path):
    """embd_quant writes token_embd in the main block type (what real checkpoints ship); the oracle's lookup of a
    row equals the dequantised blocks, and equals the reference's own lookup_embedding where it is built."""
    path = pkg.synth.write_gguf(str(tmp_path / "e.gguf"), "tiny", scheme=1, embd_quant=True)
    g = pkg.gguf.GGUF(path)
    t = g.tensors["token_embd.weight"]
    assert t["type"] == 12 and (t["rows"], t["cols"]) == (512, 256)
    table = ol.dequant("oracle", 12, t["data"]).reshape(512, 256)
    if ol.have_ref():
        r = ol.RefModel(path)
        out = np.empty(256, np.float32)
        assert ol.ref().ref_model_embedding(r.h, 77, ol._p(out)) == 0
        assert np.array_equal(out, table[77])
    plain = pkg.synth.write_gguf(str(tmp_path / "p.gguf"), "tiny", scheme=1)
    assert pkg.gguf.GGUF(plain).tensors["token_embd.weight"]["type"] == 0


def test_prefill_chunk_plan(pkg):
    """Sequence-aware ingestion lays the prompts end to end and cuts every 512 tokens: every token appears exactly once,
    runs of a sequence are contiguous in position, a chunk never exceeds its size, and each prompt ends exactly one run."""
    rng = np.random.default_rng(1)
    for lens, chunk in ([[120, 17, 100, 127, 64, 99, 111, 125, 97], 512], [[512], 512], [[513, 1, 510], 512],
                        [list(rng.integers(1, 4097, 64)), 512], [[5, 5, 5], 4]):
        plan = pkg.api.prefill_plan(lens, chunk)
        per_chunk = {}
        for c, row0, n, start, ends in plan:
            assert n >= 1 and row0 == per_chunk.get(c, 0)      # runs tile each chunk without gaps
            per_chunk[c] = row0 + n
        assert all(v <= chunk for v in per_chunk.values())
        assert sorted(per_chunk) == list(range(len(per_chunk)))
        assert all(per_chunk[c] == chunk for c in list(per_chunk)[:-1])  # every chunk but the last is full
        seq, pos = 0, 0
        for c, row0, n, start, ends in plan:                       # runs follow the sequences in order
            assert start == pos
            pos += n
            if pos == lens[seq]:
                assert ends == seq
                seq, pos = seq + 1, 0
            else:
                assert ends == -1
        assert seq == len(lens) and pos == 0
