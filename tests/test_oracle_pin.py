"""Pins the C oracle: against the committed golden fixtures (made by running the reference's own
CPU code, tests/golden/make_golden.py) and, where the reference library was built
(oracle/_ref), against that library directly on fresh inputs. CPU only."""
import hashlib
import os

import numpy as np
import pytest

import oracle_lib as ol

GOLD = os.path.join(os.path.dirname(__file__), "golden")
needs_ref = pytest.mark.skipif(not ol.have_ref(), reason="reference CPU library not built on this machine")
TYPES = {"q8_0": 8, "q4_k": 12, "q6_k": 14}


@pytest.fixture(scope="module")
def ops():
    return np.load(os.path.join(GOLD, "ops.npz"))


@pytest.fixture(scope="module")
def tiny_gold():
    return np.load(os.path.join(GOLD, "tiny_models.npz"))


@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_golden_bit_exact(ops, name):
    out = ol.dequant("oracle", TYPES[name], ops[f"{name}_blocks"])
    assert np.array_equal(out.view(np.uint32), ops[f"{name}_out"].view(np.uint32))


def test_fp16_table_golden(ops):
    L = ol.oracle()
    plain = np.array([L.orc_fp16_to_fp32(h, 0) for h in range(65536)], np.float32).view(np.uint32)
    scale = np.array([L.orc_fp16_to_fp32(h, 1) for h in range(65536)], np.float32).view(np.uint32)
    assert np.array_equal(plain, ops["fp16_plain"])
    assert np.array_equal(scale, ops["fp16_scale"])
    # the scale flavour folds finite negatives onto positives (Q8_0 quirk)
    assert scale[0xBC00] == np.float32(1.0).view(np.uint32)


def test_matvec_golden(ops, pkg):
    seed, _, rows, cols = (int(v) for v in ops["matvec_w_seed"])
    w = pkg.synth.fill_normal(rows * cols, seed, 1, 0.02).reshape(rows, cols)
    x = pkg.synth.fill_normal(cols, seed, 2, 1.0)
    assert np.array_equal(ol.matvec_f32("oracle", w, x), ops["matvec_y"])


@pytest.mark.parametrize("scheme", [0, 1, 2, 3])
def test_tiny_model_golden(tiny_gold, tiny_models, scheme):
    path = tiny_models[scheme]
    with open(path, "rb") as f:
        digest = np.frombuffer(hashlib.sha256(f.read()).digest(), np.uint8)
    assert np.array_equal(digest, tiny_gold[f"s{scheme}_sha256"]), "synthetic model writer changed: regenerate fixtures"
    m = ol.OracleModel.from_gguf(path)
    tok, ids = 7, []
    for pos in range(24):
        out = m.decode(tok, pos)
        if pos < 3:
            assert np.array_equal(out, tiny_gold[f"s{scheme}_decode_logits"][pos])
        tok = int(out.argmax())
        ids.append(tok)
    assert ids == tiny_gold[f"s{scheme}_decode_ids"].tolist()
    m.reset()
    out = m.prefill(tiny_gold[f"s{scheme}_prompt"])
    assert np.array_equal(out, tiny_gold[f"s{scheme}_prefill_logits"])
    tok, ids = int(out.argmax()), []
    for pos in range(40, 56):
        ids.append(tok)
        tok = int(m.decode(tok, pos).argmax())
    assert ids == tiny_gold[f"s{scheme}_after_prefill_ids"].tolist()


@needs_ref
@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_vs_reference_random(name, pkg):
    typ = TYPES[name]
    w = pkg.synth.fill_normal(256 * 64, 99, typ, 0.02)
    blocks = pkg.synth.quantize(typ, w)
    a, b = ol.dequant("oracle", typ, blocks), ol.dequant("ref", typ, blocks)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    # the synthetic quantizers are sane: dequantized values track the source
    assert np.abs(a - w).max() < {8: 6e-4, 12: 8e-3, 14: 3e-3}[typ]


@needs_ref
def test_elementwise_ops_vs_reference():
    rng = np.random.default_rng(3)
    L, R = ol.oracle(), ol.ref()
    x = rng.standard_normal(1000).astype(np.float32) * 3
    w = (1 + 0.1 * rng.standard_normal(1000)).astype(np.float32)
    for eps in (1e-5, 1e-6, 1e-3):
        a, b = np.empty_like(x), np.empty_like(x)
        L.orc_rmsnorm_vector(ol._p(x), ol._p(w), ol._p(a), x.size, eps)
        R.ref_rmsnorm_vector(ol._p(x), ol._p(w), ol._p(b), x.size, eps)
        assert np.array_equal(a, b)
        xb = np.tile(x, 3)
        a, b = np.empty_like(xb), np.empty_like(xb)
        L.orc_rmsnorm_batch(ol._p(xb), ol._p(w), ol._p(a), 3, x.size, eps)
        R.ref_rmsnorm_batch(ol._p(xb), ol._p(w), ol._p(b), 3, x.size, eps)
        assert np.array_equal(a, b)
    a, b = np.empty_like(x), np.empty_like(x)
    L.orc_softmax(ol._p(x), ol._p(a), x.size)
    R.ref_softmax(ol._p(x), ol._p(b), x.size)
    assert np.array_equal(a, b)
    L.orc_silu(ol._p(x), ol._p(a), x.size)
    R.ref_silu(ol._p(x), ol._p(b), x.size)
    assert np.array_equal(a, b)
    tab = ol.rope_table(10000.0, 64, 32)
    v = rng.standard_normal(4 * 64).astype(np.float32)
    for pos in (0, 5, 31, 32):  # 32 is out of range: both leave the vector untouched
        a, b = v.copy(), v.copy()
        L.orc_rope_vector(ol._p(a), 4, 64, pos, ol._p(tab), 32)
        R.ref_rope_vector(ol._p(b), 4, 64, pos, ol._p(tab), 32, 1)
        assert np.array_equal(a, b)
    assert np.array_equal(a, v)


@needs_ref
def test_matvec_vs_reference_random(pkg):
    w = pkg.synth.fill_normal(37 * 768, 21, 1, 0.02).reshape(37, 768)
    x = pkg.synth.fill_normal(768, 21, 2, 1.0)
    assert np.array_equal(ol.matvec_f32("oracle", w, x), ol.matvec_f32("ref", w, x))


@needs_ref
@pytest.mark.parametrize("scheme", [0, 1])
def test_model_vs_reference_live(tiny_models, scheme):
    """The restated forward equals TinyLlamaModel::forward / forward_cpu_batch bit for bit."""
    o, r = ol.OracleModel.from_gguf(tiny_models[scheme]), ol.RefModel(tiny_models[scheme])
    tok = 11
    for pos in range(8):
        a, b = o.decode(tok, pos), r.decode(tok, pos)
        assert np.array_equal(a, b)
        tok = int(a.argmax())
    o.reset()
    r.reset()
    ids = np.random.default_rng(8).integers(0, 512, 33)
    assert np.array_equal(o.prefill(ids), r.prefill(ids))


def test_kv_quantizer_restatement():
    """Known answers for the INT8 KV quantizer arithmetic (scale = absmax/127, or 1 below 1e-8;
    round half away from zero; clamp to +-127)."""
    L = ol.oracle()
    x = np.array([0.0, 1.27, -1.27, 0.005, -0.005, 0.015, 0.635], np.float32)
    q, s = np.empty(x.size, np.int8), np.empty(1, np.float32)
    L.orc_kv_quantize_i8(ol._p(x), x.size, ol._p(q), ol._p(s))
    assert s[0] == np.float32(1.27) / np.float32(127.0)
    assert q.tolist() == [0, 127, -127, 1, -1, 2, 64]  # 0.5 rounds away from zero
    z = np.zeros(8, np.float32)
    q = np.empty(8, np.int8)
    L.orc_kv_quantize_i8(ol._p(z), 8, ol._p(q), ol._p(s))
    assert s[0] == 1.0 and not q.any()
