"""Parity of the CUDA path (through the C ABI) with the CPU oracle and the golden fixtures.

Tolerances (stated here, used below):
  dequantized blocks     bit-exact
  matvec                 |y - ref| <= 1e-3 * max(|ref_i|, 1e-3 * max|ref|)   (ref = Kahan FP32 dot, utils.cpp:349-397)
  logits                 <= 2e-2 absolute; greedy ids identical for 32 steps
"""
import os

import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TYPES = {"q8_0": 8, "q4_k": 12, "q6_k": 14}


def rel_err(y, ref):
    den = np.maximum(np.abs(ref), 1e-3 * np.abs(ref).max())
    return float((np.abs(y - ref) / den).max())


@pytest.fixture(scope="module")
def ops():
    return np.load(os.path.join(GOLD, "ops.npz"))


@pytest.fixture(scope="module")
def tiny_gold():
    return np.load(os.path.join(GOLD, "tiny_models.npz"))


@pytest.mark.parametrize("name", list(TYPES))
def test_dequant_bit_exact_golden_and_random(pkg, ops, name):
    typ = TYPES[name]
    blocks = ops[f"{name}_blocks"]
    out = pkg.api.dequant(typ, blocks, blocks.size // ol.BLOCK_BYTES[typ])
    assert np.array_equal(out.view(np.uint32), ops[f"{name}_out"].view(np.uint32))
    rnd = np.random.default_rng(typ).integers(0, 256, 513 * ol.BLOCK_BYTES[typ], dtype=np.uint8)
    out = pkg.api.dequant(typ, rnd, 513)
    ref = ol.dequant("oracle", typ, rnd)
    # random bytes include NaN / Inf scale fields: NaNs must sit in the same places (their payload
    # bits are not defined by IEEE arithmetic), everything else must match bit for bit
    assert np.array_equal(np.isnan(out), np.isnan(ref))
    ok = ~np.isnan(ref)
    assert np.array_equal(out.view(np.uint32)[ok], ref.view(np.uint32)[ok])
    assert pkg.api.dequant(typ, np.zeros(0, np.uint8), 0).size == 0  # empty input


@pytest.mark.parametrize("planes", [3, 2])
@pytest.mark.parametrize("name", list(TYPES))
@pytest.mark.parametrize("rows,cols", [(2, 256), (6, 512), (64, 4096), (130, 11008), (34, 1024)])
def test_matvec_vs_kahan_dot(pkg, name, rows, cols, planes):
    typ = TYPES[name]
    w = pkg.synth.fill_normal(rows * cols, 77, rows + typ, 0.02)
    blocks = pkg.synth.quantize(typ, w)
    x = pkg.synth.fill_normal(cols, 78, cols, 1.0)
    wd = ol.dequant("oracle", typ, blocks).reshape(rows, cols)
    ref = ol.matvec_f32("oracle", wd, x)
    y = pkg.api.matvec(typ, blocks, rows, cols, x, act_planes=planes)
    err = rel_err(y, ref)
    if planes == 3:
        assert err <= 1e-3, err
    else:  # 16-bit activations: looser floor, still 1e-3 on elements that are not near-cancelled
        den = np.maximum(np.abs(ref), 1e-1 * np.abs(ref).max())
        assert float((np.abs(y - ref) / den).max()) <= 1e-3


@pytest.mark.parametrize("name,rows,cols", [("q4_k", 7144, 4096), ("q6_k", 4800, 11008), ("q8_0", 7000, 2048),
                                            ("q6_k", 9000, 4096), ("q4_k", 40300, 4096)])
def test_matvec_many_tiles_per_cta(pkg, name, rows, cols):
    """Shapes where every CTA walks several tiles: the ring of stages wraps, slots are refilled by the
    last warp to leave them, and (last case) the parked partial sums are flushed more than once."""
    typ = TYPES[name]
    w = pkg.synth.fill_normal(rows * cols, 91, rows + typ, 0.02)
    blocks = pkg.synth.quantize(typ, w)
    x = pkg.synth.fill_normal(cols, 92, cols, 1.0)
    wd = ol.dequant("oracle", typ, blocks).reshape(rows, cols)
    ref = ol.matvec_f32("oracle", wd, x)
    y = pkg.api.matvec(typ, blocks, rows, cols, x)
    assert rel_err(y, ref) <= 1e-3


@pytest.mark.parametrize("name,rows,cols,tokens", [("q4_k", 128, 256, 16), ("q8_0", 64, 256, 16), ("q6_k", 130, 512, 32),
                                                   ("q4_k", 1024, 4096, 64), ("q6_k", 512, 11008, 48), ("q4_k", 300, 1024, 300),
                                                   ("q8_0", 520, 2048, 17), ("q4_k", 18944, 4096, 256), ("q4_k", 1024, 4096, 512),
                                                   ("q6_k", 512, 1024, 400)])
def test_matmul_tensor_core(pkg, name, rows, cols, tokens):
    """The tcgen05 / TMEM matmul (batch >= 16 and prompt path) against the FP64 product of the dequantised
    weights. Operands are rounded to fp16, so the tolerance is 1e-3 of the largest output (measured 3e-4)."""
    typ = TYPES[name]
    w = pkg.synth.fill_normal(rows * cols, 11, rows + typ, 0.02)
    blocks = pkg.synth.quantize(typ, w)
    x = pkg.synth.fill_normal(tokens * cols, 12, cols, 1.0).reshape(tokens, cols)
    wd = ol.dequant("oracle", typ, blocks).reshape(rows, cols)
    ref = (wd.astype(np.float64) @ x.astype(np.float64).T).T
    y = pkg.api.matmul(typ, blocks, rows, cols, x)
    assert np.abs(y - ref).max() <= 1e-3 * np.abs(ref).max()


def test_matvec_batch_and_edge_values(pkg):
    rows, cols = 8, 512
    w = pkg.synth.fill_normal(rows * cols, 5, 9, 0.02)
    blocks = pkg.synth.quantize(12, w)
    wd = ol.dequant("oracle", 12, blocks).reshape(rows, cols)
    x = np.stack([pkg.synth.fill_normal(cols, 6, i + 1, 1.0) for i in range(3)])
    x[1] = 0.0                      # all-zero activation vector
    x[2, :256] = 0.0                # one all-zero 256-block
    x[2, 300] = 1e4                 # outlier dominating its block's scale
    y = pkg.api.matvec(12, blocks, rows, cols, x)
    for b in range(3):
        ref = ol.matvec_f32("oracle", wd, x[b])
        assert np.all(np.abs(y[b] - ref) <= 1e-3 * np.maximum(np.abs(ref), 1e-3 * max(np.abs(ref).max(), 1e-30)))
    assert not y[1].any()


@pytest.mark.parametrize("n", [256, 2048, 4096, 11008, 14336])
def test_rmsnorm_decode_prologue(pkg, n):
    """The RMSNorm the decode path runs (prologue of the matvec kernel: FP32 sum of squares, rsqrtf, then the
    24-bit block quantisation of the activations) against rmsnorm_vector_cpu. Bound: 1e-6 of the largest output
    (2 ulp of the reciprocal square root + 2^-23 of a block's largest magnitude)."""
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32) * 2
    x[5] = 40.0  # an outlier that dominates its block's scale
    w = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    ref = np.empty_like(x)
    ol.oracle().orc_rmsnorm_vector(ol._p(x), ol._p(w), ol._p(ref), x.size, 1e-5)
    out = pkg.api.rmsnorm(x, w, 1e-5)
    assert np.abs(out - ref).max() <= 1e-6 * np.abs(ref).max()


def test_rmsnorm_batch_path(pkg):
    """The RMSNorm of the prompt / batch >= 16 path (one block per token, output rounded to fp16 for the tensor-core
    matmul) against rmsnorm_batch_cpu: the only difference allowed is the fp16 rounding (2^-11 relative)."""
    rng = np.random.default_rng(3)
    x = (rng.standard_normal((37, 4096)) * 3).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float32)
    ref = np.empty_like(x)
    ol.oracle().orc_rmsnorm_batch(ol._p(x), ol._p(w), ol._p(ref), 37, 4096, 1e-5)
    out = pkg.api.rmsnorm_batch(x, w, 1e-5)
    assert np.all(np.abs(out - ref) <= 2.0 ** -11 * np.abs(ref) * 1.001 + 1e-7)


def _quantized(pkg, typ, rows, cols, seed):
    w = pkg.synth.fill_normal(rows * cols, seed, rows + typ, 0.02)
    blocks = pkg.synth.quantize(typ, w)
    return blocks, ol.dequant("oracle", typ, blocks).reshape(rows, cols)


@pytest.mark.parametrize("pos", [0, 1, 777])
def test_fused_qkv_rope_launch_7b_head_shape(pkg, pos):
    """RMSNorm + q/k/v projections + RoPE as ONE launch of the decode step, at hidden 4096 / head_dim 128 (q, k Q4_K;
    v Q6_K; 8 KV heads to keep the CPU side short), against the oracle's composition: rmsnorm_vector, Kahan
    matvec, apply_rope_vector. Matvec tolerance (1e-3 relative, floor 1e-3 of the largest output)."""
    H, nq, nkv, hd = 4096, 32, 8, 128
    bq, wq = _quantized(pkg, 12, H, H, 41)
    bk, wk = _quantized(pkg, 12, nkv * hd, H, 42)
    bv, wv = _quantized(pkg, 14, nkv * hd, H, 43)
    rng = np.random.default_rng(pos)
    x = rng.standard_normal(H).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    xn = np.empty_like(x)
    ol.oracle().orc_rmsnorm_vector(ol._p(x), ol._p(nw), ol._p(xn), H, 1e-5)
    q, k, v = (ol.matvec_f32("oracle", w, xn) for w in (wq, wk, wv))
    table = ol.rope_table(10000.0, hd, pos + 1)
    ol.oracle().orc_rope_vector(ol._p(q), nq, hd, pos, ol._p(table), pos + 1)
    ol.oracle().orc_rope_vector(ol._p(k), nkv, hd, pos, ol._p(table), pos + 1)
    gq, gk, gv = pkg.api.fused_qkv_rope((12, 12, 14), (bq, bk, bv), H, nq, nkv, x, nw, 1e-5, pos, 10000.0)
    assert rel_err(gq, q) <= 1e-3
    assert rel_err(gk, k) <= 1e-3
    assert rel_err(gv, v) <= 1e-3


@pytest.mark.parametrize("typ", [12, 8])
def test_fused_gate_up_swiglu_launch_7b_shape(pkg, typ):
    """RMSNorm + gate/up projections + SwiGLU as ONE launch (hidden 4096, FFN 11008) against the oracle's decode
    expressions (model.cpp:734-735 with silu_cpu): silu(g) * u with the Kahan dot for g and u."""
    H, F = 4096, 11008
    bg, wg = _quantized(pkg, typ, F, H, 51)
    bu, wu = _quantized(pkg, typ, F, H, 52)
    rng = np.random.default_rng(typ)
    x = rng.standard_normal(H).astype(np.float32)
    nw = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    xn = np.empty_like(x)
    ol.oracle().orc_rmsnorm_vector(ol._p(x), ol._p(nw), ol._p(xn), H, 1e-5)
    g, u = ol.matvec_f32("oracle", wg, xn), ol.matvec_f32("oracle", wu, xn)
    act = np.empty_like(g)
    ol.oracle().orc_silu(ol._p(g), ol._p(act), F)
    ref = act * u
    out = pkg.api.fused_gate_up_swiglu(typ, bg, bu, F, H, x, nw, 1e-5)
    assert rel_err(out, ref) <= 2e-3  # a product of two outputs that each carry the matvec tolerance


@pytest.mark.parametrize("kv_i8", [False, True])
@pytest.mark.parametrize("nq,nkv,hd,n_ctx,splits", [(4, 2, 64, 0, 1), (4, 2, 64, 1, 3), (8, 8, 128, 77, 4),
                                                     (8, 2, 128, 300, 8), (4, 1, 32, 129, 5), (32, 4, 64, 1000, 6)])
def test_attention_decode(pkg, kv_i8, nq, nkv, hd, n_ctx, splits):
    rng = np.random.default_rng(n_ctx + nq)
    q = rng.standard_normal(nq * hd).astype(np.float32)
    kc = rng.standard_normal((n_ctx + 1, nkv, hd)).astype(np.float32)
    vc = rng.standard_normal((n_ctx + 1, nkv, hd)).astype(np.float32)
    if n_ctx > 2:
        kc[1] = 0.0  # an all-zero row: INT8 scale falls back to 1.0
    ref = ol.attention_decode(q, kc, vc, nq, nkv, hd, kv_int8=kv_i8)
    out = pkg.api.attention_decode(q, kc[-1], vc[-1], kc[:-1], vc[:-1], nq, nkv, hd,
                                   kv_dtype=pkg.KV_I8 if kv_i8 else pkg.KV_F32, n_splits=splits)
    assert np.abs(out - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("kv_i8", [False, True])
@pytest.mark.parametrize("nq,nkv,hd,n_ctx,n_tok", [(4, 2, 64, 40, 40), (4, 4, 64, 130, 1), (8, 2, 128, 333, 77),
                                                  (32, 8, 128, 1100, 256), (2, 1, 128, 64, 64), (2, 2, 64, 65, 65)])
def test_attention_prefill(pkg, kv_i8, nq, nkv, hd, n_ctx, n_tok):
    """Prompt attention on the fp16 tensor cores against the per-token FP32 attention of the oracle
    (each token attends to the rows up to its own position). Tolerance 3e-3 of the largest output:
    Q, FP32 K / V rows and the probabilities are rounded to fp16 (2^-11 relative each)."""
    rng = np.random.default_rng(n_ctx * 7 + nq)
    q = rng.standard_normal((n_tok, nq * hd)).astype(np.float32)
    kc = rng.standard_normal((n_ctx, nkv, hd)).astype(np.float32)
    vc = rng.standard_normal((n_ctx, nkv, hd)).astype(np.float32)
    if n_ctx > 2:
        kc[1] = 0.0
        vc[2] = 0.0  # all-zero rows: INT8 scale falls back to 1.0
    start = n_ctx - n_tok
    out = pkg.api.attention_prefill(q, kc, vc, nq, nkv, hd, kv_dtype=pkg.KV_I8 if kv_i8 else pkg.KV_F32)
    worst, big = 0.0, 1.0
    for i in range(n_tok):
        ref = ol.attention_decode(q[i], kc[:start + i + 1], vc[:start + i + 1], nq, nkv, hd, kv_int8=kv_i8)
        worst = max(worst, float(np.abs(out[i] - ref).max()))
        big = max(big, float(np.abs(ref).max()))
    assert worst <= 3e-3 * big, (worst, big)


def run_greedy(eng, orc, first, steps, start=0):
    tok, ids_e, ids_o, worst, margins = first, [], [], 0.0, []
    for pos in range(start, start + steps):
        logits, amax = eng.decode([tok], [pos])
        ref = orc.decode(tok, pos)
        worst = max(worst, float(np.abs(logits[0] - ref).max()))
        ids_e.append(int(amax[0]))
        ids_o.append(int(ref.argmax()))
        top2 = np.sort(ref)[-2:]
        margins.append(float(top2[1] - top2[0]))
        assert int(amax[0]) == int(logits[0].argmax())
        tok = ids_o[-1]
    return ids_e, ids_o, worst, margins


@pytest.mark.parametrize("planes", [3, 2])
@pytest.mark.parametrize("scheme", [0, 1, 2, 3])
def test_engine_decode_fp32_kv(pkg, tiny_models, tiny_gold, scheme, planes):
    eng = pkg.Engine.from_gguf(tiny_models[scheme], kv_dtype=pkg.KV_F32, act_planes=planes)
    orc = ol.OracleModel.from_gguf(tiny_models[scheme])
    ids_e, ids_o, worst, margins = run_greedy(eng, orc, 7, 32)
    assert worst <= 2e-2, worst
    if planes == 3:  # 24-bit activations: the default, and the mode the greedy-id gate is defined on
        assert ids_e == ids_o
        assert ids_e[:24] == tiny_gold[f"s{scheme}_decode_ids"].tolist()
        assert worst <= 1e-4, worst  # far inside the gate
    else:  # 16-bit activations (speed option): ids may only differ where the oracle's top-2 gap is a near-tie
        assert all(a == b or m < 1e-3 for a, b, m in zip(ids_e, ids_o, margins))
    eng.close()


@pytest.mark.parametrize("scheme", [0, 1])
def test_engine_decode_int8_kv(pkg, tiny_models, scheme):
    eng = pkg.Engine.from_gguf(tiny_models[scheme], kv_dtype=pkg.KV_I8)
    orc = ol.OracleModel.from_gguf(tiny_models[scheme], kv_int8=True)
    ids_e, ids_o, worst, _ = run_greedy(eng, orc, 3, 32)
    assert worst <= 2e-2, worst
    assert ids_e == ids_o
    eng.close()


@pytest.mark.parametrize("scheme", [0, 1])
def test_engine_prefill_then_decode(pkg, tiny_models, tiny_gold, scheme):
    eng = pkg.Engine.from_gguf(tiny_models[scheme])
    prompt = tiny_gold[f"s{scheme}_prompt"]
    logits = eng.prefill(prompt)
    assert np.abs(logits - tiny_gold[f"s{scheme}_prefill_logits"]).max() <= 2e-2
    tok, ids = int(logits.argmax()), []
    for pos in range(40, 56):
        ids.append(tok)
        lg, amax = eng.decode([tok], [pos])
        tok = int(amax[0])
    assert ids == tiny_gold[f"s{scheme}_after_prefill_ids"].tolist()
    eng.close()


def test_generate_greedy_matches_stepwise_and_oracle(pkg, tiny_models):
    eng = pkg.Engine.from_gguf(tiny_models[1], kv_dtype=pkg.KV_I8, max_seqs=3)
    orc = ol.OracleModel.from_gguf(tiny_models[1], kv_int8=True, max_seqs=3)
    firsts = [5, 400, 77]
    out, ms = eng.generate_greedy(firsts, [0, 0, 0], 32)
    assert ms > 0
    for b, first in enumerate(firsts):
        tok, ids = first, []
        for pos in range(32):
            tok = int(orc.decode(tok, pos, seq=b).argmax())
            ids.append(tok)
        assert out[:, b].tolist() == ids
    # a second call continues from the caches it left
    out2, _ = eng.generate_greedy(out[-1], [32, 32, 32], 8)
    for b in range(3):
        tok = int(out[-1, b])
        for pos in range(32, 40):
            tok = int(orc.decode(tok, pos, seq=b).argmax())
            assert out2[pos - 32, b] == tok
    eng.close()


def _penalise(logits, generated, penalty, window=64):
    """apply_repetition_penalty of the reference (api.cpp:86-97), restated: once per occurrence in the window."""
    out = logits.copy()
    for tid in generated[-window:]:
        out[tid] = np.float32(out[tid] / np.float32(penalty)) if out[tid] > 0 else np.float32(out[tid] * np.float32(penalty))
    return out


@pytest.mark.parametrize("penalty", [1.3, 1.0])
def test_generate_greedy_with_repetition_penalty_on_device(pkg, tiny_models, penalty):
    """The device-resident loop with the reference's repetition penalty (default 1.3 in TinyLlamaSession::generate)
    against the oracle's logits put through a restatement of apply_repetition_penalty + first-maximum argmax: 100
    steps, so ids leave the 64-token window again, for two sequences with different histories."""
    eng = pkg.Engine.from_gguf(tiny_models[1], max_seqs=2)
    orc = ol.OracleModel.from_gguf(tiny_models[1], max_seqs=2)
    firsts, hist = [5, 400], [[9, 5], [400]]
    out, _ = eng.generate_greedy_penalized(firsts, [0, 0], 100, penalty, histories=hist)
    for b in range(2):
        gen, tok = list(hist[b]), firsts[b]
        exact = 0
        for pos in range(100):
            lg = _penalise(orc.decode(tok, pos, seq=b), gen, penalty)
            tok = int(out[pos, b])  # follow the engine's choice, so that one near-tie cannot derail the rest of the check
            exact += int(tok == int(lg.argmax()))
            assert lg[tok] >= lg.max() - 1e-3, (b, pos, tok, int(lg.argmax()))
            gen.append(tok)
        assert exact >= 98, exact
    if penalty > 1.0:  # the penalty changes the sequence (a tiny model falls into a cycle without it)
        plain, _ = pkg.Engine.from_gguf(tiny_models[1], max_seqs=2).generate_greedy(firsts, [0, 0], 100)
        assert not np.array_equal(plain, out)
    eng.close()


def test_batch_decode_ragged_positions_and_slots(pkg, tiny_models):
    """Independent sequences at different positions, mapped to shuffled KV slots."""
    eng = pkg.Engine.from_gguf(tiny_models[3], max_seqs=4)
    orc = ol.OracleModel.from_gguf(tiny_models[3], max_seqs=4)
    rng = np.random.default_rng(5)
    lens = [3, 17, 1, 40]
    slots = [2, 0, 3, 1]
    last = []
    for s, n in zip(slots, lens):
        ids = rng.integers(0, 512, n)
        eng.prefill(ids, slot=s)
        orc.prefill(ids, seq=s)
        last.append(int(ids[-1]))
    toks = [9, 10, 11, 12]
    logits, amax = eng.decode(toks, lens, slots=slots)
    for b in range(4):
        ref = orc.decode(toks[b], lens[b], seq=slots[b])
        assert np.abs(logits[b] - ref).max() <= 2e-2
        assert int(amax[b]) == int(ref.argmax())
    eng.close()


@pytest.mark.parametrize("scheme,kv", [(1, "f32"), (0, "i8"), (2, "f32")])
def test_batch16_decode_takes_tensor_core_path(pkg, tiny_models, scheme, kv):
    """Batches of 16 and more run their linear layers on the tcgen05 matmul: logits against the oracle
    (2e-2 absolute) over three steps with ragged positions, greedy ids where the oracle's top-2 gap is clear."""
    B = 20
    kvd = pkg.KV_I8 if kv == "i8" else pkg.KV_F32
    eng = pkg.Engine.from_gguf(tiny_models[scheme], max_seqs=B, kv_dtype=kvd)
    orc = ol.OracleModel.from_gguf(tiny_models[scheme], max_seqs=B, kv_int8=(kv == "i8"))
    rng = np.random.default_rng(17)
    pos = [0] * B
    for s in range(0, B, 3):  # some sequences start with a short history (ingested by the batch-1 path)
        ids = rng.integers(0, 512, 1 + s % 5)
        eng.prefill(ids, slot=s)
        orc.prefill(ids, seq=s)
        pos[s] = len(ids)
    toks = [int(t) for t in rng.integers(0, 512, B)]
    for step in range(3):
        logits, amax = eng.decode(toks, pos)
        nxt = []
        for b in range(B):
            ref = orc.decode(toks[b], pos[b], seq=b)
            assert np.abs(logits[b] - ref).max() <= 2e-2
            top = np.sort(ref)[-2:]
            if top[1] - top[0] > 1e-2:
                assert int(amax[b]) == int(ref.argmax())
            nxt.append(int(ref.argmax()))
        toks, pos = nxt, [p + 1 for p in pos]
    eng.close()


@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("kv", ["f32", "i8"])
def test_batch_decode_grouped_query_attention_long_contexts(pkg, tiny_models, kv, splits, monkeypatch):
    """Batched decode of a grouped-query model (2 query heads per KV head) with ragged contexts of up to two
    64-key tiles: the tensor-core attention that serves a whole group per CTA, all four key quarters and the
    merge of their partial softmaxes. Logits against the oracle: 2e-2 absolute (FP32 cache); with the INT8
    cache the prompt's K/V rows come from fp16 matmuls and may round to a neighbouring int8 step, so the
    bound is relative to the largest logit as in the prompt tests."""
    B = 16
    monkeypatch.setenv("B200_GQA_SPLITS", str(splits))  # context runs per sequence (3: with empty runs and the cross-CTA merge)
    kvd = pkg.KV_I8 if kv == "i8" else pkg.KV_F32
    eng = pkg.Engine.from_gguf(tiny_models[1], max_seqs=B, kv_dtype=kvd)
    orc = ol.OracleModel.from_gguf(tiny_models[1], max_seqs=B, kv_int8=(kv == "i8"))
    rng = np.random.default_rng(23)
    lens = [int(n) for n in rng.integers(1, 118, B)]
    lens[0], lens[1], lens[2] = 63, 64, 117
    for s in range(B):
        ids = rng.integers(0, 512, lens[s])
        eng.prefill(ids, slot=s)
        orc.prefill(ids, seq=s)
    toks = [int(t) for t in rng.integers(0, 512, B)]
    pos = list(lens)
    for step in range(3):
        logits, amax = eng.decode(toks, pos)
        nxt = []
        for b in range(B):
            ref = orc.decode(toks[b], pos[b], seq=b)
            tol = 2e-2 if kv == "f32" else max(2e-2, 1.5e-2 * float(np.abs(ref).max()))
            assert np.abs(logits[b] - ref).max() <= tol, (b, pos[b])
            nxt.append(int(ref.argmax()))
        toks, pos = nxt, [p + 1 for p in pos]
    eng.close()


@pytest.mark.parametrize("kv", ["f32", "i8"])
def test_prefill_batch_equals_one_call_per_sequence(pkg, tiny_models, kv):
    """Sequence-aware ingestion of ragged prompts in shared 512-token chunks (nine sequences, 860 tokens: two chunks, a
    prompt that straddles the chunk border, prompts shorter than a tile) against one b200_prefill call per sequence:
    logits and the following decode step agree to 1e-4 (each token's matmul column and attention rows are its own, so
    the two differ at most by the order of a few fp32 additions where a prompt straddles a chunk border); and against
    the oracle with the tensor-core path's tolerance."""
    kvd = pkg.KV_I8 if kv == "i8" else pkg.KV_F32
    lens = [120, 17, 100, 127, 64, 99, 111, 125, 97]
    rng = np.random.default_rng(31)
    prompts = [rng.integers(0, 512, n).astype(np.int32) for n in lens]
    slots = [3, 0, 8, 1, 7, 2, 6, 4, 5]
    a = pkg.Engine.from_gguf(tiny_models[1], max_seqs=9, kv_dtype=kvd)
    b = pkg.Engine.from_gguf(tiny_models[1], max_seqs=9, kv_dtype=kvd)
    got = a.prefill_batch(prompts, slots=slots)
    exact = 0
    for i, p in enumerate(prompts):
        one = b.prefill(p, slot=slots[i])
        assert np.abs(got[i] - one).max() <= (1e-4 if kv == "f32" else max(1e-4, 1.5e-2 * float(np.abs(one).max()))), i
        exact += int(np.array_equal(got[i], one))
    print(f"prefill_batch: {exact} of {len(prompts)} prompts bit-identical to the per-sequence call")
    toks = [int(g.argmax()) for g in got]
    la, _ = a.decode(toks[:4], lens[:4], slots=slots[:4])
    lb, _ = b.decode(toks[:4], lens[:4], slots=slots[:4])
    assert np.abs(la - lb).max() <= (1e-4 if kv == "f32" else max(1e-4, 1.5e-2 * float(np.abs(lb).max())))
    orc = ol.OracleModel.from_gguf(tiny_models[1], kv_int8=(kv == "i8"), max_seqs=9)
    for i in (1, 3):
        ref = orc.prefill(prompts[i], seq=slots[i])
        tol = 2e-2 if kv == "f32" else max(2e-2, 1.5e-2 * float(np.abs(ref).max()))
        assert np.abs(got[i] - ref).max() <= tol
    with pytest.raises(pkg.B200Error, match="same KV slot"):
        a.prefill_batch(prompts[:2], slots=[1, 1])
    with pytest.raises(pkg.B200Error, match="exceeds the KV capacity"):
        a.prefill_batch([np.zeros(200, np.int32)], slots=[0])
    a.close()
    b.close()


def test_forward_from_hidden_state(pkg, tiny_models):
    """b200_forward mirrors TinyLlamaModel::forward: hidden vector in, logits out, input updated in place."""
    eng = pkg.Engine.from_gguf(tiny_models[1])
    orc = ol.OracleModel.from_gguf(tiny_models[1])
    x = eng.lookup_embedding(42)
    g = pkg.gguf.GGUF(tiny_models[1])
    emb = np.frombuffer(g.tensors["token_embd.weight"]["data"], np.float32).reshape(512, 256)
    assert np.array_equal(x, emb[42])
    logits = eng.forward(x, 0)
    ref = orc.decode(42, 0)
    assert np.abs(logits - ref).max() <= 2e-2
    assert np.abs(x - orc.layer_trace()[-1]).max() <= 1e-4  # residual stream after the last layer
    eng.close()


@pytest.mark.parametrize("scheme,typ", [(1, 12), (0, 8), (2, 14)])
def test_quantised_embedding_table(pkg, tmp_path, scheme, typ):
    """A checkpoint whose token_embd is Q4_K / Q8_0 / Q6_K (as real quantised checkpoints ship it): the lookup returns
    the reference dequantiser's values bit for bit and the decode logits match the oracle on the same file."""
    path = pkg.synth.write_gguf(str(tmp_path / "e.gguf"), "tiny", scheme=scheme, embd_quant=True, norm_random=True)
    g = pkg.gguf.GGUF(path)
    t = g.tensors["token_embd.weight"]
    assert t["type"] == typ
    table = ol.dequant("oracle", typ, t["data"]).reshape(512, 256)
    eng = pkg.Engine.from_gguf(path)
    orc = ol.OracleModel.from_gguf(path)
    for tok in (0, 77, 511):
        assert np.array_equal(eng.lookup_embedding(tok).view(np.uint32), table[tok].view(np.uint32))
    ids_e, ids_o, worst, _ = run_greedy(eng, orc, 9, 8)
    assert worst <= 2e-2 and ids_e == ids_o
    eng.close()


def test_kv_reset_and_errors(pkg, tiny_models):
    eng = pkg.Engine.from_gguf(tiny_models[0], max_ctx=16)
    a, _ = eng.decode([1], [0])
    eng.decode([2], [1])
    eng.kv_reset(0)
    b, _ = eng.decode([1], [0])
    assert np.array_equal(a, b)
    with pytest.raises(pkg.B200Error, match="exceeds the KV capacity"):
        eng.decode([1], [16])
    with pytest.raises(pkg.B200Error, match="token id out of range"):
        eng.decode([512], [0])
    with pytest.raises(pkg.B200Error, match="batch out of range"):
        eng.decode([1, 2], [0, 0])
    with pytest.raises(pkg.B200Error):
        eng.prefill(np.arange(17))
    eng.close()
    with pytest.raises(pkg.B200Error, match="cannot open"):
        pkg.Engine.from_gguf("/nonexistent/model.gguf")


def test_bounded_wait_runs_out_and_is_reported(pkg, tiny_models):
    """A consumer of a tensor-parallel exchange whose packets never arrive: the poll gives up after its (shortened)
    limit, the kernel returns, status 4 comes back, and the same process keeps computing correctly afterwards."""
    assert pkg.api.selftest_exchange_timeout() == 4
    assert "bounded wait" in pkg.api.lib().b200_last_error().decode()
    eng = pkg.Engine.from_gguf(tiny_models[1])
    orc = ol.OracleModel.from_gguf(tiny_models[1])
    lg, _ = eng.decode([5], [0])
    assert np.abs(lg[0] - orc.decode(5, 0)).max() <= 2e-2
    eng.close()


def test_upload_tensor_path_and_validation(pkg, tiny_models):
    """create + upload_tensor + finalize gives the same engine as load_gguf; malformed input is refused."""
    g = pkg.gguf.GGUF(tiny_models[1])
    eng = pkg.Engine.create(g.config())
    with pytest.raises(pkg.B200Error, match="unknown tensor name"):
        eng.upload_tensor("blk.9.attn_q.weight", 12, np.zeros(144, np.uint8), 1, 256)
    t = g.tensors["blk.0.attn_q.weight"]
    with pytest.raises(pkg.B200Error, match="byte count"):
        eng.upload_tensor("blk.0.attn_q.weight", 12, t["data"][:-144], t["rows"], t["cols"])
    with pytest.raises(pkg.B200Error):
        eng.finalize()  # tensors missing
    for name in g.order:
        t = g.tensors[name]
        eng.upload_tensor(name, t["type"], t["data"], t["rows"], t["cols"])
    eng.finalize()
    ref = pkg.Engine.from_gguf(tiny_models[1])
    a, _ = eng.decode([5], [0])
    b, _ = ref.decode([5], [0])
    assert np.array_equal(a, b)
    eng.close()
    ref.close()


def test_step_trace_records(pkg, tiny_models, monkeypatch):
    """B200_TRACE=1: every matvec / attention launch of a step leaves eight ordered device timestamps."""
    monkeypatch.setenv("B200_TRACE", "1")
    eng = pkg.Engine.from_gguf(tiny_models[1])
    monkeypatch.delenv("B200_TRACE")
    eng.decode([3], [0])
    eng.decode([5], [1])
    t = eng.read_trace().astype(np.int64)
    L = eng.desc.num_hidden_layers
    assert len(t) == 3 + 5 * L  # embed | per layer: QKV, attention, O projection, gate/up, down | lm_head | select
    body = t[1:1 + 5 * L]
    assert (body > 0).all()
    assert (np.diff(body, axis=1) >= 0).all()          # entry <= inputs <= prologue <= end within a launch
    assert (np.diff(body[:, 0]) > 0).all()             # launches enter in stream order
    plain = pkg.Engine.from_gguf(tiny_models[1])
    with pytest.raises(RuntimeError):
        plain.read_trace()
    plain.close()
    eng.close()


@pytest.mark.parametrize("name,rows,cols", [("q4_k", 48, 8192), ("q6_k", 40, 14336), ("q4_k", 33, 28672), ("q6_k", 18, 28672),
                                            ("q8_0", 20, 8192)])
def test_matvec_long_rows_of_the_8b_and_70b_shapes(pkg, name, rows, cols):
    """Input widths of the 8B / 70B shapes: 32, 56 and 112 blocks per row (2, 4 and 7 stages per tile)."""
    typ = TYPES[name]
    w = pkg.synth.fill_normal(rows * cols, 31, rows + typ, 0.02)
    blocks = pkg.synth.quantize(typ, w)
    x = pkg.synth.fill_normal(cols, 32, cols, 1.0)
    wd = ol.dequant("oracle", typ, blocks).reshape(rows, cols)
    ref = ol.matvec_f32("oracle", wd, x)
    y = pkg.api.matvec(typ, blocks, rows, cols, x)
    assert rel_err(y, ref) <= 1e-3
    xs = pkg.synth.fill_normal(32 * cols, 33, cols, 1.0).reshape(32, cols)
    ref2 = (wd.astype(np.float64) @ xs.astype(np.float64).T).T
    y2 = pkg.api.matmul(typ, blocks, rows, cols, xs)
    assert np.abs(y2 - ref2).max() <= 1e-3 * np.abs(ref2).max()


@pytest.mark.parametrize("kv", ["f32", "i8"])
@pytest.mark.parametrize("shape,scheme", [("llama3-8b", 2), ("llama2-70b", 1)])
def test_two_layer_models_of_the_large_shapes(pkg, tmp_path, shape, scheme, kv):
    """Two layers of the 8B (GQA 32/8, FFN 14336, all Q6_K) and 70B (GQA 64/8, hidden 8192, FFN 28672, Q4_K_M-style)
    shapes with a small vocabulary: decode steps (matvec path) and a 20-token prompt (tensor-core path) against the
    oracle. With an INT8 cache the prompt tolerance is relative: fp16-level differences in K/V flip the rounding of
    some cached int8 values by one step, which moves the logits by about as much as the cache quantisation itself
    (measured 0.7 % of the largest logit; with an FP32 cache the same path stays below 2e-2 absolute)."""
    path = pkg.synth.write_gguf(str(tmp_path / "m.gguf"), shape, scheme=scheme, n_layers=2, vocab=4096, max_pos=256)
    i8 = kv == "i8"
    eng = pkg.Engine.from_gguf(path, kv_dtype=pkg.KV_I8 if i8 else pkg.KV_F32, max_seqs=2, max_ctx=64)
    orc = ol.OracleModel.from_gguf(path, kv_int8=i8, max_seqs=2)
    tok = 11
    for pos in range(3):
        logits, amax = eng.decode([tok], [pos])
        ref = orc.decode(tok, pos, seq=0)
        assert np.abs(logits[0] - ref).max() <= 2e-2
        assert int(amax[0]) == int(ref.argmax())
        tok = int(ref.argmax())
    ids = (np.arange(20, dtype=np.int32) * 37 + 5) % 4096
    got = eng.prefill(ids, slot=1)          # 20 tokens: the tensor-core path
    ref = orc.prefill(ids, seq=1)
    tol = 1.5e-2 * float(np.abs(ref).max()) if i8 else 2e-2
    assert np.abs(got - ref).max() <= tol
    eng.close()
