"""The allocation-free attention entry point against the ordinary one.

b200_attention_decode_noalloc is for callers that cannot allocate device memory when they call
(memory comes from a pool sized once at start-up, the allocator is frozen after initialisation,
there is no room for cudaMalloc in the latency budget): they pass device buffers they already own and the library uses its built-in scratch.
This file sorts last on purpose, so that a run that stops at the first failure has already been
through every other test. It holds device memory through torch only because the test needs some
owner for the buffers; the entry point itself never sees torch.
"""
import numpy as np
import pytest

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def _case(pkg, seed, nq, nkv, hd, n_ctx, splits):
    import torch
    rng = np.random.default_rng(seed)
    q = rng.standard_normal(nq * hd).astype(np.float32)
    kc = rng.standard_normal((n_ctx + 1, nkv, hd)).astype(np.float32)
    vc = rng.standard_normal((n_ctx + 1, nkv, hd)).astype(np.float32)
    ref = pkg.api.attention_decode(q, kc[-1], vc[-1], kc[:-1], vc[:-1], nq, nkv, hd, kv_dtype=pkg.KV_F32, n_splits=splits)
    max_ctx = n_ctx + 5
    dev = torch.device("cuda", 0)
    # the engine's cache layout: [kv_head][position][head_dim]
    kcache = torch.zeros((nkv, max_ctx, hd), dtype=torch.float32, device=dev)
    vcache = torch.zeros((nkv, max_ctx, hd), dtype=torch.float32, device=dev)
    kcache[:, :n_ctx] = torch.from_numpy(kc[:-1].transpose(1, 0, 2).copy()).to(dev)
    vcache[:, :n_ctx] = torch.from_numpy(vc[:-1].transpose(1, 0, 2).copy()).to(dev)
    d_q = torch.from_numpy(q).to(dev)
    d_new = torch.from_numpy(np.concatenate([kc[-1].ravel(), vc[-1].ravel()])).to(dev)
    d_pos = torch.tensor([n_ctx], dtype=torch.int32, device=dev)
    d_out = torch.empty(nq * hd, dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    pkg.api.attention_decode_noalloc(d_q.data_ptr(), d_new.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), None, None,
                                     d_pos.data_ptr(), nq, nkv, hd, max_ctx, pkg.KV_F32, splits, d_out.data_ptr(), None)
    torch.cuda.synchronize()
    out = d_out.cpu().numpy()
    # the call also appended the new row to the caches
    assert np.array_equal(kcache[:, n_ctx].cpu().numpy(), kc[-1])
    assert np.array_equal(vcache[:, n_ctx].cpu().numpy(), vc[-1])
    return out, ref


def test_noalloc_matches_regular_entry_point_twice(pkg):
    # two calls in a row with different shapes: the second one finds the first one's scratch contents
    out1, ref1 = _case(pkg, 1, nq=8, nkv=2, hd=128, n_ctx=300, splits=8)
    assert np.abs(out1 - ref1).max() <= 2e-5 * max(1.0, np.abs(ref1).max())
    out2, ref2 = _case(pkg, 2, nq=32, nkv=4, hd=64, n_ctx=77, splits=5)
    assert np.abs(out2 - ref2).max() <= 2e-5 * max(1.0, np.abs(ref2).max())
    out3, ref3 = _case(pkg, 1, nq=8, nkv=2, hd=128, n_ctx=300, splits=8)
    assert np.array_equal(out3, out1)


def test_noalloc_rejects_oversize(pkg):
    with pytest.raises(pkg.B200Error, match="exceeds the built-in scratch"):
        pkg.api.attention_decode_noalloc(1, 1, 1, 1, None, None, 1, 128, 128, 128, 64, pkg.KV_F32, 32, 1, None)
    with pytest.raises(pkg.B200Error, match="exceeds the built-in scratch"):
        pkg.api.attention_decode_noalloc(1, 1, 1, 1, None, None, 1, 4, 4, 256, 64, pkg.KV_F32, 2, 1, None)


def _quantize_rows(rows):
    """[n][hd] FP32 -> (int8 rows, FP32 scales) with the oracle's restatement of the reference quantizer."""
    n, hd = rows.shape
    q = np.empty((n, hd), np.int8)
    sc = np.empty(n, np.float32)
    for i in range(n):
        r = np.ascontiguousarray(rows[i])
        one = np.empty(1, np.float32)
        ol.oracle().orc_kv_quantize_i8(ol._p(r), hd, ol._p(q[i]), ol._p(one))
        sc[i] = one[0]
    return q, sc


@pytest.mark.parametrize("kv_i8", [False, True])
def test_noalloc_against_the_oracle(pkg, kv_i8):
    """The same entry point checked directly against the CPU oracle's attention (not only against the other CUDA
    entry point), with an FP32 and with an INT8 cache that the test fills itself."""
    import torch
    nq, nkv, hd, n_ctx, splits = 8, 4, 64, 203, 6
    rng = np.random.default_rng(11)
    q = rng.standard_normal(nq * hd).astype(np.float32)
    kc = rng.standard_normal((n_ctx + 1, nkv, hd)).astype(np.float32)
    vc = rng.standard_normal((n_ctx + 1, nkv, hd)).astype(np.float32)
    ref = ol.attention_decode(q, kc, vc, nq, nkv, hd, kv_int8=kv_i8)
    max_ctx = n_ctx + 3
    dev = torch.device("cuda", 0)
    d_q = torch.from_numpy(q).to(dev)
    d_new = torch.from_numpy(np.concatenate([kc[-1].ravel(), vc[-1].ravel()])).to(dev)
    d_pos = torch.tensor([n_ctx], dtype=torch.int32, device=dev)
    d_out = torch.empty(nq * hd, dtype=torch.float32, device=dev)
    if kv_i8:
        kq = torch.zeros((nkv, max_ctx, hd), dtype=torch.int8, device=dev)
        vq = torch.zeros((nkv, max_ctx, hd), dtype=torch.int8, device=dev)
        ks = torch.zeros((nkv, max_ctx), dtype=torch.float32, device=dev)
        vs = torch.zeros((nkv, max_ctx), dtype=torch.float32, device=dev)
        for h in range(nkv):
            a, b = _quantize_rows(kc[:-1, h])
            kq[h, :n_ctx], ks[h, :n_ctx] = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
            a, b = _quantize_rows(vc[:-1, h])
            vq[h, :n_ctx], vs[h, :n_ctx] = torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)
        args = (kq.data_ptr(), vq.data_ptr(), ks.data_ptr(), vs.data_ptr())
    else:
        kf = torch.zeros((nkv, max_ctx, hd), dtype=torch.float32, device=dev)
        vf = torch.zeros((nkv, max_ctx, hd), dtype=torch.float32, device=dev)
        kf[:, :n_ctx] = torch.from_numpy(kc[:-1].transpose(1, 0, 2).copy()).to(dev)
        vf[:, :n_ctx] = torch.from_numpy(vc[:-1].transpose(1, 0, 2).copy()).to(dev)
        args = (kf.data_ptr(), vf.data_ptr(), None, None)
    torch.cuda.synchronize()
    pkg.api.attention_decode_noalloc(d_q.data_ptr(), d_new.data_ptr(), *args, d_pos.data_ptr(), nq, nkv, hd, max_ctx,
                                     pkg.KV_I8 if kv_i8 else pkg.KV_F32, splits, d_out.data_ptr(), None)
    torch.cuda.synchronize()
    out = d_out.cpu().numpy()
    assert np.abs(out - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())
    if kv_i8:  # the appended row was quantised like the oracle does it
        a, b = _quantize_rows(kc[-1])
        assert np.array_equal(kq[:, n_ctx].cpu().numpy(), a)
        assert np.array_equal(ks[:, n_ctx].cpu().numpy(), b)
    # a position outside the cache: nothing is appended, the output is NaN (the host cannot see the value)
    guard_k = (kq if kv_i8 else kf).clone()
    d_pos.fill_(max_ctx)
    pkg.api.attention_decode_noalloc(d_q.data_ptr(), d_new.data_ptr(), *args, d_pos.data_ptr(), nq, nkv, hd, max_ctx,
                                     pkg.KV_I8 if kv_i8 else pkg.KV_F32, splits, d_out.data_ptr(), None)
    torch.cuda.synchronize()
    assert torch.isnan(d_out).all()
    assert torch.equal(guard_k, kq if kv_i8 else kf)


def test_noalloc_rejects_bad_arguments(pkg):
    with pytest.raises(pkg.B200Error, match="head_dim must be"):
        pkg.api.attention_decode_noalloc(1, 1, 1, 1, None, None, 1, 4, 4, 96, 64, pkg.KV_F32, 2, 1, None)
    with pytest.raises(pkg.B200Error, match="kv_dtype"):
        pkg.api.attention_decode_noalloc(1, 1, 1, 1, None, None, 1, 4, 4, 64, 64, 7, 2, 1, None)
