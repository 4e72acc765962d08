"""Tensor-parallel engines (one process per GPU; one-shot all-reduce over peer memory, or NCCL) against the CPU oracle.
Needs two GPUs; skipped otherwise."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rank(rank, world, path, id_q, out_q, kv_i8, fused):
    import os
    os.environ["B200_TP_FUSED"] = "1" if fused else "0"  # peer-memory exchange inside the matvec kernels, or ncclAllReduce
    import __graft_entry__
    pkg = __graft_entry__.load_package()
    if rank == 0:
        nid = pkg.api.nccl_unique_id()
        for _ in range(world - 1):
            id_q.put(nid)
    else:
        nid = id_q.get(timeout=120)
    eng = pkg.Engine.from_gguf(path, kv_dtype=pkg.KV_I8 if kv_i8 else pkg.KV_F32, max_seqs=2, device=rank, tp_rank=rank,
                               tp_size=world, nccl_id=nid)
    logs = []
    tok = 7
    for pos in range(12):
        logits, amax = eng.decode([tok], [pos])
        logs.append(logits[0].copy())
        tok = int(amax[0])
    # two sequences at once, second slot fresh
    lg2, am2 = eng.decode([tok, 9], [12, 0], slots=[0, 1])
    gen, _ = eng.generate_greedy([int(am2[0]), int(am2[1])], [13, 1], 6, slots=[0, 1])
    out_q.put((rank, np.stack(logs), lg2, gen))
    eng.close()


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("kv_i8", [False, True])
def test_tp2_matches_oracle(pkg, tmp_path, kv_i8, fused):
    if pkg.api.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    import oracle_lib as ol
    path = pkg.synth.write_gguf(str(tmp_path / "mha.gguf"), "tiny_mha", scheme=1, norm_random=True)
    ctx = mp.get_context("spawn")
    id_q, out_q = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 2, path, id_q, out_q, kv_i8, fused)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted((out_q.get(timeout=300) for _ in procs), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    orc = ol.OracleModel.from_gguf(path, kv_int8=kv_i8, max_seqs=2)
    tok = 7
    for pos in range(12):
        ref = orc.decode(tok, pos)
        for r in range(2):
            assert np.abs(res[r][1][pos] - ref).max() <= 2e-2
            assert int(res[r][1][pos].argmax()) == int(ref.argmax())
        tok = int(ref.argmax())
    ref0, ref1 = orc.decode(tok, 12, seq=0), orc.decode(9, 0, seq=1)
    for r in range(2):
        assert np.abs(res[r][2][0] - ref0).max() <= 2e-2 and np.abs(res[r][2][1] - ref1).max() <= 2e-2
    assert np.array_equal(res[0][3], res[1][3])  # both ranks sample the same tokens
    t0, t1 = int(ref0.argmax()), int(ref1.argmax())
    for s in range(6):
        t0, t1 = int(orc.decode(t0, 13 + s, seq=0).argmax()), int(orc.decode(t1, 1 + s, seq=1).argmax())
        assert res[0][3][s].tolist() == [t0, t1]
