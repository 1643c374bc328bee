"""CPU, world_size 2 over gloo: the host logic of the multi-GPU paths."""
import os
import random
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, m, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    from tests.conftest import load_package
    load_package()
    from zkllm_ccs2024_b200 import sharding as S
    b, e = S.row_shard(m, world, rank)
    full = torch.arange(m * 36, dtype=torch.int32)
    got = S.all_gather_rows(full[b * 36:e * 36].clone(), m, 36)
    ok_rows = bool(torch.equal(got, full))
    rng = random.Random(100 + rank)
    parts = [rng.randrange(S.R_MOD) for _ in range(3)]
    red = S.fr_limbs_to_ints(S.fr_allreduce_sum(S.fr_ints_to_limbs(parts)))
    # a 64-element tensor in two blocks: block evaluations at the low challenges combine into the whole evaluation
    from oracle import pyref as R
    rs = random.Random(7)
    t = [rs.randrange(R.R_MOD) for _ in range(64)]
    u = [rs.randrange(R.R_MOD) for _ in range(6)]
    local = R.mle_eval(t[rank * 32:(rank + 1) * 32], u[:5])
    whole = S.fr_limbs_to_ints(S.sharded_mle_combine(S.fr_ints_to_limbs([local]), u[5:]))[0]
    ok_mle = whole == R.mle_eval(t, u)
    # inner-product sumcheck on 64-element vectors dealt out round-robin: local rounds, one exchange, shared last round
    a = [rs.randrange(R.R_MOD) for _ in range(64)]
    b = [rs.randrange(R.R_MOD) for _ in range(64)]
    claim = sum(x * y for x, y in zip(a, b)) % R.R_MOD
    la, lb, sums = a[rank::world], b[rank::world], []
    for r in range(S.zkip_local_rounds(len(la))):
        v, half = u[5 - r], len(la) // 2
        c = [0, 0, 0]
        for g in range(half):
            da, db = la[g + half] - la[g], lb[g + half] - lb[g]
            c = [c[0] + la[g] * lb[g], c[1] + la[g] * db + lb[g] * da, c[2] + da * db]
        sums += [x % R.R_MOD for x in c]
        la = [(la[g] + v * (la[g + half] - la[g])) % R.R_MOD for g in range(half)]
        lb = [(lb[g] + v * (lb[g + half] - lb[g])) % R.R_MOD for g in range(half)]
    polys, final = S.sharded_zkip(S.fr_ints_to_limbs(sums), S.fr_ints_to_limbs(la), S.fr_ints_to_limbs(lb), u, claim)
    proof = []
    ok_zkip = final == R.zkip(claim, a, b, u, proof) and polys == proof
    # multi-Hadamard sumcheck of three 64-element tensors dealt out the same way
    Xs = [[rs.randrange(R.R_MOD) for _ in range(64)] for _ in range(3)]
    vh = [rs.randrange(R.R_MOD) for _ in range(6)]
    eqw = [S.block_weight(u, i) for i in range(64)]
    hclaim = sum(eqw[i] * Xs[0][i] * Xs[1][i] * Xs[2][i] for i in range(64)) % R.R_MOD
    sums, tails = S.multi_hadamard_local_rounds([X[rank::world] for X in Xs], u[1:], vh[1:])
    hpolys, hfinal = S.sharded_multi_hadamard(sums, tails, u, vh, hclaim)
    hproof = []
    ok_had = hfinal == R.multi_hadamard_sumchecks(hclaim, Xs, u, vh, hproof) and hpolys == hproof
    q.put((rank, ok_rows and ok_mle and ok_zkip and ok_had, parts, red))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("m", [7, 8])
def test_row_sharding_and_field_allreduce(m):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, m, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    from tests.conftest import load_package
    load_package()
    from zkllm_ccs2024_b200 import sharding as S
    parts = {r: p for r, _, p, _ in res}
    exp = [(parts[0][i] + parts[1][i]) % S.R_MOD for i in range(3)]
    for rank, ok_rows, _, red in res:
        assert ok_rows, "gathered rows are not the full matrix in rank order"
        assert red == exp


def test_row_shard_covers_everything():
    from tests.conftest import load_package
    load_package()
    from zkllm_ccs2024_b200 import sharding as S
    for m in (0, 1, 5, 4096, 4097):
        for world in (1, 2, 3, 8):
            spans = [S.row_shard(m, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            assert max(e - b for b, e in spans) - min(e - b for b, e in spans) <= 1


def test_cpp_zkip_combine_matches_the_python_one():
    """zkb_zkip_combine is pure host arithmetic: it runs without a GPU and must agree with sharding.zkip_combine"""
    from tests.conftest import load_package
    z = load_package()
    from zkllm_ccs2024_b200 import sharding as S
    from oracle import pyref as R
    rng = random.Random(9)
    for n, world in ((64, 2), (64, 4), (32, 8), (16, 1)):
        k = n.bit_length() - 1
        a = [rng.randrange(R.R_MOD) for _ in range(n)]
        b = [rng.randrange(R.R_MOD) for _ in range(n)]
        u = [rng.randrange(R.R_MOD) for _ in range(k)]
        claim = sum(x * y for x, y in zip(a, b)) % R.R_MOD
        per_rank, flat = [], []
        for p in range(world):
            la, lb, sums = a[p::world], b[p::world], []
            for r in range(S.zkip_local_rounds(len(la))):
                v, half = u[k - 1 - r], len(la) // 2
                c = [0, 0, 0]
                for g in range(half):
                    da, db = la[g + half] - la[g], lb[g + half] - lb[g]
                    c = [c[0] + la[g] * lb[g], c[1] + la[g] * db + lb[g] * da, c[2] + da * db]
                sums.append([x % R.R_MOD for x in c])
                la = [(la[g] + v * (la[g + half] - la[g])) % R.R_MOD for g in range(half)]
                lb = [(lb[g] + v * (lb[g + half] - lb[g])) % R.R_MOD for g in range(half)]
            per_rank.append((sums, la, lb))
            flat += [c for row in sums for c in row] + la + lb
        want_polys, want_final = S.zkip_combine(per_rank, u, claim)
        polys, final = np.zeros((3 * k, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        z.call("zkb_zkip_combine", z._p(S.fr_ints_to_limbs(flat)), z.u32(world), z.u32(k), z._p(S.fr_ints_to_limbs(u)),
               z._p(S.fr_ints_to_limbs([claim])), z._p(polys), z._p(final))
        got = S.fr_limbs_to_ints(polys)
        assert [got[3 * r:3 * r + 3] for r in range(k)] == want_polys
        assert S.fr_limbs_to_ints(final)[0] == want_final
        # a wrong claim is refused with the reference's message
        with pytest.raises(z.ZkbError) as e:
            z.call("zkb_zkip_combine", z._p(S.fr_ints_to_limbs(flat)), z.u32(world), z.u32(k), z._p(S.fr_ints_to_limbs(u)),
                   z._p(S.fr_ints_to_limbs([claim + 1])), z._p(polys), z._p(final))
        assert "claim != p(0) + p(1)" in str(e.value)


def test_cpp_multi_hadamard_combine_matches_the_reference_algorithm():
    """zkb_multi_hadamard_combine is host arithmetic: per-rank blocks computed in Python go in, and the round polynomials of
    multi_hadamard_sumchecks on the whole tensors (oracle) must come out, for 1, 2, 4 and 8 ranks."""
    from tests.conftest import load_package
    z = load_package()
    from zkllm_ccs2024_b200 import sharding as S
    from oracle import pyref as R
    rng = random.Random(19)
    for n, K, world in ((32, 3, 2), (32, 2, 4), (16, 4, 8), (16, 1, 1), (8, 6, 8)):
        k = n.bit_length() - 1
        kP = world.bit_length() - 1
        Xs = [[rng.randrange(R.R_MOD) for _ in range(n)] for _ in range(K)]
        u = [rng.randrange(R.R_MOD) for _ in range(k)]
        v = [rng.randrange(R.R_MOD) for _ in range(k)]
        eqw = [S.block_weight(u, i) for i in range(n)]
        claim = 0
        for i in range(n):
            t = eqw[i]
            for X in Xs:
                t = t * X[i] % R.R_MOD
            claim = (claim + t) % R.R_MOD
        want = []
        want_final = R.multi_hadamard_sumchecks(claim, Xs, u, v, want)
        per_rank, flat = [], []
        for p in range(world):
            sums, tails = S.multi_hadamard_local_rounds([X[p::world] for X in Xs], u[kP:], v[kP:])
            per_rank.append((sums, tails))
            flat += [c for row in sums for c in row] + tails
        py_polys, py_final = S.multi_hadamard_combine(per_rank, u, v, claim)
        assert py_polys == want and py_final == want_final
        polys, final = np.zeros(((K + 1) * k, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        args = lambda c: (z._p(S.fr_ints_to_limbs(flat)), z.u32(world), z.u32(K), z.u32(k), z._p(S.fr_ints_to_limbs(u)),
                          z._p(S.fr_ints_to_limbs(v)), z._p(S.fr_ints_to_limbs([c])), z._p(polys), z._p(final))
        z.call("zkb_multi_hadamard_combine", *args(claim))
        got = S.fr_limbs_to_ints(polys)
        assert [got[(K + 1) * r:(K + 1) * (r + 1)] for r in range(k)] == want
        assert S.fr_limbs_to_ints(final)[0] == want_final
        with pytest.raises(z.ZkbError) as e:
            z.call("zkb_multi_hadamard_combine", *args(claim + 1))
        assert "multi_hadamard_sumchecks: claim != p(0) + p(1)" in str(e.value)


def _layer_split_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    import types
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
    import bench
    calls = []

    def fake_layer_workload(impl, modes, seq, embed, hidden, tmpdir=None, log=None, device=None, workdir=None, params_dir=None,
                            share=None):
        calls.append({"modes": modes, "workdir": workdir, "params_dir": params_dir, "share": share, "device": device})
        if not modes:                                   # the parameter set-up of rank 0
            Path(workdir, "marker").write_text("params")
            return {}
        assert Path(params_dir, "marker").read_text() == "params"
        return {"one resident driver process": {"seconds": 1.0 + share[0], "stages_s": {"ffn": 1.0 + share[0]},
                                                "passes_s": [2.0, 1.0 + share[0]], "outputs_sha256": "same"}}

    bench.layer_workload = fake_layer_workload
    args = types.SimpleNamespace(seq=256, embed=256, hidden=512, tmpdir=None, layer_log=None)
    out = bench.layer_split_over_ranks(dist, rank, world, str(rank), args)
    q.put((rank, out, calls))
    dist.barrier()
    dist.destroy_process_group()


def test_layer_split_over_two_ranks_host_logic():
    """bench.layer_split_over_ranks with the driver replaced by a stub: rank 0 sets the parameters up once where both can
    read them, every rank proves as process r of 2 against that directory, the slowest rank's time is the layer's, the
    output digests are compared, and the shared directory is gone afterwards."""
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_layer_split_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {r: (out, calls) for r, out, calls in (q.get(timeout=120) for _ in range(world))}
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        out, calls = res[r]
        assert out["seconds"] == 2.0 and out["seconds_per_gpu"] == [1.0, 2.0]
        assert out["all_gpus_wrote_the_same_outputs"] is True and out["parity"] is None      # no recorded digest for this shape
        prove = [c for c in calls if c["modes"]]
        assert len(prove) == 1 and prove[0]["share"] == (r, world) and prove[0]["device"] == str(r)
        assert len([c for c in calls if not c["modes"]]) == (1 if r == 0 else 0)
    shared = res[0][1][0]["workdir"]
    assert res[1][1][0]["params_dir"] == shared and not os.path.exists(shared)
