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
    q.put((rank, ok_rows and ok_mle and ok_zkip, parts, red))
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
