"""CPU: the accounting helpers of bench.py (no GPU, no library calls)."""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_table_method_windows_matches_the_library_rule():
    # msm_comb.cuh: the smallest W with max_abs <= (3 * 8^W - 3) / 7
    assert bench.table_method_windows(0) == 1
    assert bench.table_method_windows(3) == 1 and bench.table_method_windows(4) == 2
    assert bench.table_method_windows(14043) == 5 and bench.table_method_windows(14044) == 6
    assert bench.table_method_windows(8127) == 5
    assert bench.table_method_windows(2 ** 31) == 11


def test_table_method_additions_counts_nonzero_groups():
    rng = np.random.Generator(np.random.PCG64(3))
    m, n = 7, 10                                   # a ragged last group of two generators
    sc = rng.integers(-8000, 8000, size=(m, n)).astype(np.int32)
    sc[0, :4] = 0                                  # a group whose digits are zero in every window
    sc[1, 4:8] = [1, 0, 0, 0]                      # non-zero only in the lowest window
    W = bench.table_method_windows(int(np.abs(sc).max()))
    bias = sum(4 << (3 * w) for w in range(W))
    expect = 0
    for r in range(m):
        for q in range((n + 3) // 4):
            cols = [int(sc[r, c]) if c < n else 0 for c in range(4 * q, 4 * q + 4)]
            for w in range(W):
                digits = [((v + bias) >> (3 * w)) & 7 for v in cols]
                expect += any(d != 4 for d in digits)
    assert bench.table_method_additions(sc.reshape(-1), m, n, W) == expect


def test_row_shard_covers_all_rows_once():
    for m, world in ((4096, 8), (9, 2), (5, 8), (0, 3)):
        blocks = [bench.row_shard(m, world, r) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == m
        assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
        sizes = [e - b for b, e in blocks]
        assert max(sizes) - min(sizes) <= 1


def test_both_arms_name_the_workload_alike():
    cfg = bench.bench_config(4096, 11008)
    assert set(cfg) == {"workload", "rows", "generators", "seed", "l2"}
    json.dumps(cfg)


def test_fullsize_fixtures_are_present_and_consistent():
    gold = bench.golden_fullsize()
    for key in ("commit_int_4096x11008_sha256", "layer_7b_outputs_sha256", "zkfc_prove_final_claim_be", "tlookup_prove_final_claim_be",
                "softmax_16x2048_d4096"):
        assert key in gold, key
    oracle = json.loads((ROOT / "tests" / "golden" / "oracle_fullsize.json").read_text())
    assert len(oracle["zkfc_prove"]["polys"]) == 36 and len(oracle["tlookup_prove"]["polys"]) == 92
    # the CPU restatement's final claims are the reference build's
    be = lambda h: "0x" + bytes.fromhex(h)[::-1].hex()
    assert be(oracle["zkfc_prove"]["claims"][1]) == gold["zkfc_prove_final_claim_be"]
    assert be(oracle["tlookup_prove"]["final"][0]) == gold["tlookup_prove_final_claim_be"]
