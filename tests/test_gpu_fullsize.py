"""GPU: the benchmark configurations at FULL size.

* zkFC::prove on X 128x4096, W 4096x4096 and tLookupRange prep + prove on 2^23 values in a 2^16 table: every round
  polynomial against the CPU restatement at full size (tests/golden/oracle_fullsize.json, written by
  tests/golden/make_fullsize_oracle.py) and the final claims against the reference's own CUDA build
  (tests/golden/ref_fullsize.json);
* commit_int of the 4096 x 11008 benchmark matrix: SHA-256 over all 4096 affine-normalised points against the value the
  reference's build printed for the same inputs, for both algorithms of the library;
* one Llama-2-7B-shape decoder layer through the resident stage driver: SHA-256 over every integer output file
  against the reference's own drivers."""
import ctypes
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).parent / "golden"
GOLD = json.loads((GOLDEN / "ref_fullsize.json").read_text())
ORACLE = json.loads((GOLDEN / "oracle_fullsize.json").read_text())


def _be(hex_le: str) -> str:
    return "0x" + bytes.fromhex(hex_le)[::-1].hex()


def _hexes(a: np.ndarray) -> list:
    return [bytes(row).hex() for row in np.ascontiguousarray(a, dtype=np.uint32).reshape(-1, 8)]


def test_full_size_final_claims_equal_the_reference(zkb):
    torch = pytest.importorskip("torch")
    import bench
    out = bench.sumcheck_ours(zkb, torch, 1, 6454.9)
    assert _be(out["zkfc_prove"]["final_claim"]) == GOLD["zkfc_prove_final_claim_be"]
    assert _be(out["tlookup_prove"]["final_claim"]) == GOLD["tlookup_prove_final_claim_be"]


def test_full_size_zkfc_round_polynomials(zkb):
    import bench
    z = zkb
    B, I, O = bench.ZKFC_SHAPE
    X, W, Y, ub, ui, uo = bench.zkfc_inputs()
    dX, dW, dY = (z.fr_buffer(bench.ints_to_fr_limbs(t)) for t in (X, W, Y))
    polys, claims = np.zeros((36, 8), dtype=np.uint32), np.zeros((4, 8), dtype=np.uint32)
    z.call("zkb_zkfc_prove", z._p(dX), z._p(dW), z._p(dY), z.sz(B), z.sz(I), z.sz(O), z._p(ub), z._p(ui), z._p(uo), z._p(polys),
           z._p(claims), z._p(0))
    assert _hexes(polys) == ORACLE["zkfc_prove"]["polys"]
    assert _hexes(claims) == ORACLE["zkfc_prove"]["claims"]
    assert _be(_hexes(claims)[1]) == GOLD["zkfc_prove_final_claim_be"]


@pytest.mark.parametrize("indexed", [False, True])
def test_full_size_tlookup_round_polynomials(zkb, indexed):
    import bench
    z = zkb
    S, alpha, beta, u, v = bench.tlookup_inputs()
    D, N, low = bench.TL_D, bench.TL_N, bench.TL_LOW
    dS = z.fr_buffer(bench.ints_to_fr_limbs(S.astype(np.int64)))
    dT, dI, dM = z.DeviceBuffer(32 * N), z.DeviceBuffer(4 * D), z.DeviceBuffer(32 * N)
    z.call("zkb_tlookup_range_table", z.i32(low), z.sz(N), z.sz(N), z._p(dT), z._p(0))
    z.call("zkb_tlookup_range_indices", z._p(dS), z.i32(low), z._p(dI), z.sz(D), z._p(0))
    z.call("zkb_tlookup_prep", z._p(dI), z.sz(D), z.sz(N), z._p(dM), z._p(0))
    polys, final = np.zeros((4 * 23, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    if indexed:
        z.call("zkb_tlookup_prove_indexed", z._p(dS), z._p(dI), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u),
               z._p(v), z._p(polys), z._p(final), z._p(0))
    else:
        z.call("zkb_tlookup_prove", z._p(dS), z._p(dT), z._p(dM), z.sz(D), z.sz(N), z._p(alpha), z._p(beta), z._p(u), z._p(v),
               z._p(polys), z._p(final), z._p(0))
    assert _hexes(polys) == ORACLE["tlookup_prove"]["polys"]
    assert _hexes(final) == ORACLE["tlookup_prove"]["final"]
    assert _be(_hexes(final)[0]) == GOLD["tlookup_prove_final_claim_be"]


@pytest.mark.parametrize("method", [0, 1, 2])     # the library's choice, buckets, combination tables
def test_commit_4096x11008_equals_the_reference(zkb, method):
    import bench
    from oracle import cpporacle as C
    z = zkb
    m, n = 4096, 11008
    gs = bench.generator_scalars(n)
    gens = z.DeviceBuffer(144 * n)
    z.call("zkb_g1_mul", z._p(z.DeviceBuffer.from_host(bench.g1_generator_limbs())), z.sz(1), z._p(z.DeviceBuffer.from_host(gs)), z.sz(n),
           z._p(gens), z._p(0))
    d_sc = z.DeviceBuffer.from_host(bench.weights(m, n, bench.SEED + 2))
    out = z.DeviceBuffer(144 * m)
    z.call("zkb_commit_i32_method", z._p(gens), z.sz(n), z._p(d_sc), z.sz(m * n), z._p(out), ctypes.c_int(method), z._p(0))
    z.call("zkb_sync", z._p(0))
    sha = hashlib.sha256(C.g1_normalise(out.to_host(np.uint32, (m, 36))).tobytes()).hexdigest()
    assert sha == GOLD["commit_int_4096x11008_sha256"]


def test_layer_7b_outputs_equal_the_reference_drivers(tmp_path):
    import bench
    gold = GOLD.get("layer_7b_outputs_sha256")
    assert gold, "tests/golden/ref_fullsize.json has no layer_7b_outputs_sha256"
    blk = bench.layer_workload("ours", [("batch", 1)], 2048, 4096, 11008, str(tmp_path))
    assert "unavailable" not in blk, blk
    got = blk["one resident driver process"]
    assert got["outputs_sha256"] == gold, got["output_files_sha256_16"]


def test_layer_13b_outputs_equal_the_reference_drivers(tmp_path):
    import bench
    gold = GOLD.get("layer_13b_outputs_sha256")
    assert gold, "tests/golden/ref_fullsize.json has no layer_13b_outputs_sha256"
    blk = bench.layer_workload("ours", [("batch", 1)], 2048, 5120, 13824, str(tmp_path))
    assert "unavailable" not in blk, blk
    got = blk["one resident driver process"]
    assert got["outputs_sha256"] == gold, got["output_files_sha256_16"]


def test_layer_7b_proofs_shared_by_two_driver_processes(tmp_path):
    """ZKLLM_PROOF_WORLD=2: both driver processes write the reference's outputs, every proof of the layer is run by
    exactly one of them, and each process reports its share.  (Run one after the other here: they exchange nothing.)"""
    import re
    import bench
    gold = GOLD.get("layer_7b_outputs_sha256")
    params = tmp_path / "params"
    params.mkdir()
    bench.layer_workload("ours", [], 2048, 4096, 11008, workdir=str(params))
    proofs, dealt = [], set()
    for r in range(2):
        log = tmp_path / f"driver{r}.log"
        blk = bench.layer_workload("ours", [("batch", 1)], 2048, 4096, 11008, str(tmp_path), log=str(log), params_dir=str(params),
                                   share=(r, 2))
        assert blk["one resident driver process"]["outputs_sha256"] == gold
        m = re.search(r"\[share\] process (\d) of 2: (\d+) of (\d+) proofs", log.read_text())
        assert m and int(m.group(1)) == r, log.read_text()[-600:]
        proofs.append(int(m.group(2)))
        dealt.add(int(m.group(3)))
    assert len(dealt) == 1 and sum(proofs) == dealt.pop() and min(proofs) > 0
