"""Writes tests/golden/oracle_fullsize.json: every round polynomial and claim of the two sumcheck
benchmark configurations at FULL size, computed by the CPU restatement oracle/zkoracle.cpp on the
seeded inputs of bench.zkfc_inputs() / bench.tlookup_inputs():

    python tests/golden/make_fullsize_oracle.py          # about two minutes of CPU, no GPU

zkFC::prove on X 128x4096, W 4096x4096 (12 rounds of 3 coefficients, 4 claims) and tLookup::prove on
2^23 values in a 2^16 range table (23 rounds of 4 coefficients, final claim).  The final claims of
both also equal the ones recorded from the reference's own CUDA build (ref_fullsize.json).
tests/test_gpu_fullsize.py compares the CUDA library with these values coefficient by coefficient."""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402
from oracle import cpporacle as C  # noqa: E402


def hexes(a: np.ndarray) -> list:
    return [bytes(row).hex() for row in np.ascontiguousarray(a, dtype=np.uint32).reshape(-1, 8)]


def main():
    out = {"source": "oracle/zkoracle.cpp (CPU restatement) on the seeded inputs of bench.zkfc_inputs() / bench.tlookup_inputs(); "
                     "values are 32-byte little-endian hex"}
    X, W, Y, ub, ui, uo = bench.zkfc_inputs()
    B, I, O = bench.ZKFC_SHAPE
    rc, polys, claims = C.zkfc_prove(bench.ints_to_fr_limbs(X), bench.ints_to_fr_limbs(W), bench.ints_to_fr_limbs(Y), B, I, O, ub, ui, uo)
    assert rc == 0
    out["zkfc_prove"] = {"polys": hexes(polys), "claims": hexes(claims)}
    S, alpha, beta, u, v = bench.tlookup_inputs()
    T = bench.ints_to_fr_limbs(np.arange(bench.TL_LOW, bench.TL_LOW + bench.TL_N, dtype=np.int64))
    m = bench.ints_to_fr_limbs(np.bincount(S.astype(np.int64) - bench.TL_LOW, minlength=bench.TL_N).astype(np.int64))
    rc, polys, final = C.tlookup_prove(bench.ints_to_fr_limbs(S.astype(np.int64)), T, m, alpha, beta, u, v)
    assert rc == 0
    out["tlookup_prove"] = {"polys": hexes(polys), "final": hexes(final)}
    path = ROOT / "tests" / "golden" / "oracle_fullsize.json"
    path.write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {path}")


if __name__ == "__main__":
    main()
