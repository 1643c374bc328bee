"""GPU: the two sumcheck benchmark configurations at full size against final claims
recorded from the reference's own CUDA build on the same seeded inputs
(tests/golden/ref_fullsize.json): zkFC::prove on X 128x4096, W 4096x4096 and
tLookupRange prep + prove on 2^23 values in a 2^16 table."""
import json
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

GOLD = json.loads((Path(__file__).parent / "golden" / "ref_fullsize.json").read_text())


def _be(hex_le: str) -> str:
    return "0x" + bytes.fromhex(hex_le)[::-1].hex()


def test_full_size_final_claims_equal_the_reference(zkb):
    torch = pytest.importorskip("torch")
    import bench
    out = bench.sumcheck_ours(zkb, torch, 1, 6454.9)
    assert _be(out["zkfc_prove"]["final_claim"]) == GOLD["zkfc_prove_final_claim_be"]
    assert _be(out["tlookup_prove"]["final_claim"]) == GOLD["tlookup_prove_final_claim_be"]
