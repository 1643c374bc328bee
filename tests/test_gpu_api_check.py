"""GPU: the parts of the class API that no stage driver reaches - zkip_stacked / zkFCStacked, zkAttn / zkAttnStacked, zkReLU.

oracle/api_check.cu uses only the public class API; it is built twice, against this repository's host library
(oracle/_build/api_check, `make -C oracle api`) and against the reference's own CUDA sources (oracle/_ref/api_check_ref, present where the
reference was available at build time).  Both print the round polynomials and final claims of the same seeded inputs.
The library's output must equal the lines recorded from the reference build (tests/golden/api_check_<case>.txt) and,
when the reference build is present, what that build prints now.  Every prove() also checks its own verifier equations.
"""
import hashlib
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
OURS = ROOT / "oracle" / "_build" / "api_check"
REF = ROOT / "oracle" / "_ref" / "api_check_ref"
GOLDEN = ROOT / "tests" / "golden"


def squeeze(line: str) -> str:
    """a long line (a whole tensor) is kept as its key and the SHA-256 of its text"""
    if len(line) <= 4096:
        return line
    return line.split(" ")[0] + " sha256:" + hashlib.sha256(line.encode()).hexdigest()


def run(exe: Path, case: str) -> list:
    res = subprocess.run([str(exe), case], capture_output=True, text=True, timeout=1200)
    assert res.returncode == 0, f"{exe.name} {case}: {res.stdout[-1500:]}\n{res.stderr[-1500:]}"
    return [squeeze(ln) for ln in res.stdout.splitlines() if ln.split(" ")[0].startswith(("poly", "final", "out", "ok"))]


@pytest.mark.parametrize("case", ["fcstacked", "attn", "attnstacked", "relu", "misc"])
def test_class_api_matches_the_reference_build(case):
    assert OURS.exists(), "oracle/_build/api_check is missing: run make -C oracle api"
    ours = run(OURS, case)
    assert ours and ours[-1] == "ok 1"
    golden = GOLDEN / f"api_check_{case}.txt"
    assert golden.exists(), f"{golden} is missing"
    assert ours == golden.read_text().splitlines(), "output differs from the lines recorded from the reference build"
    if REF.exists():
        assert ours == run(REF, case), "output differs from the reference build run now"
