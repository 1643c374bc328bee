"""GPU: the softmax element kernels (zkb_softmax_shift / _decompose / _table) against values
recorded from the reference's own CUDA build: the small case of tests/golden/ref_golden.json in
full, and 16 rows of 2048 columns with d = 4096 (the layer's shape, where the row shift is a
2048-term left-to-right double-precision sum, zksoftmax.cu:20-32) by the recorded shifts and
SHA-256 digests of the digit and table-output tensors (tests/golden/ref_fullsize.json)."""
import ctypes
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import pyref as R

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"
BS = [1 << 8, 1 << 20, 1 << 20]
THETAS = [float(1 << 18), float(1 << 22)]
SF = float(1 << 32)


def softmax_parts(z, X, m, n, d):
    """shift, digits and table outputs as zkSoftmax::compute forms them (zksoftmax.cu:111-170), through the C ABI"""
    N = m * n
    dX = z.fr_buffer(R.fr_pack([R.int_to_fr(int(x)) for x in X]))
    d_shift, d_out, d_digits = z.DeviceBuffer(32 * m), z.DeviceBuffer(32 * N), z.DeviceBuffer(32 * N * 3)
    z.call("zkb_softmax_shift", z._p(dX), z._p(d_shift), z._p(d_out), z.sz(m), z.sz(n), ctypes.c_double(SF), ctypes.c_double(d), z._p(0))
    z.call("zkb_softmax_decompose", z._p(d_out), z._p(np.array(BS, dtype=np.uint32)), z.u32(3), z._p(d_digits), z.sz(N), z._p(0))
    z.call("zkb_sync", z._p(0))
    shift = R.fr_unpack(d_shift.to_host(np.uint32, (m, 8)))
    digits = R.fr_unpack(d_digits.to_host(np.uint32, (3 * N, 8)))
    xseg = [digits[k * N:(k + 1) * N] for k in range(3)]
    yseg, weight = [], 1
    for k in range(3):
        if k >= 1:
            table = z.DeviceBuffer(32 * BS[k])
            z.call("zkb_softmax_table", ctypes.c_double(THETAS[k - 1]), ctypes.c_double(SF), ctypes.c_double(d), ctypes.c_double(weight),
                   z.u32(BS[k]), z._p(table), z._p(0))
            z.call("zkb_sync", z._p(0))
            tv = table.to_host(np.uint32, (BS[k], 8))
            picked = tv[np.array(xseg[k], dtype=np.int64)]
            yseg.append(R.fr_unpack(np.ascontiguousarray(picked)))
        weight *= BS[k]
    y = [a * b % R.R_MOD for a, b in zip(*yseg)]
    return shift, xseg, yseg, y


def digest(vals) -> str:
    return hashlib.sha256(b"".join(int(v).to_bytes(32, "little") for v in vals)).hexdigest()


def test_softmax_small_case_equals_the_reference(zkb):
    gold = json.loads((GOLDEN / "ref_golden.json").read_text())
    (c,) = [c for c in gold["cases"] if c["kind"] == "softmax"]
    i, o = c["in"], c["out"]
    H = lambda xs: [int(x, 16) for x in xs]
    shift, xseg, yseg, y = softmax_parts(zkb, i["X"], i["m"], i["n"], i["d"])
    assert shift == H(o["shift"])
    for k in range(3):
        assert xseg[k] == H(o[f"xseg{k}"]), k
    for k in range(2):
        assert yseg[k] == H(o[f"yseg{k}"]), k
    assert y == H(o["y"])


def test_softmax_2048_columns_equals_the_reference(zkb):
    gold = json.loads((GOLDEN / "ref_fullsize.json").read_text()).get("softmax_16x2048_d4096")
    assert gold, "tests/golden/ref_fullsize.json has no softmax_16x2048_d4096 (python tests/golden/make_golden.py --fullsize)"
    from tests.golden.make_golden import softmax_large_inputs
    m, n, d = gold["m"], gold["n"], gold["d"]
    shift, xseg, yseg, y = softmax_parts(zkb, softmax_large_inputs(m, n, d), m, n, d)
    assert shift == [int(x, 16) for x in gold["shift"]]
    for k in range(3):
        assert digest(xseg[k]) == gold[f"xseg{k}_sha256"], k
    for k in range(2):
        assert digest(yseg[k]) == gold[f"yseg{k}_sha256"], k
    assert digest(y) == gold["y_sha256"]
