"""GPU: the guard bands of the library's allocator (zkb_guard_enable / ZKLLM_GUARD=1), which stand in for a memory checker.

While the guard is on, every scratch block and every zkb_malloc buffer has 256 bytes of a fixed pattern before and after it,
compared with the pattern when the block is released.  The first test shows that the detector sees a store just outside a
buffer (the stores land in the bands, which are the library's own valid memory: nothing faults).  The second runs tiny, odd
and ragged shapes of every prover under the guard and expects every band intact.  The whole GPU suite can be run the same way:
ZKLLM_GUARD=1 python -m pytest tests -m gpu  (tests/conftest.py fails the session if a band was written)."""
import ctypes
import os

import numpy as np
import pytest

from tests.util import Dev

pytestmark = pytest.mark.gpu

SESSION_WIDE = os.environ.get("ZKLLM_GUARD") == "1"


def _report(z, reset):
    blocks, damaged, first = ctypes.c_ulonglong(), ctypes.c_ulonglong(), ctypes.c_ulonglong()
    side = ctypes.c_int()
    z.call("zkb_guard_report", ctypes.byref(blocks), ctypes.byref(damaged), ctypes.byref(first), ctypes.byref(side), ctypes.c_int(reset))
    return blocks.value, damaged.value, first.value, side.value


@pytest.mark.skipif(SESSION_WIDE, reason="writes into guard bands on purpose; the session-wide check would count it")
def test_a_store_outside_a_buffer_is_seen(zkb):
    z = zkb
    z.call("zkb_guard_enable", ctypes.c_int(1))
    try:
        _report(z, 1)
        word = np.array([0x12345678], dtype=np.uint32)
        clean = z.DeviceBuffer(40)
        past_end = z.DeviceBuffer(40)        # one word past the end: the first word of the band after the buffer
        z.call("zkb_memcpy_h2d", z._p(past_end.ptr + 40), z._p(word), z.sz(4), z._p(0))
        clean.free()
        past_end.free()
        assert _report(z, 1) == (2, 1, 40, 1)
        before_start = z.DeviceBuffer(1000)  # one word before the start
        z.call("zkb_memcpy_h2d", z._p(before_start.ptr - 4), z._p(word), z.sz(4), z._p(0))
        before_start.free()
        assert _report(z, 1) == (1, 1, 1000, 0)
        odd = z.DeviceBuffer(18)             # sizes are rounded up to a word: bytes 18 and 19 are slack, byte 20 is the band
        z.call("zkb_memcpy_h2d", z._p(odd.ptr + 20), z._p(word), z.sz(4), z._p(0))
        odd.free()
        assert _report(z, 1)[1] == 1
    finally:
        z.call("zkb_guard_enable", ctypes.c_int(0))
        _report(z, 1)


def test_tiny_and_ragged_shapes_leave_every_band_intact(zkb):
    """The shapes most likely to step outside a buffer - single elements, odd lengths, lengths one past a power of two,
    ragged matrices - through every prover, commitment method and the opening, all allocated under the guard."""
    from tests import test_gpu_fr as F, test_gpu_g1 as G, test_gpu_large as L, test_gpu_sumcheck as S
    z = zkb
    z.call("zkb_guard_enable", ctypes.c_int(1))
    try:
        if not SESSION_WIDE:
            _report(z, 1)
        dev = Dev(z)
        for n in (2, 3, 7, 100, 5000):
            S.test_zkip(dev, n)
        for shape in ((1, 1, 8), (1, 8, 1), (3, 5, 7), (16, 33, 20)):
            S.test_zkfc_prove(dev, *shape)
        for shape in ((3, 5), (8, 1), (1, 16), (5, 64)):
            S.test_zkip_stacked(dev, *shape)
        for case in ((8, 8, -4), (16, 4, 0), (1024, 16, -8), (4, 1, 3)):
            S.test_tlookup_prove(dev, *case)
        for case in ((1, 8), (2, 2), (3, 1024), (6, 32)):
            S.test_multi_hadamard(dev, *case)
        for n in (1, 3, 5, 1000, 4097):
            S.test_legacy_sumchecks(dev, n)
        for case in ((1, 1, 8), (3, 17, 14), (4, 40, 31), (33, 8, 13)):
            G.test_commit_int(dev, *case)
        for case in ((300, 9), (4097, 13)):
            L.test_me_open_against_cpp_oracle(dev, *case)
        for case in ((1, 8, 5), (3, 5, 4), (2, 3, 300), (1, 37, 64)):
            F.test_partial_me(dev, *case)
        for case in ((1, 1), (5, 7), (33, 100)):
            F.test_mle_eval_2d(dev, *case)
        F.test_pad_transpose_matmul_bias_gather(dev)
        for n in (1, 7, 2049):
            F.test_inv_shifted(dev, n)
        F.test_rescale(dev)
        del dev
        blocks, damaged, first, side = _report(z, 0)
        assert blocks > 200, "the guard saw too few blocks: is it on?"
        assert damaged == 0, f"a kernel wrote outside a block of {first} bytes ({'before' if side == 0 else 'after'} it)"
    finally:
        if not SESSION_WIDE:
            z.call("zkb_guard_enable", ctypes.c_int(0))
