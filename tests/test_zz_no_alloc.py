"""GPU: the allocation-free entry point zkb_fr_mle_eval_noalloc.

Some callers of this library cannot allocate device memory: a process that handed
the whole GPU to its own memory manager when it started, or a latency-critical loop
that must not touch the allocator.  For them the multilinear evaluation exists in a
form whose working memory is a fixed array inside the library.  This file checks,
through the C ABI, that it returns exactly what zkb_fr_mle_eval returns - on two
calls in a row, because the calls share that array and the second one sees what the
first left behind - and that sizes beyond the documented limit are refused.  The
file name sorts last so that a run stopping at the first failure has already run
every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rand_fr(rng, k):
    r_top = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001 >> 224
    v = rng.integers(0, 1 << 32, size=(max(k, 1), 8), dtype=np.uint64).astype(np.uint32)
    v[:, 7] %= np.uint32(r_top)
    return v


def _both(zkb, a, u, k):
    z = zkb
    d_a = z.DeviceBuffer.from_host(a)
    ref, got = np.zeros((1, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_fr_mle_eval", z._p(d_a), z.sz(a.shape[0]), z._p(u), z.u32(k), z._p(ref), z._p(0))
    z.call("zkb_fr_mle_eval_noalloc", z._p(d_a), z.sz(a.shape[0]), z._p(u), z.u32(k), z._p(got), z._p(0))
    return ref, got


def test_two_calls_in_a_row_match_the_allocating_entry_point(zkb):
    rng = np.random.Generator(np.random.PCG64(2024))
    # first call: two-level tables (k > 12) and a ragged size; second call: a smaller
    # problem that reuses the same array with the first call's contents still in it
    for n, k in ((300001, 19), (1000, 10), (1 << 16, 16), (1, 0)):
        a, u = _rand_fr(rng, n)[:n], _rand_fr(rng, k)
        ref, got = _both(zkb, a, u, k)
        assert np.array_equal(ref, got), (n, k)
        assert ref.any()


def test_the_largest_sizes_fill_the_fixed_array_exactly(zkb):
    """k = 24 uses all 4096 entries of the high table: one element more than half the limit (ragged), then the limit itself"""
    z = zkb
    rng = np.random.Generator(np.random.PCG64(24))
    u = _rand_fr(rng, 24)
    # small signed values as field elements: cheap to make on the host at this size
    vals = rng.integers(-(1 << 30), 1 << 30, size=1 << 24, dtype=np.int64)
    d_int = z.DeviceBuffer.from_host(vals)
    d_a = z.DeviceBuffer(32 << 24)
    z.call("zkb_fr_from_i64", z._p(d_int), z._p(d_a), z.sz(1 << 24), z._p(0))
    for n in ((1 << 23) + 1, 1 << 24):
        ref, got = np.zeros((1, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
        z.call("zkb_fr_mle_eval", z._p(d_a), z.sz(n), z._p(u), z.u32(24), z._p(ref), z._p(0))
        z.call("zkb_fr_mle_eval_noalloc", z._p(d_a), z.sz(n), z._p(u), z.u32(24), z._p(got), z._p(0))
        assert np.array_equal(ref, got) and ref.any(), n


def test_sizes_beyond_the_limit_are_refused(zkb):
    z = zkb
    rng = np.random.Generator(np.random.PCG64(1))
    a, u = _rand_fr(rng, 16), _rand_fr(rng, 25)
    out = np.zeros((1, 8), dtype=np.uint32)
    with pytest.raises(z.ZkbError) as e:
        z.call("zkb_fr_mle_eval_noalloc", z._p(z.DeviceBuffer.from_host(a)), z.sz((1 << 24) + 1), z._p(u), z.u32(25), z._p(out), z._p(0))
    assert e.value.code == z.ERR_LIMIT and "2^24" in e.value.msg
    with pytest.raises(z.ZkbError) as e:
        z.call("zkb_fr_mle_eval_noalloc", z._p(z.DeviceBuffer.from_host(a)), z.sz(16), z._p(u), z.u32(3), z._p(out), z._p(0))
    assert e.value.code == z.ERR_DIM
