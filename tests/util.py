"""Helpers shared by the GPU parity tests: seeded inputs and C-ABI call wrappers."""
import ctypes
import random

import numpy as np

from oracle import pyref as R


def rand_fr(rng: random.Random, n: int) -> list:
    return [rng.randrange(R.R_MOD) for _ in range(n)]


def rand_small_fr(rng: random.Random, n: int, bits: int = 16) -> list:
    return [R.int_to_fr(rng.randrange(-(1 << bits), 1 << bits)) for _ in range(n)]


EDGE_FR = [0, 1, 2, R.R_MOD - 1, R.R_MOD - 2, (R.R_MOD + 1) // 2, (1 << 255) % R.R_MOD, (1 << 32) - 1, 1 << 32,
           (1 << 64) - 1, 1 << 64, R.FR_RADIX, R.R_MOD - R.FR_RADIX]


class Dev:
    """Thin convenience layer over the ctypes binding for tests."""

    def __init__(self, zkb):
        self.z = zkb

    def fr(self, vals):
        return self.z.fr_buffer(R.fr_pack(vals))

    def fr_out(self, n):
        return self.z.DeviceBuffer(32 * max(n, 1))

    def read_fr(self, buf, n):
        return R.fr_unpack(buf.to_host(np.uint32, (n, 8)))

    def hfr(self, vals):
        return self.z.fr_host(R.fr_pack(vals))

    def g1(self, pts):
        return self.z.DeviceBuffer.from_host(R.g1_pack(pts))

    def read_g1(self, buf, n):
        return R.g1_unpack(buf.to_host(np.uint32, (n, 36)))

    def call(self, name, *args):
        return self.z.call(name, *args)


def affine_eq(p, q) -> bool:
    return R.g1_affine(p) == R.g1_affine(q)


def seeded_generators(n: int, seed: int) -> list:
    """n G1 points k_i * G with seeded k_i (Jacobian with Z = 1 after normalising)"""
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        a = R.g1_affine(R.g1_mul(R.G1_GEN, rng.randrange(1, R.R_MOD)))
        out.append((a[0], a[1], 1))
    return out
