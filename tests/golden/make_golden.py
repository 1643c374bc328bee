"""Generates tests/golden/ref_golden.json from the reference's own CUDA build.

Needs a GPU and oracle/_ref/ref_harness (built by `make -C oracle ref` where the
reference sources are present; device-LTO like the reference's own Makefile):

    python tests/golden/make_golden.py --out tests/golden/ref_golden.json

Every case writes its seeded inputs to raw .bin files, runs one harness command
(which calls the reference's public classes) and records inputs and outputs as
hex strings.  tests/test_oracle_golden.py replays the cases through the oracle.

With --api-check it also runs oracle/_ref/api_check_ref (oracle/api_check.cu built
against the reference, `make -C oracle ref-api`) and writes the lines it prints for
each case to tests/golden/api_check_<case>.txt (tests/test_gpu_api_check.py).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import random
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import pyref as R  # noqa: E402

EDGE = [0, 1, 2, R.R_MOD - 1, R.R_MOD - 2, (R.R_MOD + 1) // 2, (1 << 32) - 1, 1 << 32, (1 << 64) - 1, 1 << 64, R.FR_RADIX]


def hx(v: int) -> str:
    return "%x" % v


class Ctx:
    def __init__(self, harness: str, tmp: Path):
        self.harness, self.tmp, self.n = harness, tmp, 0

    def fr_file(self, vals) -> str:
        if len(vals) == 0:
            return "-"
        self.n += 1
        p = self.tmp / f"t{self.n}.bin"
        R.fr_pack(vals).tofile(p)
        return str(p)

    def int_file(self, ints) -> str:
        self.n += 1
        p = self.tmp / f"t{self.n}.bin"
        np.array(ints, dtype=np.int32).tofile(p)
        return str(p)

    def g1_file(self, pts) -> str:
        self.n += 1
        p = self.tmp / f"t{self.n}.bin"
        R.g1_pack(pts).tofile(p)
        return str(p)

    def out_file(self) -> str:
        self.n += 1
        return str(self.tmp / f"o{self.n}.bin")

    def run(self, *args) -> dict:
        res = subprocess.run([self.harness, *[str(a) for a in args]], capture_output=True, text=True, timeout=600)
        if res.returncode not in (0, 1):
            raise RuntimeError(f"harness {args[0]} failed rc={res.returncode}: {res.stderr[-500:]}")
        out = {}
        for line in res.stdout.splitlines():
            toks = line.replace("(", " ").replace(")", " ").replace(",", " ").split()
            if not toks:
                continue
            key, vals = toks[0], toks[1:]
            if key == "exception":
                out["exception"] = " ".join(vals)
            elif all(t.startswith("0x") for t in vals):
                out[key] = [t[2:].lstrip("0") or "0" for t in vals]
            else:
                out[key] = vals        # reference progress text or plain numbers
        return out


def seeded_gens(n, seed):
    rng = random.Random(seed)
    out = []
    for _ in range(n):
        a = R.g1_affine(R.g1_mul(R.G1_GEN, rng.randrange(1, R.R_MOD)))
        out.append((a[0], a[1], 1))
    return out


def build(ctx: Ctx) -> list:
    cases = []
    rng = random.Random(20240601)
    rf = lambda n: [rng.randrange(R.R_MOD) for _ in range(n)]
    rs = lambda n, bits=16: [R.int_to_fr(rng.randrange(-(1 << bits), 1 << bits)) for _ in range(n)]

    def add(kind, inputs, out):
        cases.append({"kind": kind, "in": inputs, "out": out})

    a, b = EDGE + rf(13), list(reversed(EDGE)) + rf(13)
    b[0] = rng.randrange(1, R.R_MOD)
    add("frops", {"a": [hx(v) for v in a], "b": [hx(v) for v in b]}, ctx.run("frops", ctx.fr_file(a), ctx.fr_file(b)))

    ints = [0, 1, -1, 2**31 - 1, -2**31, 65536, -65536, 12345, -999, 7]
    o_int, o_long = ctx.out_file(), ctx.out_file()
    out = ctx.run("ints", ctx.int_file(ints), o_int, o_long)
    out["save_int"] = np.fromfile(o_int, dtype=np.int32).tolist()
    out["save_long"] = np.fromfile(o_long, dtype=np.int64).tolist()
    add("ints", {"ints": ints}, out)

    for n in (1, 2, 5, 8, 13):
        t, u = rf(n), rf(R.ceil_log2(n))
        add("me", {"t": [hx(v) for v in t], "u": [hx(v) for v in u]}, ctx.run("me", ctx.fr_file(t), ctx.fr_file(u)))
    for other, cur, window in ((3, 5, 4), (1, 8, 1), (4, 7, 1), (2, 3, 5)):
        t, u = rf(other * cur * window), rf(R.ceil_log2(cur))
        add("partial_me", {"t": [hx(v) for v in t], "u": [hx(v) for v in u], "cur": cur, "window": window},
            ctx.run("partial_me", ctx.fr_file(t), ctx.fr_file(u), cur, window))
    for n, k, window in ((60, 3, 8), (64, 2, 8), (61, 2, 8), (16, 4, 1)):
        t, u = rf(n), rf(k)
        add("partial_me_window", {"t": [hx(v) for v in t], "u": [hx(v) for v in u], "window": window},
            ctx.run("partial_me_window", ctx.fr_file(t), ctx.fr_file(u), window))
    for d0, d1 in ((5, 7), (4, 8), (1, 6)):
        t, u0, u1 = rf(d0 * d1), rf(R.ceil_log2(d0)), rf(R.ceil_log2(d1))
        add("multi_dim_me", {"t": [hx(v) for v in t], "u0": [hx(v) for v in u0], "u1": [hx(v) for v in u1], "d0": d0, "d1": d1},
            ctx.run("multi_dim_me", ctx.fr_file(t), ctx.fr_file(u0), ctx.fr_file(u1), d0, d1))
    t = rf(35)
    add("layout", {"t": [hx(v) for v in t], "d0": 5, "d1": 7}, ctx.run("layout", ctx.fr_file(t), 5, 7))
    x, y = rf(15), rs(35)
    add("matmul", {"x": [hx(v) for v in x], "y": [hx(v) for v in y], "M": 3, "N": 5, "P": 7},
        ctx.run("matmul", ctx.fr_file(x), ctx.fr_file(y), 3, 5, 7))

    for n in (8, 13, 100):
        a, b, u = rf(n), rf(n), rf(R.ceil_log2(n))
        claim = sum(p * q for p, q in zip(a, b)) % R.R_MOD
        add("zkip", {"claim": hx(claim), "a": [hx(v) for v in a], "b": [hx(v) for v in b], "u": [hx(v) for v in u]},
            ctx.run("zkip", ctx.fr_file([claim]), ctx.fr_file(a), ctx.fr_file(b), ctx.fr_file(u)))
    for B, I, O in ((3, 5, 7), (4, 8, 8), (1, 1, 8), (2, 16, 1)):
        X, W = rs(B * I), rs(I * O)
        Y = R.matmul(X, W, B, I, O)
        ub, ui, uo = rf(R.ceil_log2(B)), rf(R.ceil_log2(I)), rf(R.ceil_log2(O))
        add("zkfc", {"X": [hx(v) for v in X], "W": [hx(v) for v in W], "B": B, "I": I, "O": O,
                     "ub": [hx(v) for v in ub], "ui": [hx(v) for v in ui], "uo": [hx(v) for v in uo]},
            ctx.run("zkfc", ctx.fr_file(X), ctx.fr_file(W), ctx.fr_file(Y), B, I, O, ctx.fr_file(ub), ctx.fr_file(ui), ctx.fr_file(uo)))

    for D, low, length in ((64, -4, 8), (16, 0, 16), (32, -3, 6), (8, 5, 1)):
        S = [rng.randrange(low, low + length) for _ in range(D)]
        k = R.ceil_log2(D)
        alpha, beta, u, v = rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rf(k), rf(k)
        add("tlookup", {"S": S, "low": low, "len": length, "alpha": hx(alpha), "beta": hx(beta),
                        "u": [hx(x) for x in u], "v": [hx(x) for x in v]},
            ctx.run("tlookup", ctx.int_file(S), low, length, ctx.fr_file([alpha]), ctx.fr_file([beta]), ctx.fr_file(u), ctx.fr_file(v)))
    for D, low, length in ((12, 0, 8), (16, -2, 5)):
        S = [rng.randrange(low, low + length) for _ in range(D)]
        mapped = rf(length)
        k = R.ceil_log2(D)
        r_, alpha, beta, u, v = rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rf(k), rf(k)
        add("mapping", {"S": S, "low": low, "len": length, "mapped": [hx(x) for x in mapped], "r": hx(r_), "alpha": hx(alpha),
                        "beta": hx(beta), "u": [hx(x) for x in u], "v": [hx(x) for x in v]},
            ctx.run("mapping", ctx.int_file(S), low, length, ctx.fr_file(mapped), ctx.fr_file([r_]), ctx.fr_file([alpha]),
                    ctx.fr_file([beta]), ctx.fr_file(u), ctx.fr_file(v)))
    for K, N in ((2, 16), (3, 8), (1, 4)):
        Xs = [rf(N) for _ in range(K)]
        k = R.ceil_log2(N)
        u, v = rf(k), rf(k)
        prod = [1] * N
        for X in Xs:
            prod = [p * q % R.R_MOD for p, q in zip(prod, X)]
        claim = R.mle_eval(prod, u)
        add("hadamard", {"claim": hx(claim), "Xs": [[hx(x) for x in X] for X in Xs], "u": [hx(x) for x in u], "v": [hx(x) for x in v]},
            ctx.run("hadamard", ctx.fr_file([claim]), ctx.fr_file(u), ctx.fr_file(v), *[ctx.fr_file(X) for X in Xs]))
    for n in (8, 13, 2):
        a, b = rf(n), rf(n)
        k = R.ceil_log2(n)
        u, v = rf(k), rf(k)
        add("legacy", {"a": [hx(x) for x in a], "b": [hx(x) for x in b], "u": [hx(x) for x in u], "v": [hx(x) for x in v]},
            ctx.run("legacy", ctx.fr_file(a), ctx.fr_file(b), ctx.fr_file(u), ctx.fr_file(v)))
    vals = [0, 1, -1, 32767, 32768, 32769, -32767, -32768, -32769, 65536, -65536, 98304, 2**40 + 12345, -(2**40) - 77]
    vals += [rng.randrange(-2**45, 2**45) for _ in range(20)]
    for sf in (1 << 16, 1 << 20):
        add("rescale", {"x": vals, "sf": sf}, ctx.run("rescale", ctx.fr_file([R.int_to_fr(v) for v in vals]), sf))

    # softmax with the driver's parameters (self-attn.cu:87): sf = 2^32
    m, n, d = 4, 8, 16
    nrng = np.random.Generator(np.random.PCG64(77))
    X = np.rint(nrng.standard_normal(m * n) * (2.0 ** 32) * math.sqrt(d) * 1.5).astype(np.int64).tolist()
    k = R.ceil_log2(m * n)
    u, v = rf(k), rf(k)
    r_, alpha, beta = rng.randrange(R.R_MOD), rng.randrange(R.R_MOD), rng.randrange(R.R_MOD)
    add("softmax", {"X": X, "m": m, "n": n, "d": d, "u": [hx(x) for x in u], "v": [hx(x) for x in v], "r": hx(r_),
                    "alpha": hx(alpha), "beta": hx(beta)},
        ctx.run("softmax", ctx.fr_file([R.int_to_fr(x) for x in X]), m, n, d, ctx.fr_file(u), ctx.fr_file(v), ctx.fr_file([r_]),
                ctx.fr_file([alpha]), ctx.fr_file([beta])))

    gens = seeded_gens(8, 4242)
    sc = [0, 1, R.R_MOD - 1, 5] + rf(4)
    u = rf(3)
    add("g1ops", {"seed": 4242, "n": 8, "scalars": [hx(x) for x in sc], "u": [hx(x) for x in u]},
        ctx.run("g1ops", ctx.g1_file(gens), ctx.fr_file(sc), ctx.fr_file(u)))
    ints = [rng.randrange(-8000, 8000) for _ in range(16)]
    ints[0], ints[1] = 0, -8127
    full = rf(8)
    u = rf(4)
    add("commit", {"seed": 4242, "n": 8, "ints": ints, "full": [hx(x) for x in full], "u": [hx(x) for x in u]},
        ctx.run("commit", ctx.g1_file(gens), ctx.int_file(ints), ctx.fr_file(full), ctx.fr_file(u)))
    big = [2**31 - 1, -2**31, 2**20 + 3, -77, 0, 1, -1, 123456789]
    add("commit", {"seed": 4242, "n": 8, "ints": big, "full": [hx(x) for x in full], "u": [hx(x) for x in u[:3]]},
        ctx.run("commit", ctx.g1_file(gens), ctx.int_file(big), ctx.fr_file(full), ctx.fr_file(u[:3])))
    return cases


def fr_digest(hex_vals) -> str:
    """SHA-256 of the values' canonical 32-byte little-endian encodings, concatenated"""
    return hashlib.sha256(b"".join(int(h, 16).to_bytes(32, "little") for h in hex_vals)).hexdigest()


def softmax_large_inputs(m: int, n: int, d: int) -> np.ndarray:
    nrng = np.random.Generator(np.random.PCG64(78))
    return np.rint(nrng.standard_normal(m * n) * (2.0 ** 32) * math.sqrt(d) * 1.5).astype(np.int64)


def fullsize(ctx: Ctx) -> dict:
    """Cases at the layer's own sizes, recorded as digests: the softmax row shift over 2048 columns with d = 4096
    (zksoftmax.cu:20-32: a 2048-term left-to-right double-precision sum per row), its digits and table outputs."""
    m, n, d = 16, 2048, 4096
    X = softmax_large_inputs(m, n, d)
    out = ctx.run("softmax", ctx.fr_file([R.int_to_fr(int(x)) for x in X]), m, n, d)
    rec = {"m": m, "n": n, "d": d, "inputs": "tests/golden/make_golden.py: softmax_large_inputs (PCG64 seed 78)", "shift": out["shift"]}
    for key in ("y", "xseg0", "xseg1", "xseg2", "yseg0", "yseg1"):
        rec[key + "_sha256"] = fr_digest(out[key])
    return {"softmax_16x2048_d4096": rec}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--harness", default=str(ROOT / "oracle" / "_ref" / "ref_harness"))
    ap.add_argument("--out", default=str(ROOT / "tests" / "golden" / "ref_golden.json"))
    ap.add_argument("--api-check", action="store_true", help="also record the output of oracle/_ref/api_check_ref")
    ap.add_argument("--fullsize", action="store_true", help="only add the full-size digests to tests/golden/ref_fullsize.json")
    args = ap.parse_args()
    if args.fullsize:
        path = ROOT / "tests" / "golden" / "ref_fullsize.json"
        gold = json.loads(path.read_text())
        with tempfile.TemporaryDirectory() as tmp:
            gold.update(fullsize(Ctx(args.harness, Path(tmp))))
        path.write_text(json.dumps(gold, indent=1) + "\n")
        print(f"updated {path}")
        return
    if args.api_check:
        exe = ROOT / "oracle" / "_ref" / "api_check_ref"
        for case in ("fcstacked", "attn", "attnstacked", "relu", "misc"):
            res = subprocess.run([str(exe), case], capture_output=True, text=True, check=True)
            keep = [ln for ln in res.stdout.splitlines() if ln.split(" ")[0].startswith(("poly", "final", "out", "ok"))]
            # a long line (a whole tensor) is kept as its key and the SHA-256 of its text
            keep = [ln if len(ln) <= 4096 else ln.split(" ")[0] + " sha256:" + hashlib.sha256(ln.encode()).hexdigest() for ln in keep]
            (ROOT / "tests" / "golden" / f"api_check_{case}.txt").write_text("\n".join(keep) + "\n")
            print(f"wrote {len(keep)} lines for {case}")
    with tempfile.TemporaryDirectory() as tmp:
        cases = build(Ctx(args.harness, Path(tmp)))
    Path(args.out).parent.mkdir(parents=True, exist_ok=True)
    with open(args.out, "w") as f:
        json.dump({"source": "reference CUDA build (oracle/ref_harness.cu linked against the reference objects, -arch=sm_100 -dc -dlto), run on a B200", "cases": cases}, f, separators=(",", ":"))
    print(f"wrote {len(cases)} cases to {args.out}")


if __name__ == "__main__":
    main()
