"""Big-integer restatement of the reference prover path (TEST INFRASTRUCTURE ONLY).

This module is the checker that tests/, __graft_entry__.smoke() and bench.py's
baseline legs compare the CUDA library against.  Nothing in the product path may
import it.  Every function states which reference file:line it restates.  Field
elements are plain Python ints in [0, r); G1 points are (X, Y, Z) Jacobian triples
of plain ints (NOT Montgomery form) with Z == 0 meaning the identity.

Parity status: pinned.  tests/golden/ref_*.json hold outputs of the reference's
own CUDA build (oracle/ref_harness.cu linked against the reference's objects) on
seeded inputs; tests/test_oracle_golden.py checks this module against them.
"""
from __future__ import annotations

import numpy as np

# --- BLS12-381 parameters (bls12-381.cu:3-11, bls12-381.cuh:119,224) -----------------
R_MOD = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001   # Fr
Q_MOD = 0x1A0111EA397FE69A4B1BA7B6434BACD764774B84F38512BF6730D2A0F6B0F6241EABFFFEB153FFFFB9FEFFFFFFFFAAAB  # Fq
FR_RADIX = (1 << 256) % R_MOD       # Montgomery R for Fr
FQ_RADIX = (1 << 384) % Q_MOD       # Montgomery R for Fq
FR_RADIX_INV = pow(FR_RADIX, -1, R_MOD)
FQ_RADIX_INV = pow(FQ_RADIX, -1, Q_MOD)
G1_X = 0x17F1D3A73197D7942695638C4FA9AC0FC3688C4F9774B905A14E3A3F171BAC586C55E83FF97A1AEFFB3AF00ADB22C6BB
G1_Y = 0x08B3F481E3AAA0F1A09E30ED741D8AE4FCF5E095D5D00AF600DB18CB2C04B3EDD03CC744A2888AE40CAA232946C5E7E1
TWO_INV = (R_MOD + 1) // 2          # tlookup.cu:180


def ceil_log2(n: int) -> int:
    """fr-tensor.cu:26-43"""
    if n == 0:
        return 0
    return (n - 1).bit_length()


# --- limb packing ------------------------------------------------------------------
def int_to_limbs(x: int, n: int) -> np.ndarray:
    return np.array([(x >> (32 * i)) & 0xFFFFFFFF for i in range(n)], dtype=np.uint32)


def limbs_to_int(a) -> int:
    out = 0
    for i, w in enumerate(np.asarray(a, dtype=np.uint32).tolist()):
        out |= int(w) << (32 * i)
    return out


def fr_pack(vals) -> np.ndarray:
    """list of ints -> (len, 8) uint32, the FrTensor memory layout (bls12-381.cuh:116-120)"""
    vals = list(vals)
    buf = bytearray(32 * len(vals))
    for i, v in enumerate(vals):
        buf[32 * i:32 * i + 32] = int(v % R_MOD).to_bytes(32, "little")
    return np.frombuffer(bytes(buf), dtype=np.uint32).reshape(len(vals), 8).copy()


def fr_unpack(arr) -> list:
    b = np.ascontiguousarray(arr, dtype=np.uint32).tobytes()
    return [int.from_bytes(b[i:i + 32], "little") for i in range(0, len(b), 32)]


def fq_pack_mont(vals) -> np.ndarray:
    """ints (standard) -> (len, 12) uint32 in Montgomery form, the G1 tensor coordinate layout"""
    vals = list(vals)
    buf = bytearray(48 * len(vals))
    for i, v in enumerate(vals):
        buf[48 * i:48 * i + 48] = int(v * FQ_RADIX % Q_MOD).to_bytes(48, "little")
    return np.frombuffer(bytes(buf), dtype=np.uint32).reshape(len(vals), 12).copy()


def g1_pack(points) -> np.ndarray:
    """list of Jacobian (X,Y,Z) int triples -> (len, 36) uint32 Montgomery-form G1Jacobian_t array"""
    flat = []
    for (x, y, z) in points:
        flat += [x, y, z]
    return fq_pack_mont(flat).reshape(len(points), 36)


def g1_unpack(arr) -> list:
    b = np.ascontiguousarray(arr, dtype=np.uint32).tobytes()
    vals = [int.from_bytes(b[i:i + 48], "little") * FQ_RADIX_INV % Q_MOD for i in range(0, len(b), 48)]
    return [(vals[i], vals[i + 1], vals[i + 2]) for i in range(0, len(vals), 3)]


# --- fixed-point <-> Fr (fr-tensor.cu:686-711, 924-945) -----------------------------
def int_to_fr(v: int) -> int:
    return v % R_MOD


def fr_to_long(a: int) -> int:
    """scalar_to_long: small non-negative stays, otherwise -(r - a); >64-bit magnitudes give 0"""
    if a < (1 << 63):
        return a
    n = (R_MOD - a) % R_MOD
    mag = n if n < (1 << 64) else 0
    v = (-mag) & 0xFFFFFFFFFFFFFFFF           # -static_cast<long>(mag) wraps like a C long
    return v - (1 << 64) if v >> 63 else v


def fr_to_int(a: int) -> int:
    """scalar_to_int (fr-tensor.cu:930-934); result wraps like a C int"""
    if a < (1 << 31):
        return a
    n = (R_MOD - a) % R_MOD
    mag = n if n < (1 << 32) else 0
    v = (-mag) & 0xFFFFFFFF
    return v - (1 << 32) if v >> 31 else v


# --- MLE folds (LSB first) -----------------------------------------------------------
def me_step(t: list, x: int) -> list:
    """Fr_me_step, fr-tensor.cu:588-600: adjacent pairs, odd tail folds against zero"""
    out = []
    for i in range((len(t) + 1) // 2):
        a0 = t[2 * i]
        a1 = t[2 * i + 1] if 2 * i + 1 < len(t) else 0
        out.append((a0 + x * (a1 - a0)) % R_MOD)
    return out


def mle_eval(t: list, u: list) -> int:
    """FrTensor::operator()(u) / Fr_me, fr-tensor.cu:437-442,602-609"""
    t = list(t)
    if not (len(t) > ((1 << len(u)) // 2) and len(t) <= (1 << len(u))):
        raise RuntimeError("Incompatible dimensions")
    for x in u:
        t = me_step(t, x)
    return t[0]


def partial_me(t: list, u: list, cur_dim: int, window: int) -> list:
    """FrTensor::partial_me(u, cur_dim, window_size), fr-tensor.cu:518-560.

    The tensor is viewed as [other, cur_dim, window]; the cur_dim axis is folded
    LSB-first with u, a missing odd partner counting as zero."""
    if cur_dim <= ((1 << len(u)) >> 1):
        raise RuntimeError("cur_dim <= ((1<<u.size()) >> 1)")
    if cur_dim > (1 << len(u)):
        raise RuntimeError("cur_dim > (1<<u.size())")
    t = list(t)
    for x in u:
        if len(t) % (cur_dim * window) != 0:
            raise RuntimeError("t.size % (cur_dim * window_size) != 0")
        other = len(t) // (cur_dim * window)
        out_dim = (cur_dim + 1) // 2
        out = [0] * (other * out_dim * window)
        for o in range(other):
            for j in range(out_dim):
                for w in range(window):
                    a0 = t[o * cur_dim * window + (2 * j) * window + w]
                    a1 = t[o * cur_dim * window + (2 * j + 1) * window + w] if 2 * j + 1 < cur_dim else 0
                    out[(o * out_dim + j) * window + w] = (a0 + x * (a1 - a0)) % R_MOD
        t, cur_dim = out, out_dim
    return t


def multi_dim_me(t: list, us: list, shape: list) -> int:
    """FrTensor::multi_dim_me, fr-tensor.cu:643-652: fold the last axis first"""
    if len(us) != len(shape):
        raise RuntimeError("Incompatible dimensions")
    if len(shape) == 0:
        return t[0]
    if len(shape) == 1:
        return mle_eval(t, us[0])
    t2 = partial_me(t, us[-1], shape[-1], 1)
    return multi_dim_me(t2, us[:-1], shape[:-1])


def pad(t: list, shape: list, pad_val: int = 0) -> list:
    """FrTensor::pad, fr-tensor.cu:809-828: every axis (last first) grows to a power of two"""
    total = 1
    for s in shape:
        total *= s
    if total != len(t):
        raise RuntimeError("pad: cum_shape != size")
    last = shape[-1]
    last_p = 1 << ceil_log2(last)
    rows = total // last
    out = []
    for r in range(rows):
        out += t[r * last:(r + 1) * last] + [pad_val] * (last_p - last)
    if len(shape) == 1:
        return out
    new_shape = list(shape[:-1])
    new_shape[-1] *= last_p
    return pad(out, new_shape, pad_val)


def matmul(x: list, y: list, M: int, N: int, P: int) -> list:
    """FrTensor::matmul, fr-tensor.cu:831-881 (plain modular matrix product)"""
    out = [0] * (M * P)
    for i in range(M):
        for k in range(P):
            s = 0
            for j in range(N):
                s += x[i * N + j] * y[j * P + k]
            out[i * P + k] = s % R_MOD
    return out


# --- polynomials (polynomial.cu:296-360): coefficient lists, low degree first ---------
def poly_eval(c: list, x: int) -> int:
    acc, pw = 0, 1
    for ci in c:
        acc = (acc + ci * pw) % R_MOD
        pw = pw * x % R_MOD
    return acc


def poly_mul(a: list, b: list) -> list:
    out = [0] * (len(a) + len(b) - 1)
    for i, ai in enumerate(a):
        for j, bj in enumerate(b):
            out[i + j] = (out[i + j] + ai * bj) % R_MOD
    return out


def poly_add(a: list, b: list) -> list:
    n = max(len(a), len(b))
    return [((a[i] if i < len(a) else 0) + (b[i] if i < len(b) else 0)) % R_MOD for i in range(n)]


def poly_sub(a: list, b: list) -> list:
    """polySubKernel, polynomial.cu:208-219.  Where only b has a coefficient the
    reference copies it WITHOUT negating; kept as is."""
    n = max(len(a), len(b))
    out = []
    for i in range(n):
        if i < len(a):
            out.append((a[i] - (b[i] if i < len(b) else 0)) % R_MOD)
        else:
            out.append(b[i] % R_MOD)
    return out


def eq_poly(u: int) -> list:
    """Polynomial::eq(u) = (1-u) + (2u-1) t, polynomial.cu:342-353"""
    return [(1 - u) % R_MOD, (2 * u - 1) % R_MOD]


def eq_eval(u: int, v: int) -> int:
    """Polynomial::eq(u, v) = 2uv - u - v + 1, polynomial.cu:355-373"""
    return (2 * u * v - u - v + 1) % R_MOD


def zkip_stacked(claim: int, A: list, B: list, uN: list, uD: list, vN: list, N: int, D: int, proof: list) -> int:
    """zkip_stacked, zkfc.cu:187-228: A and B are [N, D]; one round per variable of the stack (paired with uN[-1], folded
    with vN[-1], coefficient tensors folded over the lower half of the stack with eq(uN[:-1]) and summed), then zkip over D."""
    A, B, uN, vN = list(A), list(B), list(uN), list(vN)
    while uN:
        if len(A) != N * D:
            raise RuntimeError("a.size != N * D")
        if len(B) != N * D:
            raise RuntimeError("b.size != N * D")
        n_out = (1 << ceil_log2(N)) >> 1
        size_out = n_out * D
        out = [[], [], []]
        nA, nB = [], []
        v = vN[-1]
        for g in range(size_out):
            a0, b0 = A[g], B[g]
            a1 = ((A[g + size_out] if g + size_out < N * D else 0) - a0) % R_MOD
            b1 = ((B[g + size_out] if g + size_out < N * D else 0) - b0) % R_MOD
            out[0].append(a0 * b0 % R_MOD)
            out[1].append((a0 * b1 + a1 * b0) % R_MOD)
            out[2].append(a1 * b1 % R_MOD)
            nA.append((a0 + v * a1) % R_MOD)
            nB.append((b0 + v * b1) % R_MOD)
        u_ = uN[:-1]
        p = [sum(partial_me(o, u_, n_out, D)) % R_MOD if u_ else sum(o) % R_MOD for o in out]
        proof.append(p)
        u = uN[-1]
        q0 = (1 - u) * poly_eval(p, 0) % R_MOD          # q = eq(u) * p
        q1 = u * poly_eval(p, 1) % R_MOD
        if claim != (q0 + q1) % R_MOD:
            raise RuntimeError("claim != q(0) + q(1)")
        claim = poly_eval(p, v)
        A, B, uN, vN, N = nA, nB, uN[:-1], vN[:-1], n_out
    return zkip(claim, A, B, uD, proof)


# --- zkip / zkFC::prove (zkfc.cu:61-151) ----------------------------------------------
def zkip(claim: int, a: list, b: list, u: list, proof: list) -> int:
    """Inner-product sumcheck, MSB first, challenges consumed from the back.
    Appends one [c0,c1,c2] per round to proof.  zkfc.cu:94-151."""
    a, b, u = list(a), list(b), list(u)
    while u:
        if len(a) != len(b):
            raise RuntimeError("a.size != b.size")
        n_in = len(a)
        n_out = (1 << ceil_log2(n_in)) >> 1
        c0 = c1 = c2 = 0
        na, nb = [], []
        v = u[-1]
        for g in range(n_out):
            a0 = a[g] if g < n_in else 0
            b0 = b[g] if g < n_in else 0
            a1 = a[g + n_out] if g + n_out < n_in else 0
            b1 = b[g + n_out] if g + n_out < n_in else 0
            c0 += a0 * b0
            c1 += a0 * (b1 - b0) + b0 * (a1 - a0)
            c2 += (a1 - a0) * (b1 - b0)
            na.append((a0 + v * (a1 - a0)) % R_MOD)
            nb.append((b0 + v * (b1 - b0)) % R_MOD)
        p = [c0 % R_MOD, c1 % R_MOD, c2 % R_MOD]
        proof.append(p)
        if claim != (poly_eval(p, 0) + poly_eval(p, 1)) % R_MOD:
            raise RuntimeError("claim != p(0) + p(1)")
        claim = poly_eval(p, v)
        a, b, u = na, nb, u[:-1]
    return claim


def zkfc_prove(X: list, W: list, Y: list, B: int, I: int, O: int, u_batch, u_input, u_output) -> dict:
    """Body of zkFC::prove (zkfc.cu:61-87) with the three challenge vectors passed in."""
    claim = multi_dim_me(Y, [u_batch, u_output], [B, O])
    x_red = partial_me(X, u_batch, B, I)
    w_red = partial_me(W, u_output, O, 1)
    proof = []
    final_claim = zkip(claim, x_red, w_red, u_input, proof)
    claim_x = multi_dim_me(X, [u_batch, u_input], [B, I])
    claim_w = multi_dim_me(W, [u_input, u_output], [I, O])
    if claim_x * claim_w % R_MOD != final_claim:
        raise RuntimeError("Claim does not match")
    return dict(claim=claim, x_red=x_red, w_red=w_red, proof=proof, final_claim=final_claim,
                claim_x=claim_x, claim_w=claim_w)


# --- tLookup (tlookup.cu:10-370) ------------------------------------------------------
def fr_inv(a: int) -> int:
    """Fermat inverse; maps 0 to 0 (bls12-381.cu:597-609)"""
    return pow(a, R_MOD - 2, R_MOD)


def tlookup_prep(indices, table_size: int) -> list:
    """tLookup::prep, tlookup.cu:23-48: multiplicities"""
    m = [0] * table_size
    for i in indices:
        m[i] += 1
    return m


def range_table(low: int, length: int) -> list:
    """tLookupRange ctor, tlookup.cu:372-391: padded by repeating the last value"""
    size = 1 << ceil_log2(length)
    return [int_to_fr((i + low) if i < length else (length + low - 1)) for i in range(size)]


def range_indices(vals: list, low: int) -> list:
    """lookuprange_tensor_prep_kernel, tlookup.cu:414-421: low limb of (v - low)"""
    return [((v - low) % R_MOD) & 0xFFFFFFFF for v in vals]


def _phase1_poly(A, S, alpha, beta, C, u):
    """tLookup_phase1_step_poly, tlookup.cu:184-200"""
    half = len(A) >> 1
    t0, t1, t2, a0s, a1s = [], [], [], 0, 0
    for i in range(half):
        c00, c01 = A[i], (A[i + half] - A[i]) % R_MOD
        c10, c11 = (S[i] + beta) % R_MOD, (S[i + half] - S[i]) % R_MOD
        t0.append(alpha * c00 * c10 % R_MOD)
        t1.append(alpha * (c01 * c10 + c00 * c11) % R_MOD)
        t2.append(alpha * c01 * c11 % R_MOD)
        a0s += c00
        a1s += c01
    u_ = u[:-1]
    p0 = [mle_eval(t0, u_), mle_eval(t1, u_), mle_eval(t2, u_)]
    p1 = [a0s % R_MOD, a1s % R_MOD]
    p = poly_add(poly_add(poly_mul(p0, eq_poly(u[-1])), p1), [C * TWO_INV % R_MOD])
    return p


def _phase2_poly(A, S, Bv, T, m, alpha_, beta, inv_ratio, alpha_sq, u):
    """tLookup_phase2_step_poly, tlookup.cu:245-279"""
    half = len(m) >> 1
    u_ = u[:-1]

    def ev(X, Y, coef):
        t0, t1, t2 = [], [], []
        for i in range(half):
            c00, c01 = X[i], (X[i + half] - X[i]) % R_MOD
            c10, c11 = (Y[i] + beta) % R_MOD, (Y[i + half] - Y[i]) % R_MOD
            t0.append(coef * c00 * c10 % R_MOD)
            t1.append(coef * (c01 * c10 + c00 * c11) % R_MOD)
            t2.append(coef * c01 * c11 % R_MOD)
        return [mle_eval(t0, u_), mle_eval(t1, u_), mle_eval(t2, u_)]

    p0 = poly_add(ev(A, S, alpha_), ev(Bv, T, inv_ratio * alpha_sq % R_MOD))
    p1 = [sum(A[:half]) % R_MOD, (sum(A[half:2 * half]) - sum(A[:half])) % R_MOD]
    d0 = d1 = d2 = 0
    for i in range(half):
        m0, m1 = m[i], (m[i + half] - m[i]) % R_MOD
        b0, b1 = Bv[i], (Bv[i + half] - Bv[i]) % R_MOD
        d0 += m0 * b0
        d1 += m1 * b0 + m0 * b1
        d2 += m1 * b1
    p2 = [d0 % R_MOD, d1 % R_MOD, d2 % R_MOD]
    return poly_sub(poly_add(poly_mul(eq_poly(u[-1]), p0), p1), [c * inv_ratio % R_MOD for c in p2])


def _fold_msb(X, v):
    half = len(X) >> 1
    return [(X[i] + v * (X[i + half] - X[i])) % R_MOD for i in range(half)]


def tlookup_prove(S: list, table: list, m: list, alpha: int, beta: int, u: list, v: list,
                  polys: list | None = None) -> int:
    """tLookup::prove, tlookup.cu:324-370, with phases :281-320.  Appends every round
    polynomial (which the reference computes and drops) to `polys` when given."""
    D, N = len(S), len(m)
    if len(m) != len(table):
        raise RuntimeError("m.size != table.size")
    if D != 1 << ceil_log2(D) or N != 1 << ceil_log2(N) or D % N != 0:
        raise RuntimeError("D or N is not power of 2, or D is not divisible by N")
    A = [fr_inv((s + beta) % R_MOD) for s in S]
    Bv = [fr_inv((t + beta) % R_MOD) for t in table]
    if len(u) != ceil_log2(D):
        raise RuntimeError("u.size() != ceilLog2(D)")
    if len(v) != ceil_log2(D):
        raise RuntimeError("v.size() != ceilLog2(D)")
    k1 = ceil_log2(D // N)
    v1, v2 = list(v[:k1]), list(v[k1:])
    C = (alpha * alpha - sum(b * mm for b, mm in zip(Bv, m))) % R_MOD
    alpha_sq = alpha * alpha % R_MOD
    claim = (alpha + alpha_sq) % R_MOD
    inv_ratio = N * fr_inv(D) % R_MOD
    S, T, m, u = list(S), list(table), list(m), list(u)
    # phase 1
    while v1:
        p = _phase1_poly(A, S, alpha, beta, C, u)
        if polys is not None:
            polys.append(p)
        if claim != (poly_eval(p, 0) + poly_eval(p, 1)) % R_MOD:
            raise RuntimeError("tLookup_phase1: claim != p(0) + p(1)")
        vv = v1[-1]
        claim = poly_eval(p, vv)
        A, S = _fold_msb(A, vv), _fold_msb(S, vv)
        alpha = alpha * eq_eval(u[-1], vv) % R_MOD
        C = C * TWO_INV % R_MOD
        u, v1 = u[:-1], v1[:-1]
    # phase 2
    alpha_ = alpha
    while v2:
        p = _phase2_poly(A, S, Bv, T, m, alpha_, beta, inv_ratio, alpha_sq, u)
        if polys is not None:
            polys.append(p)
        if claim != (poly_eval(p, 0) + poly_eval(p, 1)) % R_MOD:
            raise RuntimeError("tLookup_phase2: claim != p(0) + p(1)")
        vv = v2[-1]
        claim = poly_eval(p, vv)
        A, S, Bv, T, m = (_fold_msb(X, vv) for X in (A, S, Bv, T, m))
        e = eq_eval(u[-1], vv)
        alpha_ = alpha_ * e % R_MOD
        alpha_sq = alpha_sq * e % R_MOD
        u, v2 = u[:-1], v2[:-1]
    return claim


def tlookup_mapping_prove(S_in, S_out, table, mapped, m, r, alpha, beta, u, v, polys=None) -> int:
    """tLookupRangeMapping::prove, tlookup.cu:494-551 (pads a non-power-of-two D first)"""
    D = len(S_in)
    m = list(m)
    if D != 1 << ceil_log2(D):
        S_in = pad(list(S_in), [D], table[0])
        S_out = pad(list(S_out), [D], mapped[0])
        m[0] = (m[0] + (1 << ceil_log2(D)) - D) % R_MOD
    S_com = [(a + b * r) % R_MOD for a, b in zip(S_in, S_out)]
    T_com = [(a + b * r) % R_MOD for a, b in zip(table, mapped)]
    return tlookup_prove(S_com, T_com, m, alpha, beta, u, v, polys)


# --- multi-Hadamard and the legacy sumchecks (proof.cu:12-241) -------------------------
def multi_hadamard_sumchecks(claim: int, Xs: list, u: list, v: list, proof: list) -> int:
    """proof.cu:190-241.  Pushes the degree-K polynomials (before the eq factor)."""
    Xs = [list(x) for x in Xs]
    u, v = list(u), list(v)
    while True:
        N = len(Xs[0])
        if N == 1:
            return claim
        if N & (N - 1):
            raise RuntimeError("N is not a power of 2")
        half = N >> 1
        out = None
        for X in Xs:
            if len(X) != N:
                raise RuntimeError("Xs[i] size is not N")
            x0 = X[:half]
            x1 = [(X[i + half] - X[i]) % R_MOD for i in range(half)]
            if out is None:
                out = [x0, x1]
            else:
                new = [[0] * half for _ in range(len(out) + 1)]
                for j, col in enumerate(out):
                    for i in range(half):
                        new[j][i] = (new[j][i] + col[i] * x0[i]) % R_MOD
                        new[j + 1][i] = (new[j + 1][i] + col[i] * x1[i]) % R_MOD
                out = new
        u_ = u[:-1]
        coefs = [mle_eval(col, u_) for col in out]
        proof.append(coefs)
        p = poly_mul(coefs, eq_poly(u[-1]))
        if claim != (poly_eval(p, 0) + poly_eval(p, 1)) % R_MOD:
            raise RuntimeError("multi_hadamard_sumchecks: claim != p(0) + p(1)")
        claim = poly_eval(coefs, v[-1])
        Xs = [_fold_msb(X, v[-1]) for X in Xs]
        u, v = u_, v[:-1]


def _legacy_ip_terms(a, b):
    """Fr_ip_sc_step, proof.cu:12-27.  The kernel multiplies standard-form values with
    the raw Montgomery product and never converts back, so every term carries a factor
    R^-1 (R = 2^256 mod r)."""
    out0, out1, out2 = [], [], []
    n = len(a)
    for g in range((n + 1) // 2):
        a0, b0 = a[2 * g], b[2 * g]
        a1 = a[2 * g + 1] if 2 * g + 1 < n else 0
        b1 = b[2 * g + 1] if 2 * g + 1 < n else 0
        out0.append(a0 * b0 * FR_RADIX_INV % R_MOD)
        out1.append((a0 * (b1 - b0) + b0 * (a1 - a0)) * FR_RADIX_INV % R_MOD)
        out2.append((a1 - a0) * (b1 - b0) * FR_RADIX_INV % R_MOD)
    return out0, out1, out2


def inner_product_sumcheck(a, b, u) -> list:
    """proof.cu:29-65"""
    a, b = list(a), list(b)
    if len(a) != len(b) or len(a) <= (1 << len(u)) // 2 or len(a) > (1 << len(u)):
        raise RuntimeError("Incompatible dimensions")
    proof = []
    for x in u:
        o0, o1, o2 = _legacy_ip_terms(a, b)
        proof += [sum(o0) % R_MOD, sum(o1) % R_MOD, sum(o2) % R_MOD]
        a, b = me_step(a, x), me_step(b, x)
    proof += [a[0], b[0]]
    return proof


def hadamard_product_sumcheck(a, b, u, v) -> list:
    """proof.cu:67-107"""
    a, b, u, v = list(a), list(b), list(u), list(v)
    if len(u) != len(v):
        raise RuntimeError("Incompatible dimensions 1")
    if len(a) != len(b):
        raise RuntimeError("Incompatible dimensions 2")
    if len(a) <= (1 << (len(u) - 1)):
        raise RuntimeError("Incompatible dimensions 3")
    if len(a) > (1 << len(u)):
        raise RuntimeError("Incompatible dimensions 4")
    proof = []
    for k in range(len(v)):
        o0, o1, o2 = _legacy_ip_terms(a, b)
        u_ = u[k + 1:]
        proof += [mle_eval(o0, u_), mle_eval(o1, u_), mle_eval(o2, u_)]
        a, b = me_step(a, v[k]), me_step(b, v[k])
    proof += [a[0], b[0]]
    return proof


def binary_sumcheck(a, u, v) -> list:
    """proof.cu:109-160; same R^-1 convention on the product terms only"""
    a, u, v = list(a), list(u), list(v)
    if len(u) != len(v) or len(a) <= (1 << len(u)) // 2 or len(a) > (1 << len(u)):
        raise RuntimeError("Incompatible dimensions")
    proof = []
    for k in range(len(v)):
        n = len(a)
        o0, o1, o2 = [], [], []
        for g in range((n + 1) // 2):
            a0 = a[2 * g]
            a1 = a[2 * g + 1] if 2 * g + 1 < n else 0
            d = (a1 - a0) % R_MOD
            o0.append((a0 * a0 * FR_RADIX_INV - a0) % R_MOD)
            o1.append((2 * a0 % R_MOD * d * FR_RADIX_INV - d) % R_MOD)
            o2.append(d * d * FR_RADIX_INV % R_MOD)
        u_ = u[k + 1:]
        proof += [mle_eval(o0, u_), mle_eval(o1, u_), mle_eval(o2, u_)]
        a = me_step(a, v[k])
    proof.append(a[0])
    return proof


# --- Rescaling (rescaling.cu:8-21) -----------------------------------------------------
def _c_mod(a: int, b: int) -> int:
    """C's truncating %"""
    q = abs(a) // abs(b)
    if (a < 0) != (b < 0):
        q = -q
    return a - q * b


def relu_decomp(X: list, sf: int):
    """zkrelu_decomp_kernel, zkrelu.cu:9-30: returns (sign, magnitude, remainder, relu) Fr lists of the rescaled values"""
    q, rem = rescale(X, sf)
    sign, mag, res = [], [], []
    for v in q:
        pos = v < (R_MOD + 1) // 2        # a non-negative small integer
        sign.append(1 if pos else 0)
        mag.append(v if pos else (R_MOD - v) % R_MOD)
        res.append(v if pos else 0)
    return sign, mag, rem, res


def rescale(X: list, sf: int):
    """returns (rescaled, remainder) Fr lists"""
    out, rem = [], []
    hsf = sf >> 1
    for x in X:
        xv = fr_to_long(x)
        t = _c_mod(xv + hsf, sf)
        x_rem = (t + sf if t < 0 else t) - hsf
        xr = xv - x_rem
        q = abs(xr) // sf
        out.append(int_to_fr(q if xr >= 0 else -q))
        rem.append(int_to_fr(x_rem))
    return out, rem


# --- G1 (bls12-381.cu:1361-1464: dbl-2009-l, madd-2007-bl, add-2007-bl) -----------------
G1_ZERO = (0, 0, 0)
G1_GEN = (G1_X, G1_Y, 1)


def g1_double(P):
    X1, Y1, Z1 = P
    if Z1 == 0:
        return G1_ZERO
    A = X1 * X1 % Q_MOD
    B = Y1 * Y1 % Q_MOD
    C = B * B % Q_MOD
    D = 2 * ((X1 + B) ** 2 - A - C) % Q_MOD
    E = 3 * A % Q_MOD
    F = E * E % Q_MOD
    X3 = (F - 2 * D) % Q_MOD
    Y3 = (E * (D - X3) - 8 * C) % Q_MOD
    Z3 = 2 * Y1 * Z1 % Q_MOD
    return (X3, Y3, Z3)


def g1_add(P, Q):
    X1, Y1, Z1 = P
    X2, Y2, Z2 = Q
    if Z1 == 0:
        return Q
    if Z2 == 0:
        return P
    Z1Z1 = Z1 * Z1 % Q_MOD
    Z2Z2 = Z2 * Z2 % Q_MOD
    U1 = X1 * Z2Z2 % Q_MOD
    U2 = X2 * Z1Z1 % Q_MOD
    S1 = Y1 * Z2 * Z2Z2 % Q_MOD
    S2 = Y2 * Z1 * Z1Z1 % Q_MOD
    if U1 == U2 and S1 == S2:
        return g1_double(P)
    H = (U2 - U1) % Q_MOD
    I = (2 * H) ** 2 % Q_MOD
    J = H * I % Q_MOD
    rr = 2 * (S2 - S1) % Q_MOD
    V = U1 * I % Q_MOD
    X3 = (rr * rr - J - 2 * V) % Q_MOD
    Y3 = (rr * (V - X3) - 2 * S1 * J) % Q_MOD
    Z3 = ((Z1 + Z2) ** 2 - Z1Z1 - Z2Z2) * H % Q_MOD
    return (X3, Y3, Z3)


def g1_neg(P):
    return (P[0], (-P[1]) % Q_MOD, P[2])


def g1_mul(P, k: int):
    """G1Jacobian_mul, g1-tensor.cu:445-453: double-and-add over the raw 256 scalar bits"""
    out = G1_ZERO
    a = P
    while k:
        if k & 1:
            out = g1_add(out, a)
        a = g1_double(a)
        k >>= 1
    return out


def g1_affine(P):
    """(x, y) ints, or None for the identity.  Parity on G1 outputs is defined on this."""
    X, Y, Z = P
    if Z == 0:
        return None
    zi = pow(Z, -1, Q_MOD)
    return (X * zi * zi % Q_MOD, Y * zi * zi * zi % Q_MOD)


def g1_on_curve(P) -> bool:
    a = g1_affine(P)
    return a is None or (a[1] * a[1] - a[0] ** 3 - 4) % Q_MOD == 0


def g1_sum(points):
    acc = G1_ZERO
    for p in points:
        acc = g1_add(acc, p)
    return acc


# --- Commitment (commitment.cu:22-141) ---------------------------------------------------
def commit_int(generators: list, scalars: list) -> list:
    """Commitment::commit_int, commitment.cu:31-58.  scalars are Fr ints that encode
    int32 values; each row of len(generators) scalars gives one G1 point."""
    n = len(generators)
    if len(scalars) % n:
        raise RuntimeError("Commitment::commit_int - Incompatible dimensions")
    out = []
    for r in range(len(scalars) // n):
        acc = G1_ZERO
        for j in range(n):
            s = fr_to_int(scalars[r * n + j])
            if s == 0:
                continue
            term = g1_mul(generators[j], abs(s))
            acc = g1_add(acc, term if s > 0 else g1_neg(term))
        out.append(acc)
    return out


def commit(generators: list, scalars: list) -> list:
    """Commitment::commit, commitment.cu:22-29 (full-width scalars)"""
    n = len(generators)
    if len(scalars) % n:
        raise RuntimeError("Commitment::commit - Incompatible dimensions")
    return [g1_sum(g1_mul(generators[j], scalars[r * n + j]) for j in range(n))
            for r in range(len(scalars) // n)]


def me_open(t: list, gens: list, u: list, proof: list) -> int:
    """Commitment::me_open, commitment.cu:79-129.  Appends the three G1 elements of
    every round and the final generator to `proof` (Jacobian int triples)."""
    t, gens = list(t), list(gens)
    if len(t) != len(gens):
        raise RuntimeError("Commitment::me_open - Incompatible dimensions %d %d" % (len(t), len(gens)))
    for x in u:
        old = len(t)
        new = (old + 1) // 2
        ns, ng, acc, acc0, acc1 = [], [], G1_ZERO, G1_ZERO, G1_ZERO
        for g in range(new):
            g0, g1i = 2 * g, 2 * g + 1
            if g1i >= old:
                ns.append((t[g0] - x * t[g0]) % R_MOD)
                ng.append(g1_mul(gens[g0], x))
                acc = g1_add(acc, g1_mul(gens[g0], t[g0]))
                continue
            ns.append((t[g0] + x * (t[g1i] - t[g0])) % R_MOD)
            ng.append(g1_add(gens[g1i], g1_mul(g1_add(gens[g0], g1_neg(gens[g1i])), x)))
            acc = g1_add(acc, g1_add(g1_mul(gens[g0], t[g0]), g1_mul(gens[g1i], t[g1i])))
            acc0 = g1_add(acc0, g1_mul(gens[g1i], t[g0]))
            acc1 = g1_add(acc1, g1_mul(gens[g0], t[g1i]))
        proof += [acc, acc0, acc1]
        t, gens = ns, ng
    proof.append(gens[0])
    return t[0]


def commitment_open(gens: list, t: list, com_size: int, u: list, proof: list | None = None) -> int:
    """Commitment::open, commitment.cu:133-141"""
    k = ceil_log2(com_size)
    u_out = u[len(u) - k:]
    u_in = u[:len(u) - k]
    folded = t if not u_out else _legacy_partial_me(t, u_out, len(t) // com_size)
    return me_open(folded, gens, u_in, proof if proof is not None else [])


def _legacy_partial_me(t: list, u: list, window: int) -> list:
    """FrTensor::partial_me(u, window_size), fr-tensor.cu:512-516,612-641"""
    if len(t) <= window * (1 << (len(u) - 1)):
        raise RuntimeError("partial_me: Incompatible dimensions")
    t = list(t)
    for x in u:
        n_in = len(t)
        nwin = (n_in + 2 * window - 1) // (2 * window)
        out = []
        for g in range(window * nwin):
            w, k = divmod(g, window)
            g0 = 2 * w * window + k
            g1i = (2 * w + 1) * window + k
            if g1i < n_in:
                out.append((t[g0] + x * (t[g1i] - t[g0])) % R_MOD)
            elif g0 < n_in:
                out.append((t[g0] - x * t[g0]) % R_MOD)
            else:
                out.append(0)
        t = out
    return t
