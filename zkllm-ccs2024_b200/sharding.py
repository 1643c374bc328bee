"""Host-side logic of the multi-GPU paths: one process per GPU, torch.distributed
for the exchange steps.

The reference is single-GPU.  Work is split only where the prover's algebra
splits without changing any result:

  * row commitments are independent MSMs over shared generators: rank g takes a
    contiguous block of rows and the m commitments are all-gathered in rank order;
  * sums of field elements (round-polynomial coefficients of a sharded sumcheck)
    are gathered and added modulo r on every rank - modular addition is not a
    reduction NCCL offers;
  * a sum of G1 points is gathered and added in rank order;
  * a multilinear evaluation (FrTensor::operator()(u), fr-tensor.cu:437-442) of a
    tensor split into equal contiguous blocks is the sum of the blocks' own
    evaluations at the low challenges, each weighted by eq(high challenges; rank);
  * the inner-product sumcheck (zkip, zkfc.cu:94-151) pairs index i with i + N/2, so
    with the vectors dealt out round-robin (rank p holds i = p, p + P, ...) every
    round but the last log2 P is local.  All challenges are arguments, so a rank
    runs all its local rounds back to back (zkb_zkip_partial) and the ranks exchange
    their coefficient sums and their one surviving pair ONCE; the last log2 P rounds
    and the verifier replay then run on every rank on P-element vectors.

Everything here runs on the `gloo` backend as well, which is how it is tested
without GPUs.
"""
from __future__ import annotations

import numpy as np

R_MOD = 0x73EDA753299D7D483339D80809A1D80553BDA402FFFE5BFEFFFFFFFF00000001


def row_shard(m: int, world: int, rank: int) -> tuple:
    """[begin, end) of the rows rank `rank` commits; the first m % world ranks take one more"""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    base, extra = divmod(m, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def all_gather_rows(local, m: int, row_words: int, group=None):
    """Gathers per-rank row blocks (torch int32 tensor of [rows_local * row_words]) into the
    full [m * row_words] tensor, in rank order.  Shards may differ in size by one row."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = [row_shard(m, world, r) for r in range(world)]
    max_rows = max(e - b for b, e in sizes)
    padded = torch.zeros(max_rows * row_words, dtype=local.dtype, device=local.device)
    padded[: local.numel()] = local
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded, group=group)
    return torch.cat([bufs[r][: (e - b) * row_words] for r, (b, e) in enumerate(sizes)])


def fr_limbs_to_ints(a: np.ndarray) -> list:
    b = np.ascontiguousarray(a, dtype=np.uint32).tobytes()
    return [int.from_bytes(b[i:i + 32], "little") for i in range(0, len(b), 32)]


def fr_ints_to_limbs(vals) -> np.ndarray:
    buf = b"".join(int(v % R_MOD).to_bytes(32, "little") for v in vals)
    return np.frombuffer(buf, dtype=np.uint32).reshape(-1, 8).copy()


def fr_allreduce_sum(partials: np.ndarray, group=None) -> np.ndarray:
    """Every rank passes k partial sums ((k, 8) uint32, standard form) and receives the k
    sums modulo r.  96-160 bytes per rank and round: latency, not bandwidth."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = "cuda" if backend == "nccl" else "cpu"
    t = torch.from_numpy(np.ascontiguousarray(partials, dtype=np.uint32).view(np.int32).copy()).to(dev)
    bufs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(bufs, t, group=group)
    k = partials.shape[0]
    acc = [0] * k
    for b in bufs:
        for i, v in enumerate(fr_limbs_to_ints(b.cpu().numpy().view(np.uint32).reshape(k, 8))):
            acc[i] = (acc[i] + v) % R_MOD
    return fr_ints_to_limbs(acc)


def block_weight(u_high, rank: int) -> int:
    """eq(u_high; rank): challenge j pairs with bit j of the rank (the index bits above a block)"""
    w = 1
    for j, u in enumerate(u_high):
        w = w * (u if (rank >> j) & 1 else (1 - u)) % R_MOD
    return w


def sharded_mle_combine(local_value: np.ndarray, u_high, group=None) -> np.ndarray:
    """The tensor is split into world = 2^len(u_high) equal contiguous blocks, rank p holding block p.
    `local_value` ((1, 8) uint32) is this rank's block evaluated at the low challenges (zkb_fr_mle_eval
    on the block); returns the evaluation of the whole tensor at (u_low, u_high) on every rank."""
    import torch.distributed as dist

    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if world != 1 << len(u_high):
        raise ValueError("world size must be 2^len(u_high)")
    v = fr_limbs_to_ints(local_value)[0]
    return fr_allreduce_sum(fr_ints_to_limbs([v * block_weight(u_high, rank) % R_MOD]), group)


def zkip_local_rounds(n_local: int) -> int:
    """rounds a rank can run alone on its round-robin share of n_local (a power of two) entries"""
    if n_local < 1 or n_local & (n_local - 1):
        raise ValueError("the local share must be a power of two long")
    return n_local.bit_length() - 1


def zkip_combine(per_rank, u, claim: int):
    """per_rank[p] = (sums, tail_a, tail_b) of rank p in integers: `sums` the 3 coefficient sums of each local
    round, tail_a / tail_b the share as folded by those rounds (one entry each when every local round ran).
    u: all k challenges (consumed from the back, as zkip does).  Returns (polys, final_claim): the k round
    polynomials [c0, c1, c2] and the claim after the last round - what zkip on the whole vectors produces.
    Raises RuntimeError("claim != p(0) + p(1)") like the reference when a round does not verify."""
    world = len(per_rank)
    if world < 1 or world & (world - 1):
        raise ValueError("the number of ranks must be a power of two")
    n_local_rounds = len(per_rank[0][0])
    polys = [[sum(pr[0][r][c] for pr in per_rank) % R_MOD for c in range(3)] for r in range(n_local_rounds)]
    # entry j of rank p is global index j * world + p
    tail = len(per_rank[0][1])
    a = [per_rank[i % world][1][i // world] for i in range(tail * world)]
    b = [per_rank[i % world][2][i // world] for i in range(tail * world)]
    k = len(u)
    for r in range(n_local_rounds, k):
        v = u[k - 1 - r]
        half = len(a) // 2
        if half < 1:
            raise ValueError("more challenges than variables")
        c0 = c1 = c2 = 0
        na, nb = [], []
        for g in range(half):
            da, db = a[g + half] - a[g], b[g + half] - b[g]
            c0 += a[g] * b[g]
            c1 += a[g] * db + b[g] * da
            c2 += da * db
            na.append((a[g] + v * da) % R_MOD)
            nb.append((b[g] + v * db) % R_MOD)
        polys.append([c0 % R_MOD, c1 % R_MOD, c2 % R_MOD])
        a, b = na, nb
    for r, (c0, c1, c2) in enumerate(polys):
        if claim != (2 * c0 + c1 + c2) % R_MOD:
            raise RuntimeError("claim != p(0) + p(1)")
        v = u[k - 1 - r]
        claim = (c0 + v * (c1 + v * c2)) % R_MOD
    return polys, claim


def sharded_zkip(local_sums: np.ndarray, tail_a: np.ndarray, tail_b: np.ndarray, u, claim: int, group=None):
    """The exchange step: every rank passes what zkb_zkip_partial returned for its share ((rounds*3, 8),
    (tail, 8), (tail, 8) uint32) and receives (polys, final_claim) of the whole sumcheck."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    rounds, tail = local_sums.shape[0] // 3, tail_a.shape[0]
    payload = np.concatenate([np.ascontiguousarray(x, dtype=np.uint32).reshape(-1, 8) for x in (local_sums, tail_a, tail_b)])
    t = torch.from_numpy(payload.view(np.int32).copy()).to(dev)
    bufs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(bufs, t, group=group)
    per_rank = []
    for bfr in bufs:
        vals = fr_limbs_to_ints(bfr.cpu().numpy().view(np.uint32).reshape(-1, 8))
        sums = [vals[3 * r:3 * r + 3] for r in range(rounds)]
        per_rank.append((sums, vals[3 * rounds:3 * rounds + tail], vals[3 * rounds + tail:3 * rounds + 2 * tail]))
    return zkip_combine(per_rank, u, claim)


# ---- zkFC::prove (zkfc.cu:61-87) with the weights split over the ranks -------------------
# W [I, O] is dealt out by rows round-robin and X [B, I] by the matching columns: rank p
# holds W[p::P, :] and X[:, p::P]; Y [B, O] is on every rank.  The heavy pass - every
# entry of W once - is local, and the inner-product sumcheck over I splits as zkip does.

def zkfc_local_part(z, d_X_local, d_W_local, B: int, I_local: int, O: int, u_batch, u_input, u_output, world: int):
    """One rank's device work through the C ABI (z: the loaded binding).  u_*: (k, 8) uint32 challenge arrays;
    the first log2(world) entries of u_input belong to the rank index.  Returns host integers:
    (sums, tail_a, tail_b, X_local(u_batch, u_input_high), W_local(u_input_high, u_output))."""
    kP = world.bit_length() - 1
    kI = u_input.shape[0]
    u_in_high = fr_host_or_dummy(u_input[kP:])
    x_red, w_red = z.DeviceBuffer(32 * I_local), z.DeviceBuffer(32 * I_local)
    if u_batch.shape[0]:
        z.call("zkb_fr_partial_me", z._p(d_X_local), z.sz(B * I_local), z._p(fr_host_or_dummy(u_batch)), z.u32(u_batch.shape[0]),
               z.sz(B), z.sz(I_local), z._p(x_red), z._p(0))
    else:
        z.call("zkb_memcpy_d2d", z._p(x_red), z._p(d_X_local), z.sz(32 * I_local), z._p(0))
    if u_output.shape[0]:
        z.call("zkb_fr_partial_me", z._p(d_W_local), z.sz(I_local * O), z._p(fr_host_or_dummy(u_output)), z.u32(u_output.shape[0]),
               z.sz(O), z.sz(1), z._p(w_red), z._p(0))
    else:
        z.call("zkb_memcpy_d2d", z._p(w_red), z._p(d_W_local), z.sz(32 * I_local), z._p(0))
    rounds = zkip_local_rounds(I_local)
    sums = np.zeros((max(3 * rounds, 1), 8), dtype=np.uint32)
    ta, tb = np.zeros((1, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_zkip_partial", z._p(x_red), z._p(w_red), z.sz(I_local), z._p(fr_host_or_dummy(u_input)), z.u32(kI), z.u32(rounds),
           z._p(sums), z._p(ta), z._p(tb), z._p(0))
    cx, cw = np.zeros((1, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_fr_mle_eval_2d", z._p(d_X_local), z.sz(B), z.sz(I_local), z._p(fr_host_or_dummy(u_batch)), z.u32(u_batch.shape[0]),
           z._p(u_in_high), z.u32(kI - kP), z._p(cx), z._p(0))
    z.call("zkb_fr_mle_eval_2d", z._p(d_W_local), z.sz(I_local), z.sz(O), z._p(u_in_high), z.u32(kI - kP),
           z._p(fr_host_or_dummy(u_output)), z.u32(u_output.shape[0]), z._p(cw), z._p(0))
    v = fr_limbs_to_ints(sums)
    return ([v[3 * r:3 * r + 3] for r in range(rounds)], fr_limbs_to_ints(ta), fr_limbs_to_ints(tb),
            fr_limbs_to_ints(cx)[0], fr_limbs_to_ints(cw)[0])


def fr_host_or_dummy(limbs: np.ndarray) -> np.ndarray:
    """a valid (k, 8) uint32 array for a challenge vector that may be empty"""
    a = np.ascontiguousarray(limbs, dtype=np.uint32).reshape(-1, 8)
    return a if a.shape[0] else np.zeros((1, 8), dtype=np.uint32)


def zkfc_combine(parts, claim: int, u_input_ints):
    """parts[p] = zkfc_local_part of rank p; claim = Y(u_batch, u_output).  Returns the dictionary zkFC::prove's
    body produces: proof polynomials, final claim, claim_X, claim_W; raises "Claim does not match" like the
    reference when claim_X * claim_W differs from the final claim."""
    world = len(parts)
    kP = world.bit_length() - 1
    polys, final = zkip_combine([(s_, a_, b_) for s_, a_, b_, _, _ in parts], u_input_ints, claim)
    u_rank = u_input_ints[:kP]
    claim_x = sum(block_weight(u_rank, p) * parts[p][3] for p in range(world)) % R_MOD
    claim_w = sum(block_weight(u_rank, p) * parts[p][4] for p in range(world)) % R_MOD
    if claim_x * claim_w % R_MOD != final:
        raise RuntimeError("Claim does not match")
    return {"proof": polys, "claim": claim, "final_claim": final, "claim_x": claim_x, "claim_w": claim_w}


def sharded_zkfc_prove(z, d_X_local, d_W_local, d_Y, B: int, I_local: int, O: int, u_batch, u_input, u_output, group=None):
    """zkFC::prove's body over torch.distributed: local passes, ONE all-gather of a few hundred bytes, the shared
    last rounds and the verifier replay on every rank (zkb_zkip_combine, the C++ twin of zkip_combine).  Returns the
    dictionary of zkfc_combine with the proof as a (3 k, 8) uint32 array."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    kP = world.bit_length() - 1
    part = zkfc_local_part(z, d_X_local, d_W_local, B, I_local, O, u_batch, u_input, u_output, world)
    claim = np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_fr_mle_eval_2d", z._p(d_Y), z.sz(B), z.sz(O), z._p(fr_host_or_dummy(u_batch)), z.u32(u_batch.shape[0]),
           z._p(fr_host_or_dummy(u_output)), z.u32(u_output.shape[0]), z._p(claim), z._p(0))
    rounds = len(part[0])
    flat = [c for r_ in part[0] for c in r_] + part[1] + part[2] + [part[3], part[4]]
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.from_numpy(fr_ints_to_limbs(flat).view(np.int32).copy()).to(dev)
    bufs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(bufs, t, group=group)
    allp = torch.stack(bufs).cpu().numpy().view(np.uint32).reshape(world, 3 * rounds + 4, 8)
    k = u_input.shape[0]
    polys, final = np.zeros((max(3 * k, 1), 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_zkip_combine", z._p(np.ascontiguousarray(allp[:, :3 * rounds + 2])), z.u32(world), z.u32(k),
           z._p(fr_host_or_dummy(u_input)), z._p(claim), z._p(polys), z._p(final))
    u_rank = fr_limbs_to_ints(u_input[:kP])
    cx = fr_limbs_to_ints(np.ascontiguousarray(allp[:, 3 * rounds + 2]))
    cw = fr_limbs_to_ints(np.ascontiguousarray(allp[:, 3 * rounds + 3]))
    claim_x = sum(block_weight(u_rank, p) * cx[p] for p in range(world)) % R_MOD
    claim_w = sum(block_weight(u_rank, p) * cw[p] for p in range(world)) % R_MOD
    fin = fr_limbs_to_ints(final)[0]
    if claim_x * claim_w % R_MOD != fin:
        raise RuntimeError("Claim does not match")
    return {"proof": polys[:3 * k], "claim": fr_limbs_to_ints(claim)[0], "final_claim": fin, "claim_x": claim_x, "claim_w": claim_w}


# ---- tLookup::prove (tlookup.cu:281-370) split the same way -------------------------------
# S (D values), the table T and the multiplicities m (N each) are dealt out round-robin; a rank
# runs its log2(D/P) local rounds (zkb_tlookup_partial) with the challenges of its own index
# bits: u[log2 P:] for the eq weights, and v without the log2 P entries of the shared last rounds
# (tlookup_local_challenges).  The eq weight of the rank's own low bits is one constant per rank.

def tlookup_local_challenges(u, v, D: int, N: int, world: int):
    """(u_local, v_local) to hand to zkb_tlookup_partial on a rank's share; u, v: sequences of the global challenges"""
    kP = world.bit_length() - 1
    k1 = (D // N).bit_length() - 1
    return list(u[kP:]), list(v[:k1]) + list(v[k1 + kP:])


def tlookup_combine(per_rank, D: int, N: int, alpha: int, beta: int, u, v):
    """per_rank[p] = (sums, A, S, B, T, m) of rank p in integers: sums = what zkb_tlookup_partial returned for ALL the
    rank's local rounds (1 + 11 per round), A..m its surviving entries (one each).  u, v: the global challenges.
    Returns (polys, final_claim) - the log2(D) round polynomials [c0..c3] and the claim tLookup::prove returns; raises
    RuntimeError with the reference's message when a round does not verify."""
    world = len(per_rank)
    kP = world.bit_length() - 1
    kD, kN = D.bit_length() - 1, N.bit_length() - 1
    k1 = kD - kN
    if world & (world - 1) or kN < kP:
        raise ValueError("the number of ranks must be a power of two and at most the table size")
    n_local = kD - kP
    w = [block_weight(u[:kP], p) for p in range(world)]
    bm = sum(pr[0][0] for pr in per_rank) % R_MOD
    rounds = []
    for r in range(n_local):
        weighted = 3 if r < k1 else 6
        row = []
        for c in range(11):
            if c < weighted:
                row.append(sum(w[p] * per_rank[p][0][1 + 11 * r + c] for p in range(world)) % R_MOD)
            else:
                row.append(sum(per_rank[p][0][1 + 11 * r + c] for p in range(world)) % R_MOD)
        rounds.append(row)
    # the last log2(world) rounds on the surviving entries: entry of rank p is index p
    arr = [[per_rank[p][1 + a][0] for p in range(world)] for a in range(5)]
    for r in range(n_local, kD):
        A, S, B, T, m = arr
        half = len(A) // 2
        nbits = half.bit_length() - 1
        vv = v[kD - 1 - (r - k1)]
        q = [0] * 11
        nxt = [[], [], [], [], []]
        for g in range(half):
            e = block_weight(u[:nbits], g)
            a0, a1, s0, s1 = A[g], A[g + half], S[g], S[g + half]
            c01, c10, c11 = a1 - a0, s0 + beta, s1 - s0
            q[0] += e * a0 * c10
            q[1] += e * (a0 * c11 + c01 * c10)
            q[2] += e * c01 * c11
            q[6] += a0
            q[7] += c01
            nxt[0].append((a0 + vv * c01) % R_MOD)
            nxt[1].append((s0 + vv * c11) % R_MOD)
            b0, b1, t0, t1, m0, m1f = B[g], B[g + half], T[g], T[g + half], m[g], m[g + half]
            d01, d10, d11 = b1 - b0, t0 + beta, t1 - t0
            q[3] += e * b0 * d10
            q[4] += e * (b0 * d11 + d01 * d10)
            q[5] += e * d01 * d11
            m1 = m1f - m0
            q[8] += m0 * b0
            q[9] += m0 * d01 + m1 * b0
            q[10] += m1 * d01
            nxt[2].append((b0 + vv * d01) % R_MOD)
            nxt[3].append((t0 + vv * d11) % R_MOD)
            nxt[4].append((m0 + vv * m1) % R_MOD)
        rounds.append([x % R_MOD for x in q])
        arr = nxt
    # assembly of the round polynomials and the verifier replay, as the single-GPU prover does on the host
    inv = lambda x: pow(x, R_MOD - 2, R_MOD)
    two_inv = inv(2)
    al, al_sq = alpha, alpha * alpha % R_MOD
    C = (al_sq - bm) % R_MOD
    claim = (alpha + al_sq) % R_MOD
    inv_ratio = N * inv(D) % R_MOD
    polys = []
    for r, q in enumerate(rounds):
        ub = u[kD - 1 - r]
        e0, e1 = (1 - ub) % R_MOD, (2 * ub - 1) % R_MOD
        if r < k1:
            p0 = [al * q[i] % R_MOD for i in range(3)]
            vb = v[k1 - 1 - r]
        else:
            coef_b = inv_ratio * al_sq % R_MOD
            p0 = [(al * q[i] + coef_b * q[3 + i]) % R_MOD for i in range(3)]
            vb = v[kD - 1 - (r - k1)]
        p = [p0[0] * e0, p0[1] * e0 + p0[0] * e1, p0[2] * e0 + p0[1] * e1, p0[2] * e1]
        if r < k1:
            p[0] += q[3] + C * two_inv
            p[1] += q[4]
        else:
            p[0] += q[6] - q[8] * inv_ratio
            p[1] += q[7] - q[9] * inv_ratio
            p[2] -= q[10] * inv_ratio
        p = [x % R_MOD for x in p]
        polys.append(p)
        if claim != (2 * p[0] + p[1] + p[2] + p[3]) % R_MOD:
            raise RuntimeError("tLookup_phase1: claim != p(0) + p(1)" if r < k1 else "tLookup_phase2: claim != p(0) + p(1)")
        claim = (p[0] + vb * (p[1] + vb * (p[2] + vb * p[3]))) % R_MOD
        e = (ub * vb + (1 - ub) * (1 - vb)) % R_MOD
        al = al * e % R_MOD
        if r < k1:
            C = C * two_inv % R_MOD
        else:
            al_sq = al_sq * e % R_MOD
    return polys, claim


def sharded_tlookup_prove(z, d_S_local, d_T_local, d_m_local, D: int, N: int, alpha: np.ndarray, beta: np.ndarray,
                          u: np.ndarray, v: np.ndarray, group=None):
    """tLookup::prove over torch.distributed: rank p holds S[p::P], T[p::P], m[p::P] on its GPU (device buffers of the
    binding z); alpha, beta: (1, 8) uint32; u, v: (log2 D, 8) uint32, the global challenges.  Local rounds through
    zkb_tlookup_partial, ONE all-gather, then zkb_tlookup_combine (the C++ twin of tlookup_combine) on every rank.
    Returns (polys, final_claim) as (4 log2 D, 8) and (1, 8) uint32 arrays; raises z.ZkbError when a round fails."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    kP = world.bit_length() - 1
    kD = D.bit_length() - 1
    k1 = (D // N).bit_length() - 1
    u = np.ascontiguousarray(u, dtype=np.uint32).reshape(-1, 8)
    v = np.ascontiguousarray(v, dtype=np.uint32).reshape(-1, 8)
    ul = fr_host_or_dummy(u[kP:])
    vl = fr_host_or_dummy(np.concatenate([v[:k1], v[k1 + kP:]]))
    rounds = kD - kP
    part = np.zeros((1 + 11 * rounds + 5, 8), dtype=np.uint32)
    z.call("zkb_tlookup_partial", z._p(d_S_local), z._p(d_T_local), z._p(d_m_local), z.sz(D // world), z.sz(N // world),
           z._p(np.ascontiguousarray(beta, dtype=np.uint32)), z._p(ul), z._p(vl), z.u32(rounds), z._p(part),
           z._p(part[1 + 11 * rounds:]), z._p(0))
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.from_numpy(part.view(np.int32)).to(dev)
    bufs = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(bufs, t, group=group)
    parts = np.ascontiguousarray(torch.stack(bufs).cpu().numpy().view(np.uint32))
    polys, final = np.zeros((4 * kD, 8), dtype=np.uint32), np.zeros((1, 8), dtype=np.uint32)
    z.call("zkb_tlookup_combine", z._p(parts), z.u32(world), z.sz(D), z.sz(N), z._p(np.ascontiguousarray(alpha, dtype=np.uint32)),
           z._p(np.ascontiguousarray(beta, dtype=np.uint32)), z._p(fr_host_or_dummy(u)), z._p(fr_host_or_dummy(v)), z._p(polys),
           z._p(final))
    return polys, final


# ---- multi_hadamard_sumchecks (proof.cu:190-241) split the same way ------------------------
# The K tensors are dealt out round-robin.  Round r weights the K + 1 coefficients of
# prod_k (X_k[g] + t (X_k[g + M/2] - X_k[g])) by eq over the variables below the current one; that
# weight factors into eq over the rank's index bits (one constant per rank) and eq over the rest, so
# a rank runs its log2(N/P) rounds alone with u[log2 P:], v[log2 P:] (zkb_multi_hadamard_partial) and
# the exchange carries its sums and its K surviving entries.

def multi_hadamard_local_rounds(Xs_local, u_local, v_local):
    """A rank's own rounds in integers (what zkb_multi_hadamard_partial computes on the device): returns
    (sums, tails) - the K + 1 coefficient sums of every round and the K surviving entries."""
    Xs = [[int(x) % R_MOD for x in X] for X in Xs_local]
    u, v = list(u_local), list(v_local)
    K, sums = len(Xs), []
    while len(Xs[0]) > 1:
        half = len(Xs[0]) // 2
        below = len(u) - 1
        c = [0] * (K + 1)
        for g in range(half):
            prod = [1] + [0] * K
            for j, X in enumerate(Xs):
                a0, d = X[g], (X[g + half] - X[g]) % R_MOD
                for i in range(j + 1, 0, -1):
                    prod[i] = (prod[i] * a0 + prod[i - 1] * d) % R_MOD
                prod[0] = prod[0] * a0 % R_MOD
            e = block_weight(u[:below], g)
            c = [(ci + e * pi) % R_MOD for ci, pi in zip(c, prod)]
        sums.append(c)
        Xs = [[(X[g] + v[-1] * (X[g + half] - X[g])) % R_MOD for g in range(half)] for X in Xs]
        u, v = u[:-1], v[:-1]
    return sums, [X[0] for X in Xs]


def multi_hadamard_combine(per_rank, u, v, claim: int):
    """per_rank[p] = (sums, tails) of rank p as multi_hadamard_local_rounds returns them for its share X_k[p::P] with
    the challenges u[log2 P:], v[log2 P:].  u, v: the global challenges.  Returns (polys, final_claim) - what
    multi_hadamard_sumchecks on the whole tensors pushes and returns; raises RuntimeError with the reference's message."""
    world = len(per_rank)
    if world < 1 or world & (world - 1):
        raise ValueError("the number of ranks must be a power of two")
    kP = world.bit_length() - 1
    K = len(per_rank[0][1])
    n_local = len(per_rank[0][0])
    w = [block_weight(u[:kP], p) for p in range(world)]
    polys = [[sum(w[p] * per_rank[p][0][r][i] for p in range(world)) % R_MOD for i in range(K + 1)] for r in range(n_local)]
    more, _ = multi_hadamard_local_rounds([[per_rank[p][1][j] for p in range(world)] for j in range(K)], u[:kP], v[:kP])
    polys += more
    kN = n_local + kP
    for r, c in enumerate(polys):
        ub, vb = u[kN - 1 - r], v[kN - 1 - r]
        e0, e1 = (1 - ub) % R_MOD, (2 * ub - 1) % R_MOD
        if claim != (c[0] * e0 + sum(c) * (e0 + e1)) % R_MOD:
            raise RuntimeError("multi_hadamard_sumchecks: claim != p(0) + p(1)")
        acc = 0
        for coef in reversed(c):
            acc = (acc * vb + coef) % R_MOD
        claim = acc
    return polys, claim


def sharded_multi_hadamard(sums, tails, u, v, claim: int, group=None):
    """The exchange step: every rank passes its (sums, tails) in integers and receives (polys, final_claim)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    per_rank = [None] * world
    dist.all_gather_object(per_rank, (sums, tails), group=group)
    return multi_hadamard_combine(per_rank, u, v, claim)
