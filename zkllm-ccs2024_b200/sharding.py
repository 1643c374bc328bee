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
    evaluations at the low challenges, each weighted by eq(high challenges; rank).

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
