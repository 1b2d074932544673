"""Multi-GPU partitioning of the attention path: (batch x KV-head) groups are independent in the forward and in every
backward pass, so a job is split by handing each rank whole KV groups (a KV head together with its H / Hk query heads, so
the GQA fold of dK / dV stays local).  No data-path collective exists; ranks only meet to report times.

`kv_group_range(B, Hk, rank, world)` gives a rank's contiguous range of flattened (batch, kv head) groups and
`shard_bnhd` cuts (B, N, heads, D) tensors accordingly.  Groups are flattened batch-major; a rank's range may cover
several batches with all their heads, or a slice of the heads of one batch -- never a partial mix, which keeps every shard
a plain (B', N, H', D) tensor: world must divide B * Hk, and either world divides B or B divides world.
"""
from __future__ import annotations


def kv_group_range(B: int, Hk: int, rank: int, world: int):
    """(first, count) of the flattened (batch, kv head) groups owned by `rank`."""
    total = B * Hk
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    if total % world:
        raise ValueError(f"batch * nheads_k ({total}) must be divisible by the number of ranks ({world})")
    if B % world and world % B:
        raise ValueError(f"cannot cut batch {B} x nheads_k {Hk} into {world} rectangular shards")
    per = total // world
    return rank * per, per


def shard_bnhd(q, k, v, rank: int, world: int, dO=None):
    """Views of q (B, N, H, D), k / v (B, N, Hk, D) (and dO) holding `rank`'s KV groups and their query heads."""
    B, N, H, D = q.shape
    Hk = k.shape[2]
    rep = H // Hk
    first, count = kv_group_range(B, Hk, rank, world)
    if count >= Hk:                       # whole batches
        b0, nb = first // Hk, count // Hk
        cut = lambda t: t[b0:b0 + nb]
        out = [cut(q), cut(k), cut(v)]
        if dO is not None:
            out.append(cut(dO))
        return out
    b, hk0 = first // Hk, first % Hk      # a slice of one batch's heads
    out = [q[b:b + 1, :, hk0 * rep:(hk0 + count) * rep], k[b:b + 1, :, hk0:hk0 + count], v[b:b + 1, :, hk0:hk0 + count]]
    if dO is not None:
        out.append(dO[b:b + 1, :, hk0 * rep:(hk0 + count) * rep])
    return out
