"""Context parallelism for long sequences: the sequence is split across the ranks of a process group, one GPU each.

The reference has no sequence parallelism (its long-context tool is the head split of delta_matching/split.py:17-92);
this module is the ring that the 65536-token configuration runs on at 8 GPUs.  head_dim 128 only.

Layout.  With W ranks the sequence is cut into 2W chunks of c = N / (2W) rows and rank r holds chunks r and 2W-1-r
(zig-zag), so that under a causal mask every rank owns the same number of (row block, key block) tiles.  A rank's q, k, v,
dO, O, dq, dk, dv are (B, 2c, heads, D): chunk r first, chunk 2W-1-r second.

Exchange.  K-side data is small next to the attention work (the e4m3 codes of K and V are N*D bytes per KV head), so it
is made whole on every rank before the kernels run:
  1. per-64-row-chunk column sums of K travel round the ring; every rank folds all of them in sequence order, which
     gives the K mean of the whole sequence with the bits a single GPU computes;
  2. every rank quantizes its own K (centred by that mean) and V, and the codes with their scales travel round the ring
     (W-1 send/recv steps to the next rank, NCCL over NVLink);
  3. forward, pass 0, pass 1 and pass 2 run on the local rows against the whole K8 / V8 through a row map (DmCp);
  4. pass 1 leaves fp32 dK / dV partials for every key of the sequence; they are folded over the query heads of a KV
     group, sent to the ranks that own the keys, and summed there in rank order, then rounded to bf16 once.
O, LSE, delta and dQ of a row depend only on that row and on K / V, so they carry the bits of a single-GPU run; dK and dV
differ from it only by the order of the fp32 sum over row blocks.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib
from .core import _check_inputs

__all__ = ["zigzag_map", "zigzag_rows", "zigzag_shard", "zigzag_unshard", "ring_all_gather", "exchange_to_owners",
           "dm_attn_func_cp"]


# ----------------------------------------------------------------------------------------------------------------------
# geometry
# ----------------------------------------------------------------------------------------------------------------------
def chunk_rows(N: int, world: int) -> int:
    c, rem = divmod(N, 2 * world)
    if rem or c % 256:
        raise ValueError(f"context parallelism over {world} ranks needs seqlen divisible by {512 * world} "
                         f"(two chunks of a multiple of 256 rows per rank); got {N}")
    return c


def zigzag_map(rank: int, world: int, N: int) -> "_lib.DmCp":
    """Row map of rank `rank`: chunk `rank` then chunk 2*world-1-rank, in 128-row blocks."""
    c = chunk_rows(N, world)
    return _lib.DmCp(2 * c, c // 128, rank * (c // 128), (2 * world - 1 - rank) * (c // 128))


def zigzag_rows(rank: int, world: int, N: int) -> torch.Tensor:
    """Global row indices (int64, CPU) of the rows rank `rank` holds, in local order (N = rows of any per-row or per-block
    tensor, a multiple of 2 * world)."""
    c, rem = divmod(N, 2 * world)
    if rem:
        raise ValueError(f"{N} rows do not split into {2 * world} chunks")
    return torch.cat([torch.arange(rank * c, (rank + 1) * c), torch.arange((2 * world - 1 - rank) * c, (2 * world - rank) * c)])


def zigzag_shard(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """The rows of a whole-sequence tensor that rank `rank` holds (a copy)."""
    return x.index_select(dim, zigzag_rows(rank, world, x.shape[dim]).to(x.device)).contiguous()


def zigzag_unshard(parts, dim: int = 1) -> torch.Tensor:
    """Inverse of zigzag_shard: the whole-sequence tensor from the per-rank tensors, listed by rank."""
    world = len(parts)
    c = parts[0].shape[dim] // 2
    chunks = [None] * (2 * world)
    for r, p in enumerate(parts):
        chunks[r], chunks[2 * world - 1 - r] = p.narrow(dim, 0, c), p.narrow(dim, c, c)
    return torch.cat(chunks, dim=dim)


# ----------------------------------------------------------------------------------------------------------------------
# communication (device-agnostic: NCCL on GPUs, gloo in the CPU tests)
# ----------------------------------------------------------------------------------------------------------------------
def _peer(group, idx: int) -> int:
    return idx if group is None or group is dist.group.WORLD else dist.get_global_rank(group, idx)


def ring_all_gather(x: torch.Tensor, group=None):
    """All ranks' `x` (same shape everywhere), listed by rank, moved by W-1 ring steps: at every step a rank passes the
    block it received last to the next rank and takes a new one from the previous rank."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    out = [None] * world
    out[rank] = x
    nxt, prv = _peer(group, (rank + 1) % world), _peer(group, (rank - 1) % world)
    for step in range(1, world):
        src = (rank - step) % world
        buf = torch.empty_like(x)
        ops = [dist.P2POp(dist.isend, out[(rank - step + 1) % world], nxt, group), dist.P2POp(dist.irecv, buf, prv, group)]
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        out[src] = buf
    return out


def exchange_to_owners(x: torch.Tensor, group=None) -> torch.Tensor:
    """x is [W, ...]: slice d is this rank's contribution to what rank d owns.  Returns [W, ...] whose slice s is rank s's
    contribution to what THIS rank owns (slice order = rank order, which fixes the order of the sum that follows)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    x = x.contiguous()
    assert x.shape[0] == world
    out = torch.empty_like(x)
    out[rank].copy_(x[rank])
    ops = []
    for step in range(1, world):
        dst, src = (rank + step) % world, (rank - step) % world
        ops.append(dist.P2POp(dist.isend, x[dst], _peer(group, dst), group))
        ops.append(dist.P2POp(dist.irecv, out[src], _peer(group, src), group))
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    return out


def _pack(tensors):
    return torch.cat([t.contiguous().view(torch.uint8).reshape(-1) for t in tensors])


def _unpack(buf, like):
    out, at = [], 0
    for t in like:
        nb = t.numel() * t.element_size()
        out.append(buf[at:at + nb].view(t.dtype).reshape(t.shape))
        at += nb
    return out


def _sequence_order(parts, dim: int = 1):
    """Per-rank [BH, 2 * c', ...] tensors (listed by rank) -> [BH, 2W * c', ...] in sequence order."""
    return zigzag_unshard(parts, dim=dim).contiguous()


# ----------------------------------------------------------------------------------------------------------------------
# the per-rank compute, callable without a process group (the tests drive it for every rank on one GPU)
# ----------------------------------------------------------------------------------------------------------------------
def local_forward(q, K8, K8s, V8, V8s, cp, B, H, Hk, causal):
    Q8, Q8s = _lib.quant(0, q)
    o, lse = _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal, cp=cp)
    return o, lse, Q8, Q8s


def heads_per_call(B, H, Hk, nq, N, limit_bytes=None):
    """Query heads per pass-1 / pass-2 call of a rank: whole KV groups, as many as keep the dS' tiles (B * heads * nq * N
    bytes) inside the workspace limit of the head-group split (DM_BWD_WS_LIMIT_GB, 8 GiB by default), and a divisor of H."""
    from . import split
    limit = split._BWD_WS_LIMIT if limit_bytes is None else limit_bytes
    rep = H // Hk
    best = rep
    for groups in range(1, Hk + 1):
        if Hk % groups == 0 and B * groups * rep * nq * N <= limit:
            best = groups * rep
    return best


def local_backward(dO, o, lse, Q8, Q8s, K8, K8s, V8, V8s, cp, B, H, Hk, causal, matched, fold=True):
    """dq (B, nq, H, D) bf16 and this rank's fp32 partial dK, dV over its local rows: (B, N, Hk, D), folded over the query
    heads of each KV group, or with fold=False the per-query-head partials (B, N, H, D) as pass 1 left them.  Pass 1 and
    pass 2 run per group of KV groups (heads_per_call), so the dS' workspace stays bounded at long sequences."""
    dO8, dO8s, delta = _lib.quant_do(dO, None if matched else o)
    if matched:
        delta = _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal, cp=cp)
    N, D, nq = K8.shape[1], K8.shape[2], Q8.shape[1]
    hp = heads_per_call(B, H, Hk, nq, N)
    dev = Q8.device
    dkp = torch.empty(B, N, H, D, device=dev, dtype=torch.float32)
    dvp = torch.empty(B, N, H, D, device=dev, dtype=torch.float32)
    dq = torch.empty(B, nq, H, D, device=dev, dtype=torch.bfloat16)
    ws = None
    for h0 in range(0, H, hp):
        _, _, ws = _lib.bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal, h0=h0, hcount=hp, out=(dkp, dvp),
                                  ws=ws, cp=cp, out_fp32=True)
        _lib.bwd_pass2(ws, K8, B, H, Hk, N, D, causal, h0=h0, hcount=hp, out=dq, cp=cp)
    del ws
    if not fold:
        return dq, dkp, dvp
    return (dq,) + fold_query_heads(dkp, dvp, B, N, H, Hk, D)


def fold_query_heads(dkp, dvp, B, N, H, Hk, D):
    """(B, N, H, D) fp32 partials per query head -> (B, N, Hk, D): the sum over the query heads of a KV group, in head order."""
    if H != Hk:
        dkp = _lib.fold_f32(dkp.view(B, N, Hk, H // Hk, D), 3)
        dvp = _lib.fold_f32(dvp.view(B, N, Hk, H // Hk, D), 3)
    return dkp, dvp


def owner_slices(x, world: int):
    """(B, N, Hk, D) -> [W, B, 2c, Hk, D]: slice d holds the rows rank d owns (its two chunks)."""
    B, N = x.shape[0], x.shape[1]
    c = N // (2 * world)
    v = x.view(B, 2 * world, c, *x.shape[2:])
    first = v[:, :world]                                  # chunks 0 .. W-1 belong to ranks 0 .. W-1
    second = v[:, world:].flip(1)                         # chunks 2W-1 .. W belong to ranks 0 .. W-1
    return torch.cat([first, second], dim=2).transpose(0, 1).contiguous()


# ----------------------------------------------------------------------------------------------------------------------
# autograd
# ----------------------------------------------------------------------------------------------------------------------
class _DMAttnCP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, matched, group):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        B, nq, H, D = q.shape
        Hk = k.shape[2]
        N = nq * world
        cp = zigzag_map(rank, world, N)
        # 1. the K mean of the whole sequence
        part = _lib.kmean_partials(k)                                              # [B*Hk, nq/64, D]
        km = _lib.kmean_fold(_sequence_order(ring_all_gather(part, group)), B, Hk, N, D)
        # 2. local codes, then the ring
        K8l, K8sl = _lib.quant(1, k, km)
        V8l, V8sl = _lib.quant(2, v)
        like = (K8l, V8l, K8sl, V8sl)
        got = [_unpack(b, like) for b in ring_all_gather(_pack(like), group)]
        K8, V8, K8s, V8s = (_sequence_order([g[i] for g in got]) for i in range(4))
        del got
        # 3. forward on the local rows
        o, lse, Q8, Q8s = local_forward(q, K8, K8s, V8, V8s, cp, B, H, Hk, causal)
        ctx.save_for_backward(o, lse, Q8, Q8s, K8, K8s, V8, V8s)
        ctx.meta = (cp, B, H, Hk, causal, matched, group, world)
        return o

    @staticmethod
    def backward(ctx, dO):
        o, lse, Q8, Q8s, K8, K8s, V8, V8s = ctx.saved_tensors
        cp, B, H, Hk, causal, matched, group, world = ctx.meta
        dq, dkp, dvp = local_backward(dO, o, lse, Q8, Q8s, K8, K8s, V8, V8s, cp, B, H, Hk, causal, matched, fold=False)
        # 4. the partials are folded over the query heads straight into one slice per owner of the keys, go there in one
        # exchange after the last pass, and are summed in rank order.  (Exchanging group by group on a second stream beside the
        # next group's passes was slower: the persistent kernels give every SM a fixed share of the items, so the SMs that an
        # exchange kernel holds while it waits for its peer finish their share late and the whole launch waits for them.)
        both = _lib.fold_to_owners(dkp, dvp, Hk, world)                                       # [W, 2, B, 2c, Hk, D]
        del dkp, dvp
        dkv = _lib.fold_f32(exchange_to_owners(both, group), 0, torch.bfloat16)               # [2, B, 2c, Hk, D]
        return dq, dkv[0], dkv[1], None, None, None


def dm_attn_func_cp(q, k, v, causal: bool = True, mode: str = "matched", group=None):
    """Delta-Matching fp8 attention over a sequence split across the ranks of `group` (default: the world group).

    q (B, N/W, H, 128), k / v (B, N/W, Hk, 128) bf16: this rank's two zig-zag chunks of the sequence (see zigzag_shard).
    Returns this rank's rows of O; backward returns this rank's rows of dq, dk, dv.  Same numerics contract and argument
    checks as dm_attn_func."""
    _check_inputs(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal, None, mode)
    if q.shape[-1] != 128:
        raise ValueError("context parallelism is built for head_dim 128 only")
    if k.shape[1] != q.shape[1]:
        raise ValueError("context parallelism is self-attention: q and k must hold the same local rows")
    chunk_rows(q.shape[1] * dist.get_world_size(group), dist.get_world_size(group))
    return _DMAttnCP.apply(q, k, v, causal, mode == "matched", group)
