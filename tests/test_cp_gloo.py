"""The context-parallel exchange on CPU ranks (gloo): the zig-zag row ownership, the ring that makes K-side data whole in
sequence order, and the route of dK / dV partials to the ranks that own the keys, summed there in rank order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from delta_matching_b200 import cp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _partial(rank, B, N, Hk, D):
    g = torch.Generator().manual_seed(100 + rank)
    return torch.randn(B, N, Hk, D, generator=g)


def _worker(rank, world, port, N):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    B, Hk, D = 2, 2, 8
    g = torch.Generator().manual_seed(7)
    codes = torch.randint(0, 255, (B * Hk, N, D), generator=g, dtype=torch.uint8)       # whole-sequence K-side data
    scales = torch.randn(B * Hk, N // 64, generator=g)
    mine = (cp.zigzag_shard(codes, rank, world), cp.zigzag_shard(scales, rank, world))
    # the ring: every rank's packed block arrives, listed by rank; unpacked and put in sequence order it is the whole
    got = [cp._unpack(b, mine) for b in cp.ring_all_gather(cp._pack(mine))]
    assert torch.equal(cp._sequence_order([x[0] for x in got]), codes)
    assert torch.equal(cp._sequence_order([x[1] for x in got]), scales)
    # partials for every key go to the key's owner; slices arrive in rank order
    part = _partial(rank, B, N, Hk, D)
    recv = cp.exchange_to_owners(cp.owner_slices(part, world))
    for s in range(world):
        assert torch.equal(recv[s], cp.zigzag_shard(_partial(s, B, N, Hk, D), rank, world)), (rank, s)
    total = recv[0].clone()
    for s in range(1, world):
        total += recv[s]
    want = _partial(0, B, N, Hk, D)
    for s in range(1, world):
        want = want + _partial(s, B, N, Hk, D)
    assert torch.equal(total, cp.zigzag_shard(want, rank, world))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ring_and_owner_exchange(world):
    mp.spawn(_worker, args=(world, _free_port(), 512 * world), nprocs=world, join=True)


def test_zigzag_geometry():
    N, W = 4096, 4
    rows = torch.cat([cp.zigzag_rows(r, W, N) for r in range(W)])
    assert torch.equal(rows.sort().values, torch.arange(N))                 # every row has exactly one owner
    for r in range(W):
        m = cp.zigzag_map(r, W, N)
        assert (m.nq, m.half_blocks, m.off0, m.off1) == (1024, 4, 4 * r, 4 * (2 * W - 1 - r))
        # causal work per rank: (row block, key block) tiles at or below the diagonal are balanced by the zig-zag
        blocks = [m.off0 + i for i in range(m.half_blocks)] + [m.off1 + i for i in range(m.nq // 128 - m.half_blocks)]
        assert sum(b + 1 for b in blocks) == (N // 128) * (N // 128 + 1) // 2 // W
    x = torch.arange(2 * N * 3).view(2, N, 3)
    assert torch.equal(cp.zigzag_unshard([cp.zigzag_shard(x, r, W) for r in range(W)]), x)
    with pytest.raises(ValueError):
        cp.zigzag_map(0, 4, 4096 + 512)
    with pytest.raises(ValueError):
        cp.zigzag_map(0, 3, 2048)
