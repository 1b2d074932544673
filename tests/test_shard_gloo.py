"""The multi-GPU partitioning on CPU ranks (gloo, world size 2): each rank runs the oracle on its (batch x KV-head) shard,
the shards are gathered, and the result must equal the unsharded run bit for bit (heads and batches are independent, and
the GQA fold stays inside a shard)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from delta_matching_b200.shard import kv_group_range, shard_bnhd
from oracle import dm_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, cfg, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    B, N, H, Hk, D = cfg
    q, k, v, dO = O.make_inputs(B, N, H, Hk, D, 1234)
    qs, ks, vs, dos = shard_bnhd(q, k, v, rank, world, dO)
    r = O.attention_fwd_bwd(qs.contiguous(), ks.contiguous(), vs.contiguous(), dos.contiguous(), True, "matched")
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)          # the only collective the path uses: max-over-ranks of a time
    assert t.item() == world
    torch.save({n: r[n] for n in ("O", "dQ", "dK", "dV")}, os.path.join(out_dir, f"rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("cfg", [(2, 256, 4, 2, 128), (1, 256, 4, 2, 128)])
def test_two_rank_sharding_equals_the_unsharded_run(cfg, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), cfg, str(tmp_path)), nprocs=world, join=True)
    B, N, H, Hk, D = cfg
    q, k, v, dO = O.make_inputs(B, N, H, Hk, D, 1234)
    full = O.attention_fwd_bwd(q, k, v, dO, True, "matched")
    parts = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]
    dim = 0 if B % world == 0 else 2
    for n in ("O", "dQ", "dK", "dV"):
        got = torch.cat([p[n] for p in parts], dim=dim)
        assert torch.equal(got, full[n]), n


def test_group_ranges():
    assert kv_group_range(4, 8, 3, 8) == (12, 4)
    assert kv_group_range(1, 8, 7, 8) == (7, 1)
    assert [kv_group_range(2, 16, r, 4)[0] for r in range(4)] == [0, 8, 16, 24]
    with pytest.raises(ValueError):
        kv_group_range(1, 8, 0, 3)
    with pytest.raises(ValueError):
        kv_group_range(3, 4, 0, 2)
