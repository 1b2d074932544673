"""dm_attn_func_cp over a real process group: one process per GPU, NCCL, the sequence split in zig-zag chunks.  Needs two
or more GPUs (skipped otherwise).  Every rank also runs the whole sequence on its own GPU and compares its rows: O and dQ
bit for bit, dK / dV within the rounding of a differently ordered fp32 sum."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def _worker(rank, world, port, shape, mode):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import delta_matching_b200 as dm
        from delta_matching_b200 import _lib
        B, N, H, Hk, D = shape
        g = torch.Generator().manual_seed(11)
        mk = lambda h: torch.randn(B, N, h, D, generator=g).to(torch.bfloat16).to(dev)
        q, k, v, dO = mk(H), mk(Hk), mk(Hk), mk(H)
        # whole sequence on this GPU
        qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
        o_ref = dm.dm_attn_func(qf, kf, vf, causal=True, mode=mode)
        o_ref.backward(dO)
        # this rank's rows through the ring
        ql, kl, vl = (dm.zigzag_shard(t, rank, world).requires_grad_(True) for t in (q, k, v))
        o = dm.dm_attn_func_cp(ql, kl, vl, causal=True, mode=mode)
        o.backward(dm.zigzag_shard(dO, rank, world))
        torch.cuda.synchronize()
        assert _lib.device_status() == 0
        sh = lambda t: dm.zigzag_shard(t, rank, world)
        assert torch.equal(o, sh(o_ref.detach())), "O"
        assert torch.equal(ql.grad, sh(qf.grad)), "dQ"
        assert _rel(kl.grad, sh(kf.grad)) < 6e-3, ("dK", _rel(kl.grad, sh(kf.grad)))
        assert _rel(vl.grad, sh(vf.grad)) < 6e-3, ("dV", _rel(vl.grad, sh(vf.grad)))
        # twice the same bits
        ql2, kl2, vl2 = (t.detach().clone().requires_grad_(True) for t in (ql, kl, vl))
        o2 = dm.dm_attn_func_cp(ql2, kl2, vl2, causal=True, mode=mode)
        o2.backward(dm.zigzag_shard(dO, rank, world))
        assert torch.equal(o2, o) and torch.equal(kl2.grad, kl.grad) and torch.equal(vl2.grad, vl.grad) and torch.equal(ql2.grad, ql.grad)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_ring_equals_whole_sequence(mode):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    world = 4 if world >= 4 else 2
    mp.spawn(_worker, args=(world, _free_port(), (1, 1024 * world, 8, 2, 128), mode), nprocs=world, join=True)
