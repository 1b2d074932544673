"""Context-parallel row maps on one GPU: every rank's kernels are run in turn on the same device against the whole K8 / V8,
and the pieces are compared with the plain whole-sequence run.  O, LSE, delta and dQ must carry the same bits; dK / dV are
sums of fp32 partials in another order, so they are compared within a rounding bound and against fp32 attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, N, H, Hk, D, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda h: torch.randn(B, N, h, D, generator=g).to(torch.bfloat16).cuda()
    return mk(H), mk(Hk), mk(Hk), mk(H)


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


@pytest.mark.parametrize("world,causal,matched", [(2, True, True), (4, True, True), (2, True, False), (2, False, False)])
def test_row_map_matches_whole_sequence(world, causal, matched):
    from delta_matching_b200 import _lib, cp as cpm
    from oracle import dm_oracle as orc

    B, N, H, Hk, D = 1, 2048, 4, 2, 128
    q, k, v, dO = _inputs(B, N, H, Hk, D, 5)
    # the whole-sequence run through the plain entry points
    o_ref, lse_ref, Q8, Q8s, K8, K8s, V8, V8s = _lib.attn_forward(q, k, v, causal)
    dq_ref, dk_ref, dv_ref = _lib.attn_backward(dO, o_ref, lse_ref, Q8, Q8s, K8, K8s, V8, V8s, B, H, Hk, causal, matched)

    # the K mean from per-rank partials folded in sequence order carries the same bits
    parts = [_lib.kmean_partials(cpm.zigzag_shard(k, r, world)) for r in range(world)]
    km = _lib.kmean_fold(cpm.zigzag_unshard(parts), B, Hk, N, D)
    assert torch.equal(km, _lib.kmean(k))
    # and so do the per-rank K / V codes put back in sequence order
    kq = [_lib.quant(1, cpm.zigzag_shard(k, r, world), km) for r in range(world)]
    assert torch.equal(cpm.zigzag_unshard([x[0] for x in kq]).view(torch.uint8), K8.view(torch.uint8))
    assert torch.equal(cpm.zigzag_unshard([x[1] for x in kq]), K8s)

    o_parts, dq_parts, dk_parts, dv_parts = [], [], [], []
    for r in range(world):
        m = cpm.zigzag_map(r, world, N)
        ql, dOl = cpm.zigzag_shard(q, r, world), cpm.zigzag_shard(dO, r, world)
        o, lse, Q8l, Q8sl = cpm.local_forward(ql, K8, K8s, V8, V8s, m, B, H, Hk, causal)
        assert torch.equal(lse, cpm.zigzag_shard(lse_ref, r, world, dim=1))
        dq, dkp, dvp = cpm.local_backward(dOl, o, lse, Q8l, Q8sl, K8, K8s, V8, V8s, m, B, H, Hk, causal, matched)
        o_parts.append(o), dq_parts.append(dq), dk_parts.append(cpm.owner_slices(dkp, world)), dv_parts.append(cpm.owner_slices(dvp, world))
    assert _lib.device_status() == 0
    assert torch.equal(cpm.zigzag_unshard(o_parts), o_ref)
    assert torch.equal(cpm.zigzag_unshard(dq_parts), dq_ref)
    # owner d receives slice d of every rank's partials and sums them in rank order
    dk = cpm.zigzag_unshard([_lib.fold_f32(torch.stack([p[d] for p in dk_parts]), 0, torch.bfloat16) for d in range(world)])
    dv = cpm.zigzag_unshard([_lib.fold_f32(torch.stack([p[d] for p in dv_parts]), 0, torch.bfloat16) for d in range(world)])
    assert _rel(dk, dk_ref) < 6e-3 and _rel(dv, dv_ref) < 6e-3       # bf16 rounding of two differently ordered fp32 sums
    _, _, dk32, dv32 = orc.fp32_reference(q.cpu(), k.cpu(), v.cpu(), dO.cpu(), causal)
    assert _rel(dk.cpu(), dk32) < 0.12 and _rel(dv.cpu(), dv32) < 0.08


def test_fold_f32_ordered_sum():
    from delta_matching_b200 import _lib
    x = torch.randn(3, 5, 8, 128, device="cuda")
    want = x[:, 0].clone()
    for c in range(1, 5):
        want = want + x[:, c]
    assert torch.equal(_lib.fold_f32(x, 1), want)
    assert torch.equal(_lib.fold_f32(x, 1, torch.bfloat16), want.to(torch.bfloat16))


@pytest.mark.parametrize("world,H,Hk", [(2, 8, 2), (4, 4, 4), (8, 6, 2)])
def test_fold_to_owners_is_the_head_fold_then_the_row_gather(world, H, Hk):
    from delta_matching_b200 import _lib, cp as cpm
    B, N, D = 2, 64 * world, 128
    dkp, dvp = torch.randn(B, N, H, D, device="cuda"), torch.randn(B, N, H, D, device="cuda")
    fk, fv = cpm.fold_query_heads(dkp, dvp, B, N, H, Hk, D)
    want = torch.stack([cpm.owner_slices(fk, world), cpm.owner_slices(fv, world)], dim=1)
    got = _lib.fold_to_owners(dkp, dvp, Hk, world)
    assert got.shape == want.shape and torch.equal(got, want)
    with pytest.raises(RuntimeError, match="multiple of 2 x ranks"):
        _lib.fold_to_owners(dkp[:, :N - 1].contiguous(), dvp[:, :N - 1].contiguous(), Hk, world)


def test_row_map_is_validated():
    from delta_matching_b200 import _lib
    Q8 = torch.zeros(2, 512, 128, device="cuda").to(_lib.E4M3)
    K8 = torch.zeros(2, 1024, 128, device="cuda").to(_lib.E4M3)
    s = torch.ones(2, 16, device="cuda")
    for bad in (_lib.DmCp(512, 2, 1, 6), _lib.DmCp(512, 2, 0, 8), _lib.DmCp(384, 2, 0, 6), _lib.DmCp(512, 2, 4, 2)):
        with pytest.raises(RuntimeError):
            _lib.fwd_fp8(Q8, K8, K8, s, s, s, 1, 2, 2, True, cp=bad)
