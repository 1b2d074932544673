"""The persistent kernels with several work items per CTA, stage by stage.

Shape B2 N2048 H16 Hk4 D128: 512 (head, row block) items in the forward and 512 (key block, head) items in pass 1 on at
most 148 CTAs, so every CTA walks three or four items and the state it carries across them (ring stages, buffer parities,
mbarrier phases, the double-buffered Q tile, the scale prefetch) is exercised.  Two kinds of check:
  * every stage against the CPU oracle, each fed the oracle's inputs for the stages before it;
  * the whole call against the same call made in head ranges small enough that no CTA gets a second item: the bits must
    be equal, whatever the walk.
"""
import pytest
import torch

from delta_matching_b200 import _lib
from oracle import dm_oracle as O

pytestmark = pytest.mark.gpu
B, N, H, Hk, D = 2, 2048, 16, 4, 128
HC = 4                       # heads per range: B * HC * (N / 128) = 128 items < 148 CTAs
_CACHE = {}


def _oracle(causal):
    if causal not in _CACHE:
        q, k, v, dO = O.make_inputs(B, N, H, Hk, D, 77)
        _CACHE[causal] = O.attention_fwd_bwd(q, k, v, dO, causal, "matched" if causal else "stale", fwd_tile_keys=128, pv="group",
                                             debug=True)
    return _CACHE[causal]


def _dev(r, *names):
    return [r[n].cuda() for n in names]


@pytest.mark.parametrize("causal", [True, False])
def test_forward_stage(causal):
    r = _oracle(causal)
    Q8, K8, V8, Q8s, K8s, V8s = _dev(r, "Q8", "K8", "V8", "Q8s", "K8s", "V8s")
    o, lse = _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal)
    assert _lib.device_status() == 0
    assert (lse.cpu() - r["LSE"]).abs().max() < 2e-4
    assert O.rel(o.cpu(), r["O"]) < 2e-3
    per_head = ((o.cpu().float() - r["O"].float()).norm(dim=(1, 3)) / r["O"].float().norm(dim=(1, 3))).max().item()
    assert per_head < 4e-3, per_head
    o2, lse2 = torch.zeros_like(o), torch.zeros_like(lse)
    for h0 in range(0, H, HC):
        _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal, h0=h0, hcount=HC, out=(o2, lse2))
    assert torch.equal(o, o2) and torch.equal(lse, lse2), "the walk over several items changed the forward's bits"


def test_matched_delta_stage():
    r = _oracle(True)
    args = _dev(r, "Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE")
    got = _lib.delta_fp8(*args, B, H, Hk, True)
    assert _lib.device_status() == 0
    ref = r["delta"]
    assert (got.cpu() - ref).abs().max() <= 2e-4 * ref.abs().max() + 1e-6
    rows, rabs = _lib.bwd_dbg_rowsum(*args, got, B, H, Hk, True)
    assert (rows.double().norm() / rabs.double().norm()).item() < 1e-6


@pytest.mark.parametrize("causal", [True, False])
def test_pass1_and_pass2_stages(causal):
    r = _oracle(causal)
    args = _dev(r, "Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE", "delta")
    dk, dv, ws = _lib.bwd_pass1(*args, B, H, Hk, causal)
    dq = _lib.bwd_pass2(ws, args[1], B, H, Hk, N, D, causal)
    assert _lib.device_status() == 0
    BH, nbn, nbm = B * H, N // 128, N // 64
    psi = ws[1].view(BH, nbm, nbn).cpu()
    ds8 = ws[0].view(BH, nbn, nbn, 128, 128).cpu()           # [bh, row block, key block, key, row]
    ref_ds = r["dS8"].view(torch.uint8).view(BH, nbn, 2, nbn, 64, 128).permute(0, 1, 3, 5, 2, 4).reshape(BH, nbn, nbn, 128, 128)
    m = torch.ones(nbm, nbn, dtype=torch.bool)
    mt = torch.ones(nbn, nbn, dtype=torch.bool)
    if causal:
        for mb in range(nbm):
            m[mb, mb // 2 + 1:] = False
        mt = mt.tril()
    assert torch.allclose(psi[:, m], r["psi"][:, m], rtol=2e-3, atol=0)
    a = ds8[:, mt].view(torch.float8_e4m3fn).float()
    b = ref_ds[:, mt].contiguous().view(torch.float8_e4m3fn).float()
    assert ((a - b).abs() > 0).float().mean() < 0.02 and O.rel(a, b) < 5e-3
    lay = lambda x: x.to(torch.bfloat16).view(B, H, N, D).permute(0, 2, 1, 3)
    assert O.rel(dv.cpu(), lay(r["dVh"])) < 2e-3
    assert O.rel(dk.cpu(), lay(r["dKh"])) < 3e-3
    assert O.rel(dq.cpu(), lay(r["dQh"])) < 3e-3
    for name, x, ref in (("dK", dk, r["dKh"]), ("dV", dv, r["dVh"]), ("dQ", dq, r["dQh"])):
        rf = lay(ref).float()
        per_head = ((x.cpu().float() - rf).norm(dim=(1, 3)) / rf.norm(dim=(1, 3))).max().item()
        assert per_head < 6e-3, (name, per_head)
    # the same in head ranges with one item per CTA: equal bits, workspace included
    dk2, dv2, dq2 = torch.zeros_like(dk), torch.zeros_like(dv), torch.zeros_like(dq)
    for h0 in range(0, H, HC):
        _, _, w = _lib.bwd_pass1(*args, B, H, Hk, causal, h0=h0, hcount=HC, out=(dk2, dv2))
        _lib.bwd_pass2(w, args[1], B, H, Hk, N, D, causal, h0=h0, hcount=HC, out=dq2)
        # workspace of a head range is [B, HC, ...]: compare with the matching heads of the whole call's
        whole = ws[0].view(B, H, -1)[:, h0:h0 + HC]
        part = w[0].view(B, HC, -1)
        if causal:
            t = mt.view(1, 1, nbn, nbn, 1).expand(B, HC, nbn, nbn, 128 * 128).reshape(B, HC, -1).to(part.device)
            assert torch.equal(whole[t], part[t])
        else:
            assert torch.equal(whole, part)
    assert _lib.device_status() == 0
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2) and torch.equal(dq, dq2), "the walk changed the backward's bits"


def test_pass1_fp32_partials_under_a_row_map_with_empty_key_blocks():
    """A rank of a sequence split holds rows [256, 512) and [1280, 1536): key blocks above its last row have no m-block
    at all (dK = dV = 0 there) and sit in the middle of a CTA's walk."""
    r = _oracle(True)
    cp = _lib.DmCp(512, 2, 2, 10)
    rows = torch.cat([torch.arange(256, 512), torch.arange(1280, 1536)])
    pick = lambda x, blk=1: x[:, (rows[::blk] // blk)].contiguous().cuda()
    Q8l, dO8l, LSEl, dll = pick(r["Q8"]), pick(r["dO8"]), pick(r["LSE"]), pick(r["delta"])
    Q8sl, dO8sl = pick(r["Q8s"], 128), pick(r["dO8s"], 128)
    K8, V8, K8s, V8s = _dev(r, "K8", "V8", "K8s", "V8s")
    args = (Q8l, K8, V8, dO8l, Q8sl, K8s, V8s, dO8sl, LSEl, dll)
    dk, dv, ws = _lib.bwd_pass1(*args, B, H, Hk, True, cp=cp, out_fp32=True)
    dq = _lib.bwd_pass2(ws, K8, B, H, Hk, N, D, True, cp=cp)
    assert _lib.device_status() == 0
    assert dk.dtype == torch.float32 and dk[:, 1536:].abs().max() == 0 and dv[:, 1536:].abs().max() == 0
    assert dk[:, :1536].abs().max() > 0
    dk2, dv2, dq2 = torch.full_like(dk, 7.0), torch.full_like(dv, 7.0), torch.zeros_like(dq)
    for h0 in range(0, H, 2):        # B * 2 * 16 key blocks = 64 items per call
        _, _, w = _lib.bwd_pass1(*args, B, H, Hk, True, h0=h0, hcount=2, out=(dk2, dv2), cp=cp, out_fp32=True)
        _lib.bwd_pass2(w, K8, B, H, Hk, N, D, True, h0=h0, hcount=2, out=dq2, cp=cp)
    assert _lib.device_status() == 0
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2) and torch.equal(dq, dq2)
    # dQ of the local rows is the whole-sequence dQ of those rows
    dq_ref = r["dQh"].to(torch.bfloat16).view(B, H, N, D).permute(0, 2, 1, 3)[:, rows]
    assert O.rel(dq.cpu(), dq_ref) < 3e-3
