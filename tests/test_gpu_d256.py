"""head_dim 256 (BASELINE config 4's geometry: Q / dO scales per 64 rows, K / V scales per 32 keys, psi per 64 x 64 tile):
the stale-delta path end to end against the CPU oracle and fp32 attention, and pass 1 / pass 2 stage by stage."""
import math

import pytest
import torch

import delta_matching_b200 as dm
from delta_matching_b200 import _lib
from oracle import dm_oracle as O

pytestmark = pytest.mark.gpu
TOL = {"O": 8e-2, "dV": 8e-2, "dQ": 1.2e-1, "dK": 1.2e-1}


def _run(q, k, v, do, mode, causal):
    q, k, v = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
    o = dm.dm_attn_func(q, k, v, causal=causal, mode=mode)
    o.backward(do.cuda())
    return o.detach().cpu(), q.grad.cpu(), k.grad.cpu(), v.grad.cpu()


@pytest.mark.parametrize("B,N,H,Hk,causal", [(1, 256, 2, 2, False), (1, 384, 4, 1, True), (2, 512, 4, 2, False)])
def test_stale_d256_matches_oracle_and_fp32(B, N, H, Hk, causal):
    q, k, v, do = O.make_inputs(B, N, H, Hk, 256, 2004)
    r = O.attention_fwd_bwd(q, k, v, do, causal, "stale", fwd_tile_keys=128, pv="group")
    ref = O.fp32_reference(q, k, v, do, causal)
    got = _run(q, k, v, do, "stale", causal)
    assert _lib.device_status() == 0
    for name, a, b in zip(("O", "dQ", "dK", "dV"), got, ref):
        e = O.rel(a, b)
        assert math.isfinite(e) and e < TOL[name], f"{name} vs fp32 attention: {e:.4f}"
    for name, a in zip(("O", "dQ", "dK", "dV"), got):
        e = O.rel(a, r[name])
        assert e < 4e-3, f"{name}: relative difference to the oracle {e:.2e}"


def test_d256_pass1_stage_and_determinism():
    B, N, H, Hk, causal = 1, 512, 2, 1, True
    q, k, v, do = O.make_inputs(B, N, H, Hk, 256, 2005)
    r = O.attention_fwd_bwd(q, k, v, do, causal, "stale", fwd_tile_keys=128, pv="group", debug=True)
    d = {n: r[n].cuda() for n in ("Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE", "delta")}
    args = (d["Q8"], d["K8"], d["V8"], d["dO8"], d["Q8s"], d["K8s"], d["V8s"], d["dO8s"], d["LSE"], d["delta"])
    dk, dv, ws = _lib.bwd_pass1(*args, B, H, Hk, causal)
    dk2, dv2, ws2 = _lib.bwd_pass1(*args, B, H, Hk, causal)
    assert _lib.device_status() == 0
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    BH, nbm, nbn = B * H, N // 64, N // 128
    psi = ws[1].view(BH, nbm, nbm).cpu()
    m = torch.ones(nbm, nbm, dtype=torch.bool).tril()                    # 64 x 64 tiles at or below the diagonal
    assert torch.allclose(psi[:, m], r["psi"][:, m], rtol=2e-3, atol=0)
    # kernel tile [row block, key block, key 128, row 128]  <-  oracle [m-block, key half block, row 64, key 64]
    ds = ws[0].view(BH, nbn, nbn, 128, 128).cpu()
    ref = r["dS8"].view(torch.uint8).view(BH, nbn, 2, nbn, 2, 64, 64).permute(0, 1, 3, 4, 6, 2, 5).reshape(BH, nbn, nbn, 128, 128)
    mt = torch.ones(nbn, nbn, dtype=torch.bool).tril()
    a = ds[:, mt].view(torch.float8_e4m3fn).float()
    b = ref[:, mt].contiguous().view(torch.float8_e4m3fn).float()
    if causal:                                                           # upper 64 x 64 quarter of diagonal tiles: never written by the oracle's loop
        pass
    assert O.rel(a, b) < 5e-3, O.rel(a, b)
    dk_ref = r["dKh"].to(torch.bfloat16).view(B, H, N, 256).permute(0, 2, 1, 3)
    dv_ref = r["dVh"].to(torch.bfloat16).view(B, H, N, 256).permute(0, 2, 1, 3)
    assert O.rel(dv.cpu(), dv_ref) < 2e-3 and O.rel(dk.cpu(), dk_ref) < 3e-3
    dq = _lib.bwd_pass2(ws, d["K8"], B, H, Hk, N, 256, causal).cpu()
    dq_ref = r["dQh"].to(torch.bfloat16).view(B, H, N, 256).permute(0, 2, 1, 3)
    assert O.rel(dq, dq_ref) < 3e-3


@pytest.mark.parametrize("B,N,H,Hk", [(1, 384, 4, 1), (2, 256, 2, 2)])
def test_matched_d256_matches_oracle_and_keeps_the_rowsum_identity(B, N, H, Hk):
    q, k, v, do = O.make_inputs(B, N, H, Hk, 256, 2006)
    r = O.attention_fwd_bwd(q, k, v, do, True, "matched", fwd_tile_keys=128, pv="group", debug=True)
    ref = O.fp32_reference(q, k, v, do, True)
    got = _run(q, k, v, do, "matched", True)
    for name, a, b in zip(("O", "dQ", "dK", "dV"), got, ref):
        assert O.rel(a, b) < TOL[name], name
    for name, a in zip(("O", "dQ", "dK", "dV"), got):
        assert O.rel(a, r[name]) < 4e-3, name
    d = [r[n].cuda() for n in ("Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE")]
    delta = _lib.delta_fp8(*d, B, H, Hk, True)
    assert (delta.cpu() - r["delta"]).abs().max() <= 2e-4 * r["delta"].abs().max() + 1e-6
    rows, rabs = _lib.bwd_dbg_rowsum(*d, delta, B, H, Hk, True)
    assert (rows.double().norm() / rabs.double().norm()).item() < 1e-6
    stale = O.stale_delta(do, r["O"]).cuda()
    rows, rabs = _lib.bwd_dbg_rowsum(*d, stale, B, H, Hk, True)
    assert (rows.double().norm() / rabs.double().norm()).item() > 1e-3
    assert _lib.device_status() == 0
