"""The backward kernels stage by stage against the CPU oracle: every stage is fed the oracle's inputs for the stages
before it, so a failure points at one kernel.  Then the structural identities of the matched delta."""
import pytest
import torch

from delta_matching_b200 import _lib
from oracle import dm_oracle as O

pytestmark = pytest.mark.gpu
CASES = [(1, 256, 2, 2, True), (1, 512, 4, 2, True), (2, 768, 2, 1, True), (1, 512, 2, 2, False)]


def _stage_inputs(B, N, H, Hk, causal, seed=1001, mode="matched"):
    q, k, v, dO = O.make_inputs(B, N, H, Hk, 128, seed)
    r = O.attention_fwd_bwd(q, k, v, dO, causal, mode if causal else "stale", fwd_tile_keys=128, pv="group", debug=True)
    return q, k, v, dO, r


def _dev(r, *names):
    return [r[n].cuda() for n in names]


@pytest.mark.parametrize("B,N,H,Hk,causal", CASES)
def test_matched_delta(B, N, H, Hk, causal):
    q, k, v, dO, r = _stage_inputs(B, N, H, Hk, causal)
    Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, LSE = _dev(r, "Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE")
    ref = O.matched_delta(r["Q8"], r["Q8s"], r["K8"], r["K8s"], r["V8"], r["V8s"], r["dO8"], r["dO8s"], r["LSE"], H, Hk, causal)
    got = _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, LSE, B, H, Hk, causal).cpu()
    assert _lib.device_status() == 0
    scale = ref.abs().max()
    assert (got - ref).abs().max() <= 2e-4 * scale + 1e-6, ((got - ref).abs().max(), scale)


@pytest.mark.parametrize("B,N,H,Hk,causal", CASES)
def test_pass1_and_pass2(B, N, H, Hk, causal):
    q, k, v, dO, r = _stage_inputs(B, N, H, Hk, causal)
    Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, LSE, delta = _dev(r, "Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE", "delta")
    dk, dv, ws = _lib.bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, LSE, delta, B, H, Hk, causal)
    assert _lib.device_status() == 0
    BH, nbn = B * H, N // 128
    # psi: [BH, N/64, N/128]
    psi = ws[1].view(BH, N // 64, nbn).cpu()
    ds8 = ws[0].view(BH, nbn, nbn, 128, 128).cpu()           # [bh, row block, key block, key, row]
    ref_psi = r["psi"]
    ref_ds = r["dS8"].view(torch.uint8).view(BH, nbn, 2, nbn, 64, 128).permute(0, 1, 3, 5, 2, 4).reshape(BH, nbn, nbn, 128, 128)
    if causal:
        m = torch.ones(N // 64, nbn, dtype=torch.bool)
        for mb in range(N // 64):
            m[mb, mb // 2 + 1:] = False
        mt = torch.ones(nbn, nbn, dtype=torch.bool).tril()
    else:
        m = torch.ones(N // 64, nbn, dtype=torch.bool)
        mt = torch.ones(nbn, nbn, dtype=torch.bool)
    assert torch.allclose(psi[:, m], ref_psi[:, m], rtol=2e-3, atol=0), (psi[:, m] - ref_psi[:, m]).abs().max()
    a = ds8[:, mt].view(torch.float8_e4m3fn).float()
    b = ref_ds[:, mt].contiguous().view(torch.float8_e4m3fn).float()
    # codes may flip by one e4m3 step where the fp32 accumulation order moved a value across a rounding boundary
    assert ((a - b).abs() > 0).float().mean() < 0.02, ((a - b).abs() > 0).float().mean()
    assert O.rel(a, b) < 5e-3
    dk_ref = r["dKh"].to(torch.bfloat16).view(B, H, N, 128).permute(0, 2, 1, 3)
    dv_ref = r["dVh"].to(torch.bfloat16).view(B, H, N, 128).permute(0, 2, 1, 3)
    assert O.rel(dv.cpu(), dv_ref) < 2e-3, O.rel(dv.cpu(), dv_ref)
    assert O.rel(dk.cpu(), dk_ref) < 3e-3, O.rel(dk.cpu(), dk_ref)
    dq = _lib.bwd_pass2(ws, K8, B, H, Hk, N, 128, causal).cpu()
    assert _lib.device_status() == 0
    dq_ref = r["dQh"].to(torch.bfloat16).view(B, H, N, 128).permute(0, 2, 1, 3)
    assert O.rel(dq, dq_ref) < 3e-3, O.rel(dq, dq_ref)


def test_pass2_alone_on_oracle_tiles():
    """Pass 2 fed the oracle's dS' codes and psi (re-laid into the kernel's [key][row] tiles) is the oracle's dQ."""
    B, N, H, Hk = 1, 512, 2, 1
    q, k, v, dO, r = _stage_inputs(B, N, H, Hk, True)
    BH, nbn = B * H, N // 128
    ds = r["dS8"].view(torch.uint8).view(BH, nbn, 2, nbn, 64, 128).permute(0, 1, 3, 5, 2, 4).reshape(-1).contiguous().cuda()
    ws = (ds, r["psi"].contiguous().cuda())
    dq = _lib.bwd_pass2(ws, r["K8"].cuda(), B, H, Hk, N, 128, True).cpu()
    dq_ref = r["dQh"].to(torch.bfloat16).view(B, H, N, 128).permute(0, 2, 1, 3)
    assert O.rel(dq, dq_ref) < 1e-3, O.rel(dq, dq_ref)


def test_rowsum_identity_matched_vs_stale():
    """rowsum(P-hat (dP - delta)) is zero to fp32 round-off with the matched delta and visibly not with the stale one."""
    B, N, H, Hk = 1, 512, 2, 2
    q, k, v, dO, r = _stage_inputs(B, N, H, Hk, True)
    args = _dev(r, "Q8", "K8", "V8", "dO8", "Q8s", "K8s", "V8s", "dO8s", "LSE")
    matched = _lib.delta_fp8(*args, B, H, Hk, True)
    stale = O.stale_delta(dO, r["O"]).cuda()
    res = {}
    for name, d in (("matched", matched), ("stale", stale)):
        rows, rabs = _lib.bwd_dbg_rowsum(*args, d, B, H, Hk, True)
        res[name] = (rows.double().norm() / rabs.double().norm()).item()
    assert _lib.device_status() == 0
    assert res["matched"] < 1e-6 and res["stale"] > 1e-3, res
