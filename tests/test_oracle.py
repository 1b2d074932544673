"""The CPU oracle against the reference's own quantizer outputs (golden vectors made by running the reference's Triton
kernels under Triton's interpreter) and against the reference's published contract for the attention passes."""
import os

import numpy as np
import pytest
import torch

from oracle import dm_oracle as O
from make_quant_golden import golden_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
E4M3 = torch.float8_e4m3fn


def _check_codes(name, exact, ours, theirs):
    """Codes must be equal except for the three documented defects of the interpreter's float8 cast: a value that lands
    exactly one binade low (theirs * 2 == ours), truncation instead of rounding inside the e4m3 subnormal range, and
    exact ties rounded away from zero instead of to even (hardware cvt.rn and this oracle round ties to even)."""
    ours, theirs = ours.float(), theirs.float()
    neq = ours != theirs
    assert neq.float().mean().item() < 0.10, name
    half = theirs * 2 == ours
    sub = (exact.abs() < 2.0 ** -6) & (theirs.abs() <= ours.abs()) & ((ours - theirs).abs() <= 2.0 ** -9)
    tie = (exact - ours).abs() == (exact - theirs).abs()
    bad = neq & ~half & ~sub & ~tie
    assert not bad.any(), f"{name}: {int(bad.sum())} code mismatches that are not an interpreter defect"


@pytest.mark.parametrize("D", [128, 256])
def test_quantizers_match_the_reference_kernels(D):
    g = np.load(os.path.join(GOLDEN, f"quant_d{D}.npz"))
    q, k, v, dO, Oo = golden_inputs(D)
    rq, rk = O.blocks(D)
    Q8, Q8s = O.quant_q(q)
    K8, K8s, km = O.quant_k(k)
    V8, V8s = O.quant_v(v)
    dO8, dO8s = O.quant_do(dO)
    assert np.array_equal(km.numpy(), g["km_frozen"]) and np.array_equal(km.numpy(), g["km_split"])
    sm = torch.tensor(D ** -0.5)
    exact = {"q": q.reshape(-1, 256, D).float() * sm, "k": k.reshape(-1, 256, D).float() - km[:, None],
             "v": v.reshape(-1, 256, D).float(), "do": dO.permute(0, 2, 1, 3).reshape(-1, 256, D).float()}
    for name, c, s, blk in (("q", Q8, Q8s, rq), ("k", K8, K8s, rk), ("v", V8, V8s, rk), ("do", dO8, dO8s, rq)):
        assert np.array_equal(s.numpy(), g[name + "8s"]), f"{name} scales differ from the reference kernel"
        theirs = torch.from_numpy(g[name + "8"]).view(E4M3)
        _check_codes(name, exact[name] / s.repeat_interleave(blk, 1)[..., None], c, theirs)
    # the all-zero blocks take the scale floor and give zero codes
    assert dO8s[0, 0].item() == np.float32(1e-30) * (np.float32(1.0) / np.float32(448.0)) and not dO8[0, :128].float().any()
    if D == 256:
        assert Q8s[0, 0].item() == np.float32(1e-30) / np.float32(448.0) and not Q8[0, :64].float().any()
    # stale delta: same value up to the (implementation-defined) summation order over d
    ds = O.stale_delta(dO, Oo)
    gd = torch.from_numpy(g["delta_stale"])
    assert (ds - gd).abs().max() <= 4e-7 * gd.abs().max()


def test_dO_scale_is_a_multiply_not_a_divide():
    x = torch.full((1, 128, 128), 0.3, dtype=torch.float32)
    _, s_div = O.quant_blocks(x, 128)
    _, s_mul = O.quant_blocks(x, 128, mul_inv=True)
    assert s_div.item() == np.float32(0.3) / np.float32(448.0)
    assert s_mul.item() == np.float32(0.3) * (np.float32(1.0) / np.float32(448.0))


@pytest.fixture(scope="module")
def cfg1():
    q, k, v, dO = O.make_inputs(1, 256, 2, 2, 128, 1001)
    return q, k, v, dO, O.fp32_reference(q, k, v, dO)


def test_config1_matched_contract(cfg1):
    """BASELINE config 1: relative error to fp32 attention inside the reference's bounds and rowsum(dS) = 0 to fp32
    round-off in the matched mode (violated by the stale delta)."""
    q, k, v, dO, (ro, rdq, rdk, rdv) = cfg1
    m = O.attention_fwd_bwd(q, k, v, dO, True, "matched", debug=True)
    s = O.attention_fwd_bwd(q, k, v, dO, True, "stale", debug=True)
    for r in (m, s):
        assert O.rel(r["O"], ro) < 0.08 and O.rel(r["dV"], rdv) < 0.08
        assert O.rel(r["dQ"], rdq) < 0.12 and O.rel(r["dK"], rdk) < 0.12
    assert torch.equal(m["O"], s["O"]) and torch.equal(m["dV"], s["dV"])
    assert not torch.equal(m["dQ"], s["dQ"]) and not torch.equal(m["dK"], s["dK"])
    res_m = (m["rows_sum"].norm() / m["rows_abs"].norm()).item()
    res_s = (s["rows_sum"].norm() / s["rows_abs"].norm()).item()
    assert res_m < 1e-6 and res_s > 1e-3


def test_forward_realizations_agree(cfg1):
    """The reference's 256-key tile with the rho chain and the 128-key tile with one fold per key group are the same
    sum in two rounding orders."""
    q, k, v, dO, _ = cfg1
    a = O.attention_fwd_bwd(q, k, v, dO, True, "matched")
    b = O.attention_fwd_bwd(q, k, v, dO, True, "matched", fwd_tile_keys=128, pv="group")
    assert O.rel(b["O"], a["O"]) < 1e-3 and (a["LSE"] - b["LSE"]).abs().max() < 1e-5
    assert O.rel(b["dQ"], a["dQ"]) < 1e-3


def test_fp64_accumulate_is_close_to_fp32(cfg1):
    q, k, v, dO, _ = cfg1
    a = O.attention_fwd_bwd(q, k, v, dO, True, "matched")
    b = O.attention_fwd_bwd(q, k, v, dO, True, "matched", acc=torch.float64)
    for n in ("O", "dQ", "dK", "dV"):
        assert O.rel(a[n], b[n]) < 2e-3


def test_gqa_noncausal_stale_and_d256():
    q, k, v, dO = O.make_inputs(1, 256, 4, 2, 128, 7)
    ro, rdq, rdk, rdv = O.fp32_reference(q, k, v, dO, causal=False)
    r = O.attention_fwd_bwd(q, k, v, dO, False, "stale")
    assert r["dK"].shape == k.shape and r["dV"].shape == v.shape
    assert O.rel(r["O"], ro) < 0.08 and O.rel(r["dV"], rdv) < 0.08 and O.rel(r["dQ"], rdq) < 0.12 and O.rel(r["dK"], rdk) < 0.12
    q, k, v, dO = O.make_inputs(1, 128, 2, 1, 256, 8)
    ro, rdq, rdk, rdv = O.fp32_reference(q, k, v, dO, causal=False)
    r = O.attention_fwd_bwd(q, k, v, dO, False, "stale")
    assert O.rel(r["O"], ro) < 0.08 and O.rel(r["dV"], rdv) < 0.08 and O.rel(r["dQ"], rdq) < 0.12 and O.rel(r["dK"], rdk) < 0.12
