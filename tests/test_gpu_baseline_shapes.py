"""Parity at the benchmark's own shapes, where one persistent CTA walks several work items.

The forward and pass 1 launch min(items, SMs) CTAs that walk their items in a snake order, carrying ring stages, buffer
parities and mbarrier phases from one item to the next.  Shapes with fewer items than SMs never start a second item, so
every case here has several items per CTA: the GPU always runs the WHOLE configuration (so the walk is the one the
benchmark times) and the CPU oracle checks the whole result, or, where that would take minutes, a sample of its
independent (batch, KV group) slices.  The shapes and seeds are the synthetic stand-ins of the five benchmark
configurations (q, k, v, dO drawn in that order from CPU generator seed 1000 + config).  Mirrors the reference's
tests/test_dm_attn.py:60-94 (tolerances against fp32 attention, identities between the two delta modes).
"""
import math

import pytest
import torch

import delta_matching_b200 as dm
from delta_matching_b200 import _lib
from oracle import dm_oracle as O

pytestmark = pytest.mark.gpu
TOL = {"O": 8e-2, "dV": 8e-2, "dQ": 1.2e-1, "dK": 1.2e-1}     # against fp32 attention (the reference's bounds)
ORACLE_TOL = 4e-3                                             # against the CPU oracle on identical input bits
NAMES = ("O", "dQ", "dK", "dV")


def _run(q, k, v, do, mode, causal=True):
    q, k, v = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o = dm.dm_attn_func(q, k, v, causal=causal, mode=mode)
    o.backward(do.cuda())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0, "a kernel reported a bounded-wait timeout"
    return o.detach().cpu(), q.grad.cpu(), k.grad.cpu(), v.grad.cpu()


def _kv_group(t, b, g, rep=1):
    """(1, N, rep, D) slice of batch b: the rep heads of KV group g (rep = 1 for k / v themselves)."""
    return t[b:b + 1, :, g * rep:(g + 1) * rep].contiguous()


def _check_group(got, q, k, v, do, b, g, causal, mode, fp32=True, **oracle_kw):
    """One (batch, KV group) slice of a whole-configuration GPU result against the oracle (and fp32 attention) run on
    just that slice: heads of different groups and batches never interact."""
    rep = q.shape[2] // k.shape[2]
    qs, ks, vs, ds = _kv_group(q, b, g, rep), _kv_group(k, b, g), _kv_group(v, b, g), _kv_group(do, b, g, rep)
    r = O.attention_fwd_bwd(qs, ks, vs, ds, causal, mode, **oracle_kw)
    sl = {"O": _kv_group(got[0], b, g, rep), "dQ": _kv_group(got[1], b, g, rep), "dK": _kv_group(got[2], b, g),
          "dV": _kv_group(got[3], b, g)}
    for n in NAMES:
        e = O.rel(sl[n], r[n])
        assert e < ORACLE_TOL, f"{n} of batch {b}, KV group {g}: relative difference to the oracle {e:.2e}"
    if fp32:
        ref = O.fp32_reference(qs, ks, vs, ds, causal)
        for n, x in zip(NAMES, ref):
            e = O.rel(sl[n], x)
            assert math.isfinite(e) and e < TOL[n], f"{n} of batch {b}, KV group {g}: {e:.4f} against fp32 attention"


def test_config2_whole_workload_both_modes():
    """B2 N2048 H16 Hk16 D128 causal: 512 forward items and 512 pass-1 items on 148 CTAs.  Every head against the oracle
    (the build's own tile geometry), a sample against the oracle's default realization (the reference's 256-key tiles and
    rho chain) and against fp32 attention; then the stale mode on the same seed shares O and dV bit for bit."""
    B, N, H, Hk = 2, 2048, 16, 16
    q, k, v, do = O.make_inputs(B, N, H, Hk, 128, 1002)
    got = _run(q, k, v, do, "matched")
    r = O.attention_fwd_bwd(q, k, v, do, True, "matched", fwd_tile_keys=128, pv="group")
    for n, a in zip(NAMES, got):
        e = O.rel(a, r[n])
        assert e < ORACLE_TOL, f"{n}: relative difference to the oracle {e:.2e}"
        # head by head too: one wrong item out of 512 must not hide in a whole-tensor norm
        per_head = ((a.float() - r[n].float()).norm(dim=(1, 3)) / r[n].float().norm(dim=(1, 3))).max().item()
        assert per_head < 2 * ORACLE_TOL, f"{n}: worst (batch, head) differs from the oracle by {per_head:.2e}"
    for b, g in ((0, 3), (1, 12)):
        _check_group(got, q, k, v, do, b, g, True, "matched")             # default realization + fp32 attention
    stale = _run(q, k, v, do, "stale")
    assert torch.equal(got[0], stale[0]) and torch.equal(got[3], stale[3])
    assert not torch.equal(got[1], stale[1]) and not torch.equal(got[2], stale[2])
    rs = O.attention_fwd_bwd(q[:1], k[:1], v[:1], do[:1], True, "stale", fwd_tile_keys=128, pv="group")
    for n, a in zip(NAMES, stale):
        assert O.rel(a[:1], rs[n]) < ORACLE_TOL, n


@pytest.mark.parametrize("scale", [1.0, 3.0, 10.0])
def test_config3_gqa_and_logit_range(scale):
    """B4 N4096 H32 Hk8 D128 causal GQA: 4096 items.  The GPU runs all of it; two (batch, KV group) slices go to the
    oracle.  With q and k scaled by 3 and by 10 (the logit-range probe) the forward error against fp32 attention grows as
    the reference documents (about 0.12 and 0.28); the oracle still has to be matched."""
    B, N, H, Hk = 4, 4096, 32, 8
    q, k, v, do = O.make_inputs(B, N, H, Hk, 128, 1003)
    if scale != 1.0:
        q, k = (q.float() * scale).to(torch.bfloat16), (k.float() * scale).to(torch.bfloat16)
    got = _run(q, k, v, do, "matched")
    assert all(torch.isfinite(t.float()).all() for t in got)
    for b, g in ((0, 0), (3, 5)):
        _check_group(got, q, k, v, do, b, g, True, "matched", fp32=(scale == 1.0), fwd_tile_keys=128, pv="group")
    if scale != 1.0:
        qs, ks, vs, ds = _kv_group(q, 2, 7, 4), _kv_group(k, 2, 7), _kv_group(v, 2, 7), _kv_group(do, 2, 7, 4)
        ref = O.fp32_reference(qs, ks, vs, ds, True)
        e = O.rel(_kv_group(got[0], 2, 7, 4), ref[0])
        assert e < (0.2 if scale == 3.0 else 0.45), f"O at logit scale {scale}: {e:.3f} against fp32 attention"


def test_config4_head_dim_256_full_stale():
    """B2 N4096 H16 Hk4 D256, non-causal, stale delta: 1024 forward items and 2048 pass-1 items (two d halves per key
    block)."""
    B, N, H, Hk = 2, 4096, 16, 4
    q, k, v, do = O.make_inputs(B, N, H, Hk, 256, 1004)
    got = _run(q, k, v, do, "stale", causal=False)
    _check_group(got, q, k, v, do, 1, 2, False, "stale", fwd_tile_keys=128, pv="group")


def test_config5_long_context_through_the_head_split():
    """B1 N65536 H32 Hk8 D128 causal GQA through the public API (the backward runs per head group because the dS' tiles of
    all heads do not fit the workspace limit).  Checked on one KV group: O and dQ of the first 8192 rows of a query head
    (a causal row sees only earlier keys, so the oracle needs only that prefix of the codes), and dK / dV of the last
    8192 keys (only later rows reach them) with the oracle's pass 1 fed the LSE and delta of those rows."""
    B, N, H, Hk, D, g, S = 1, 65536, 32, 8, 128, 3, 8192
    rep = H // Hk
    q, k, v, do = O.make_inputs(B, N, H, Hk, D, 1005)
    got = _run(q, k, v, do, "matched")
    h = g * rep + 1
    # codes and scales of the group from whole-length tensors (the K mean runs over all 65536 keys)
    qg, dog = q[:, :, g * rep:(g + 1) * rep].transpose(1, 2), do[:, :, g * rep:(g + 1) * rep].contiguous()
    Q8, Q8s = O.quant_q(qg)
    K8, K8s, _ = O.quant_k(k[:, :, g:g + 1].transpose(1, 2))
    V8, V8s = O.quant_v(v[:, :, g:g + 1].transpose(1, 2))
    dO8, dO8s = O.quant_do(dog)
    rq, rk = O.blocks(D)

    def cut(x, xs, blk, lo, hi, heads=slice(None)):
        return x[heads, lo:hi].contiguous(), xs[heads, lo // blk:hi // blk].contiguous()
    # ---- prefix: one query head, rows and keys [0, S)
    hh = slice(1, 2)
    q8, q8s = cut(Q8, Q8s, rq, 0, S, hh)
    k8, k8s = cut(K8, K8s, rk, 0, S)
    v8, v8s = cut(V8, V8s, rk, 0, S)
    d8, d8s = cut(dO8, dO8s, rq, 0, S, hh)
    o_ref, lse = O.forward(q8, q8s, k8, k8s, v8, v8s, 1, 1, True, tile_keys=128, pv="group")
    e = O.rel(got[0][:, :S, h], o_ref[:, :, 0])
    assert e < ORACLE_TOL, f"O, first {S} rows of head {h}: {e:.2e}"
    delta = O.matched_delta(q8, q8s, k8, k8s, v8, v8s, d8, d8s, lse, 1, 1, True)
    _, _, ds8, psi = O.bwd_pass1(q8, q8s, k8, k8s, v8, v8s, d8, d8s, lse, delta, 1, 1, True)
    dq_ref = O.bwd_pass2(ds8, psi, k8, 1, 1, True).to(torch.bfloat16)
    e = O.rel(got[1][0, :S, h], dq_ref[0])
    assert e < ORACLE_TOL, f"dQ, first {S} rows of head {h}: {e:.2e}"
    del ds8, psi
    # ---- tail: the group's four query heads, rows and keys [N - S, N); LSE and delta of those rows come from the kernels
    dev = lambda *ts: [t.cuda() for t in ts]
    gQ8, gQ8s, gK8, gK8s, gV8, gV8s, gdO8, gdO8s = dev(Q8, Q8s, K8, K8s, V8, V8s, dO8, dO8s)
    _, lse_g = _lib.fwd_fp8(gQ8, gK8, gV8, gQ8s, gK8s, gV8s, 1, rep, 1, True)
    delta_g = _lib.delta_fp8(gQ8, gK8, gV8, gdO8, gQ8s, gK8s, gV8s, gdO8s, lse_g, 1, rep, 1, True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    lse_t, delta_t = lse_g[:, N - S:].cpu().contiguous(), delta_g[:, N - S:].cpu().contiguous()
    del gQ8, gK8, gV8, gdO8, lse_g, delta_g
    q8, q8s = cut(Q8, Q8s, rq, N - S, N)
    k8, k8s = cut(K8, K8s, rk, N - S, N)
    v8, v8s = cut(V8, V8s, rk, N - S, N)
    d8, d8s = cut(dO8, dO8s, rq, N - S, N)
    dKh, dVh, _, _ = O.bwd_pass1(q8, q8s, k8, k8s, v8, v8s, d8, d8s, lse_t, delta_t, rep, 1, True)
    dk_ref, dv_ref = O.gqa_fold(dKh, 1, rep, 1), O.gqa_fold(dVh, 1, rep, 1)
    for n, a, b in (("dK", got[2], dk_ref), ("dV", got[3], dv_ref)):
        e = O.rel(a[:, N - S:, g], b[:, :, 0])
        assert e < ORACLE_TOL, f"{n}, last {S} keys of KV head {g}: {e:.2e}"
    # the middle of the sequence against fp32 attention: rows [N/2, N/2 + 256) of one head need every earlier key
    r0 = N // 2
    qf = q[0, r0:r0 + 256, h].float().cuda()
    s = (qf @ k[0, :r0 + 256, g].float().cuda().T) * D ** -0.5
    s = s.masked_fill(torch.arange(r0 + 256, device="cuda")[None, :] > torch.arange(r0, r0 + 256, device="cuda")[:, None], -math.inf)
    o32 = (torch.softmax(s, -1) @ v[0, :r0 + 256, g].float().cuda()).cpu()
    assert O.rel(got[0][0, r0:r0 + 256, h], o32) < TOL["O"]
