"""CUDA quantizers against the CPU oracle: k-mean, scales and codes bit-exact (the oracle is pinned to the reference's
Triton kernels by tests/test_oracle.py), on the golden inputs, on strided packed-qkv views, at both head dims."""
import numpy as np
import pytest
import torch

from delta_matching_b200 import _lib
from oracle import dm_oracle as O
from make_quant_golden import golden_inputs

pytestmark = pytest.mark.gpu


def _eq8(a, b):
    return torch.equal(a.cpu().view(torch.uint8), b.view(torch.uint8))


def _check_all(q, k, v, dO, Oo):
    """q (B, N, H, D) etc. on the CPU (any strides); compares every producer output with the oracle bit for bit."""
    Q8, Q8s = O.quant_q(q.transpose(1, 2))
    K8, K8s, km = O.quant_k(k.transpose(1, 2))
    V8, V8s = O.quant_v(v.transpose(1, 2))
    dO8, dO8s = O.quant_do(dO)
    dlt = O.stale_delta(dO, Oo)
    qd, kd, vd, dod, od = (t.cuda() for t in (q, k, v, dO, Oo))
    if q.stride() != q.contiguous().stride():      # keep the strided view on the device too
        pass
    gkm = _lib.kmean(kd)
    assert torch.equal(gkm.cpu(), km), "k-mean differs"
    for name, (gc, gs), (c, s) in (("q", _lib.quant(0, qd), (Q8, Q8s)), ("k", _lib.quant(1, kd, gkm), (K8, K8s)),
                                   ("v", _lib.quant(2, vd), (V8, V8s))):
        assert torch.equal(gs.cpu(), s), f"{name} scales differ"
        assert _eq8(gc, c), f"{name} codes differ"
    gc, gs, gd = _lib.quant_do(dod, od)
    assert torch.equal(gs.cpu(), dO8s) and _eq8(gc, dO8) and torch.equal(gd.cpu(), dlt)
    gc2, gs2, none = _lib.quant_do(dod)
    assert none is None and torch.equal(gs2, gs) and torch.equal(gc2.view(torch.uint8), gc.view(torch.uint8))


@pytest.mark.parametrize("D", [128, 256])
def test_golden_inputs(D):
    q, k, v, dO, Oo = golden_inputs(D)
    _check_all(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dO, Oo)


@pytest.mark.parametrize("B,N,H,Hk,D", [(1, 256, 2, 2, 128), (2, 512, 8, 2, 128), (2, 384, 4, 1, 256)])
def test_random_and_packed_views(B, N, H, Hk, D):
    g = torch.Generator("cpu").manual_seed(11)
    qkv = torch.randn(B, N, H + 2 * Hk, D, generator=g).to(torch.bfloat16)
    q, k, v = qkv.split([H, Hk, Hk], dim=2)
    dO = (torch.randn(B, N, H, D, generator=g) * 0.01).to(torch.bfloat16)
    Oo = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    # device tensors keep the packed strides
    qkv_d = qkv.cuda()
    qd, kd, vd = qkv_d.split([H, Hk, Hk], dim=2)
    Q8, Q8s = O.quant_q(q.transpose(1, 2))
    K8, K8s, km = O.quant_k(k.transpose(1, 2))
    V8, V8s = O.quant_v(v.transpose(1, 2))
    gkm = _lib.kmean(kd)
    assert torch.equal(gkm.cpu(), km)
    for (gc, gs), (c, s) in ((_lib.quant(0, qd), (Q8, Q8s)), (_lib.quant(1, kd, gkm), (K8, K8s)), (_lib.quant(2, vd), (V8, V8s))):
        assert torch.equal(gs.cpu(), s) and _eq8(gc, c)
    _check_all(q.contiguous(), k.contiguous(), v.contiguous(), dO, Oo)


def test_expanded_grad_and_saturation():
    """A stride-0 expanded dO (the gradient of o.sum()) is made unit-stride by the wrapper; an all-equal block saturates
    every code at +-448 / scale."""
    B, N, H, D = 1, 256, 2, 128
    dO = torch.ones(1, 1, 1, 1, dtype=torch.bfloat16).expand(B, N, H, D)
    gc, gs, _ = _lib.quant_do(dO.cuda())
    c, s = O.quant_do(dO.contiguous())
    assert torch.equal(gs.cpu(), s) and _eq8(gc, c)
    assert (gc.float() == 448.0).all()


def _special_blocks(rows, D, seed):
    """One block of `rows` rows per case: signed zeros, bf16 subnormals, a NaN, an infinity, both, all zero, huge, tiny."""
    g = torch.Generator("cpu").manual_seed(seed)
    cases = []
    for kind in range(8):
        x = torch.randn(rows, D, generator=g)
        if kind == 0:
            x[::3] = 0.0
            x[1::7] = -0.0
        elif kind == 1:
            x[::2] = x[::2] * 1e-39                       # bf16 subnormals beside ordinary values
        elif kind == 2:
            x[5, 7] = float("nan")
        elif kind == 3:
            x[9, 1] = float("inf")
        elif kind == 4:
            x[3, 3] = float("-inf")
            x[4, 4] = float("nan")
        elif kind == 5:
            x.zero_()
            x[::2] = -0.0
        elif kind == 6:
            x = x * 1e37
        else:
            x = x * 1e-25
        cases.append(x)
    return torch.cat(cases).to(torch.bfloat16)


def _expected_codes(v, rows, mul_inv):
    """What the quantizers define for non-finite data: the block maximum skips a NaN and is won by an infinity, and a NaN
    quotient (a NaN element, or infinity over infinity) becomes the code of -448."""
    n_blk = v.shape[0] // rows
    vb = v.view(n_blk, -1)
    amax = torch.where(vb.isnan(), torch.zeros_like(vb), vb.abs()).amax(dim=1)
    base = torch.maximum(amax, torch.tensor(1e-30, dtype=torch.float32))
    s = base * (torch.tensor(1.0) / torch.tensor(448.0)) if mul_inv else base / torch.tensor(448.0)
    q = vb / s[:, None]
    q = torch.where(q.isnan(), torch.full_like(q, -448.0), q)
    return O.to_e4m3(q).view(v.shape), s


@pytest.mark.parametrize("D", [128, 256])
def test_signed_zeros_subnormals_and_non_finite_blocks(D):
    rq, rkv = (128, 64) if D == 128 else (64, 32)
    for mode, rows in ((0, rq), (2, rkv), (3, rq)):
        x = _special_blocks(rows, D, 40 + mode)                       # [8 * rows, D]
        n = x.shape[0]
        n_pad = -(-n // 256) * 256                                   # the sequence length the shape check wants
        x = torch.cat([x, torch.ones(n_pad - n, D, dtype=torch.bfloat16)])
        v = x.float() * torch.tensor(D ** -0.5, dtype=torch.float32) if mode == 0 else x.float()
        want_c, want_s = _expected_codes(v, rows, mul_inv=(mode == 3))
        xd = x.view(1, n_pad, 1, D).cuda()
        if mode == 3:
            gc, gs, _ = _lib.quant_do(xd)
        else:
            gc, gs = _lib.quant(mode, xd)
        assert torch.equal(gs.cpu().view(-1), want_s), f"mode {mode}: scales differ"
        got = gc.cpu().view(torch.uint8).view(n_pad, D)
        bad = (got != want_c.view(torch.uint8)).nonzero()
        assert bad.numel() == 0, f"mode {mode}: codes differ first at {bad[0].tolist()} (case {int(bad[0][0]) // rows})"


def test_gqa_fold():
    g = torch.Generator("cpu").manual_seed(5)
    x = torch.randn(2, 256, 8, 128, generator=g).to(torch.bfloat16)
    out = _lib.gqa_fold(x.cuda(), 2).cpu()
    ref = x.view(2, 256, 2, 4, 128).float().sum(3).to(torch.bfloat16)
    assert (out.float() - ref.float()).abs().max() <= 2 * ref.float().abs().max() * 2 ** -8
    seq = x.view(2, 256, 2, 4, 128).float()
    acc = ((seq[:, :, :, 0] + seq[:, :, :, 1]) + seq[:, :, :, 2]) + seq[:, :, :, 3]
    assert torch.equal(out, acc.to(torch.bfloat16))


@pytest.mark.parametrize("D,N", [(128, 512), (256, 256)])
def test_fused_producers_equal_the_separate_ones(D, N):
    """The composite forward quantizes Q and V and sums K's chunks in one launch: same codes, scales and K mean as the
    separate entry points."""
    from delta_matching_b200 import _lib
    g = torch.Generator().manual_seed(3)
    q = torch.randn(2, N, 4, D, generator=g).to(torch.bfloat16).cuda()
    k = (torch.randn(2, N, 2, D, generator=g) + 0.5).to(torch.bfloat16).cuda()
    v = torch.randn(2, N, 2, D, generator=g).to(torch.bfloat16).cuda()
    _, _, Q8, Q8s, K8, K8s, V8, V8s = _lib.attn_forward(q, k, v, False)
    km = _lib.kmean(k)
    for got, want in zip((Q8, Q8s, K8, K8s, V8, V8s), (*_lib.quant(0, q), *_lib.quant(1, k, km), *_lib.quant(2, v))):
        assert torch.equal(got.view(torch.uint8) if got.dtype != torch.float32 else got,
                           want.view(torch.uint8) if want.dtype != torch.float32 else want)
