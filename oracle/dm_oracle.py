"""CPU oracle for the Delta-Matching fp8 attention path (TEST INFRASTRUCTURE, not product code).

A PyTorch-on-CPU restatement of the reference algorithm, function by function.  Only tests, the smoke check and
the benchmark's cpu-baseline leg may import this module; the product path never does.

Pinning status.  The quantizers (k-mean, Q/K/V/dO scales and codes) are pinned bit-for-bit against the reference's own
Triton kernels executed by Triton's CPU interpreter (fixtures under tests/golden, generator committed beside them).
The attention passes (forward, matched delta, pass 1, pass 2) have no golden vectors in the reference and its CUDA
kernels cannot be built or run without Hopper hardware and an un-vendored FlashAttention-3 tree, so for O, LSE, delta,
dQ, dK, dV this oracle is "parity unpinned" at bit level: it is checked against the reference's published contract
instead (relative error to fp32 attention below 0.08 / 0.12, rowsum(dS) = 0 to fp32 round-off in the matched mode,
O and dV identical between the two delta modes).

Reference files restated here (paths inside the reference project):
  quantizers        delta_matching/quant.py:17-86, delta_matching/producers.py:40-65,235-297, delta_matching/constants.py:5-8
  forward           csrc/softmax_fq8f.h:185-339, csrc/mainloop_fwd_sm90_fp8f.hpp:1341-1418,1496-1542,1666-1708
  matched delta     csrc/fp11_delta_v6.h:338-376,458-462
  pass 1            csrc/mainloop_bwd_sm90_fp8r.hpp:651-667,695-931,945-952
  pass 2            csrc/fq8_dq_pass2_hd128.h:209-215,283-395
  GQA fold          delta_matching/attn.py:111-118
  D=256 geometry    csrc/mainloop_bwd_sm90_fp8v10.hpp:1674-1761, csrc/fq8_dq_pass2.h:95-125,188

Arithmetic taken from the un-vendored FlashAttention-3 dependency (commit 0251105a2fb19d2957484b7f023cd8c115286ced) is
restated from its published semantics: causal mask "key j visible iff j <= i" for self-attention, fp32 -> e4m3
round-to-nearest-even saturating casts, fp32 -> bf16 round-to-nearest-even output stores.
"""
from __future__ import annotations

import math

import torch

E4M3 = torch.float8_e4m3fn
E4M3_MAX = 448.0
TINY = 1e-30
LOG2E = float(torch.tensor(math.log2(math.e), dtype=torch.float32))
LOG2_448 = float(torch.tensor(8.8073549220576042, dtype=torch.float32))
PHAT_FLOOR_B = 12.0          # csrc/softmax_fq8f.h:147
MO_E = 8.0                   # the 2^8 offset of P-hat in the backward (mainloop_bwd_sm90_fp8r.hpp:664)
F32 = torch.float32


def blocks(D: int):
    """Rows per Q/dO scale and keys per K/V scale (delta_matching/core.py:26-29)."""
    return (64, 32) if D >= 256 else (128, 64)


def _f32(x):
    return torch.tensor(x, dtype=F32)


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """fp32 -> e4m3 round-to-nearest-even, saturating at +-448 (cvt.rn.satfinite semantics)."""
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(E4M3)


# ----------------------------------------------------------------------------------------------------------------------
# quantizers (bit-exact targets)
# ----------------------------------------------------------------------------------------------------------------------
def kmean(k_bh: torch.Tensor) -> torch.Tensor:
    """k_bh [BHk, N, D] bf16 -> [BHk, D] fp32.  quant.py:17-29: 64 rows at a time, the 64 rows of a chunk added in
    ascending row order (what the reference's tl.sum(axis=0) does under Triton's interpreter; the build defines this
    order for its CUDA kernel too), chunk sums folded serially, one IEEE division by N."""
    BH, N, D = k_bh.shape
    x = k_bh.to(F32).contiguous().view(BH, N // 64, 64, D)
    s = x[:, :, 0].clone()
    for r in range(1, 64):
        s = s + x[:, :, r]
    acc = torch.zeros(BH, D, dtype=F32)
    for j in range(N // 64):
        acc = acc + s[:, j]
    return acc / _f32(float(N))


def quant_blocks(x: torch.Tensor, blk: int, mul_inv: bool = False):
    """x [BH, N, D] fp32 -> (codes e4m3 [BH, N, D], scales fp32 [BH, N // blk]).  quant.py:59-67 (scale by division)
    or producers.py:267-268 (dO: scale by multiplication with fp32(1/448))."""
    BH, N, D = x.shape
    xb = x.contiguous().view(BH, N // blk, blk * D)
    amax = xb.abs().amax(dim=-1)
    base = torch.maximum(amax, _f32(TINY))
    if mul_inv:
        s = base * (_f32(1.0) / _f32(E4M3_MAX))
    else:
        s = base / _f32(E4M3_MAX)
    q = xb / s[..., None]
    return to_e4m3(q).view(BH, N, D), s


def quant_q(q_bhnd: torch.Tensor):
    """q (B, H, N, D) bf16 -> Q8 [BH, N, D], Q8s [BH, N/rq]; x = float(q) * fp32(D^-0.5) first (quant.py:52-53)."""
    B, H, N, D = q_bhnd.shape
    x = q_bhnd.reshape(B * H, N, D).to(F32) * _f32(D ** -0.5)
    return quant_blocks(x, blocks(D)[0])


def quant_k(k_bhnd: torch.Tensor):
    """k (B, Hk, N, D) bf16 -> K8, K8s, km; x = float(k) - km (quant.py:54-56)."""
    B, Hk, N, D = k_bhnd.shape
    kc = k_bhnd.reshape(B * Hk, N, D)
    km = kmean(kc)
    x = kc.to(F32) - km[:, None, :]
    c, s = quant_blocks(x, blocks(D)[1])
    return c, s, km


def quant_v(v_bhnd: torch.Tensor):
    B, Hk, N, D = v_bhnd.shape
    return quant_blocks(v_bhnd.reshape(B * Hk, N, D).to(F32), blocks(D)[1])


def stale_delta(dO_bnhd: torch.Tensor, o_bnhd: torch.Tensor) -> torch.Tensor:
    """delta[bh, n] = sum_d float(dO) * float(O) from the raw bf16 tensors (producers.py:289-297).  The summation order
    over d is implementation-defined in the reference (a Triton reduction); the build defines it as: products rounded
    to fp32, four consecutive d added in ascending order per lane of 32 lanes (D=128; eight at D=256), then the
    xor-butterfly tree over the 32 lanes (offsets 16, 8, 4, 2, 1)."""
    B, N, H, D = dO_bnhd.shape
    p = dO_bnhd.to(F32) * o_bnhd.to(F32)
    per = D // 32
    p = p.view(B, N, H, 32, per)
    v = p[..., 0].clone()
    for i in range(1, per):
        v = v + p[..., i]
    for off in (16, 8, 4, 2, 1):
        v = v[..., :off] + v[..., off:2 * off]
    return v[..., 0].permute(0, 2, 1).reshape(B * H, N).contiguous()


def quant_do(dO_bnhd: torch.Tensor):
    """dO (B, N, H, D) bf16 -> dO8 [BH, N, D], dO8s [BH, N/rq] (producers.py:235-288)."""
    B, N, H, D = dO_bnhd.shape
    x = dO_bnhd.permute(0, 2, 1, 3).reshape(B * H, N, D).to(F32)
    return quant_blocks(x, blocks(D)[0], mul_inv=True)


# ----------------------------------------------------------------------------------------------------------------------
# attention passes (D = 128 and D = 256 geometry from `blocks`)
# ----------------------------------------------------------------------------------------------------------------------
def _mm(a, b, acc):
    """Batched a @ b^T on exact code values with the chosen accumulate dtype (fp32 = the timed CPU path, fp64 = exact
    for e4m3 operands)."""
    return torch.matmul(a.to(acc), b.to(acc).transpose(-1, -2)).to(F32) if acc != F32 else torch.matmul(a, b.transpose(-1, -2))


def _kv_index(BH, H, Hk):
    """query head bh -> kv head index (consecutive query heads share a KV head; mainloop_fwd_sm90_fp8f.hpp:1177)."""
    bh = torch.arange(BH)
    return (bh // H) * Hk + (bh % H) // (H // Hk)


def forward(Q8, Q8s, K8, K8s, V8, V8s, H, Hk, causal=True, tile_keys=None, pv="chain", acc=F32):
    """The faithful forward.  Codes [BH, N, D] / [BHk, N, D] e4m3, scales fp32.  Returns O (B, N, H, D) bf16 and
    LSE [BH, N] fp32 (natural log).  tile_keys = keys per online-softmax step (reference: 256 at D=128, 128 at D=256);
    pv = "chain" (the reference's zero-initialised tile temp with the rho chain and one promote per tile,
    mainloop_fwd_sm90_fp8f.hpp:1410-1418,1507-1515) or "group" (O += D_g * w_g per key group: the same sum in another
    rounding order, softmax_fq8f.h kGroupsPerPromote == 1 form)."""
    BH, N, D = Q8.shape
    rq, rk = blocks(D)
    if tile_keys is None:
        tile_keys = 256 if D == 128 else 128
    BM = 128
    kv = _kv_index(BH, H, Hk)
    Qf, Kf, Vf = Q8.to(F32), K8.to(F32)[kv], V8.to(F32)[kv]
    Ks, Vs = K8s[kv], V8s[kv]
    l2 = _f32(LOG2E)
    O = torch.empty(BH, N, D, dtype=F32)
    LSE = torch.empty(BH, N, dtype=F32)
    gpt = tile_keys // rk
    for I in range(N // BM):
        r0 = I * BM
        rows = torch.arange(r0, r0 + BM)
        qs = Q8s[:, r0 // rq:(r0 + BM) // rq].repeat_interleave(rq, dim=1)              # [BH, 128] per-row q scale
        m = torch.full((BH, BM), -math.inf, dtype=F32)
        l = torch.zeros(BH, BM, dtype=F32)
        Oacc = torch.zeros(BH, BM, D, dtype=F32)
        t_hi = ((r0 + BM - 1) // tile_keys) if causal else (N // tile_keys - 1)
        for T in range(t_hi, -1, -1):
            S, gm = [], []
            for g in range(gpt):
                k0 = T * tile_keys + g * rk
                s = _mm(Qf[:, r0:r0 + BM], Kf[:, k0:k0 + rk], acc) * (qs * Ks[:, k0 // rk, None])[..., None]
                if causal:
                    keys = torch.arange(k0, k0 + rk)
                    s = s.masked_fill(keys[None, None, :] > rows[None, :, None], -math.inf)
                S.append(s)
                gm.append(s.amax(dim=-1))
            tile_max = torch.stack(gm, 0).amax(dim=0)
            m_new = torch.maximum(m, tile_max)
            m_cur = torch.where(m_new == -math.inf, torch.zeros_like(m_new), m_new)
            alpha = torch.exp2((m - m_cur) * l2)
            alpha = torch.where(torch.isnan(alpha), torch.zeros_like(alpha), alpha)
            l = l * alpha
            Oacc = Oacc * alpha[..., None]
            ml2 = m_cur * l2
            accl = torch.zeros_like(l)
            ms_l, C_l = [], []
            for g in range(gpt):
                ms = torch.maximum(gm[g] * l2, ml2 - _f32(PHAT_FLOOR_B)) - _f32(LOG2_448)
                p = torch.exp2(S[g] * l2 - ms[..., None])
                accl = accl + torch.exp2(ms - ml2) * p.sum(dim=-1)
                ms_l.append(ms)
                C_l.append(to_e4m3(p).to(F32))
            l = l + accl
            if pv == "group":
                for g in range(gpt):
                    k0 = T * tile_keys + g * rk
                    Dg = _mm(C_l[g], Vf[:, k0:k0 + rk].transpose(-1, -2), acc)
                    w = Vs[:, k0 // rk] [:, None] * torch.exp2(ms_l[g] - ml2)
                    Oacc = Oacc + Dg * w[..., None]
            else:
                Tt = torch.zeros_like(Oacc)
                for g in range(gpt):
                    k0 = T * tile_keys + g * rk
                    if g > 0:
                        vr = Vs[:, (k0 - rk) // rk] / Vs[:, k0 // rk]
                        rho = (vr[:, None] * torch.exp2(ms_l[g - 1] - ms_l[g])).clamp(1e-30, 1e30)
                        Tt = Tt * rho[..., None]
                    Tt = Tt + _mm(C_l[g], Vf[:, k0:k0 + rk].transpose(-1, -2), acc)
                kl = T * tile_keys + (gpt - 1) * rk
                w = Vs[:, kl // rk][:, None] * torch.exp2(ms_l[-1] - ml2)
                Oacc = Oacc + Tt * w[..., None]
            m = m_new
        dead = (l == 0) | torch.isnan(l)
        inv = torch.where(dead, torch.zeros_like(l), 1.0 / l)
        O[:, r0:r0 + BM] = Oacc * inv[..., None]
        LSE[:, r0:r0 + BM] = torch.where(dead, torch.full_like(l, -math.inf), m + torch.log(l))
    B = BH // H
    return O.view(B, H, N, D).permute(0, 2, 1, 3).to(torch.bfloat16).contiguous(), LSE


def _phat(Sraw, dsc, lse2):
    """P-hat = 2^(min(S_raw * dsc - lse*log2e + 8, 12)) (mainloop_bwd_sm90_fp8r.hpp:746, fp11_delta_v6.h:356)."""
    return torch.exp2(torch.minimum(Sraw * dsc - lse2 + _f32(MO_E), _f32(MO_E + 4.0)))


def matched_delta(Q8, Q8s, K8, K8s, V8, V8s, dO8, dO8s, LSE, H, Hk, causal=True, acc=F32):
    """Pass 0: delta[bh, n] = 2^-8 * sum_keys P-hat * dP in true dP units, 64-key groups ascending, the per-group
    fp32 partials folded in fp64 and rounded once (fp11_delta_v6.h:338-376,458-462).  D=128 geometry."""
    BH, N, D = Q8.shape
    rq, rk = blocks(D)
    kv = _kv_index(BH, H, Hk)
    Qf, Kf, Vf, dOf = Q8.to(F32), K8.to(F32)[kv], V8.to(F32)[kv], dO8.to(F32)
    Ks, Vs = K8s[kv], V8s[kv]
    l2 = _f32(LOG2E)
    lse2 = LSE * l2
    out = torch.empty(BH, N, dtype=F32)
    BM = 128
    for I in range(N // BM):
        r0 = I * BM
        rows = torch.arange(r0, r0 + BM)
        qs = Q8s[:, r0 // rq:(r0 + BM) // rq].repeat_interleave(rq, dim=1)
        dos = dO8s[:, r0 // rq:(r0 + BM) // rq].repeat_interleave(rq, dim=1)
        accd = torch.zeros(BH, BM, dtype=torch.float64)
        g_hi = ((r0 + BM - 1) // rk) if causal else (N // rk - 1)
        for g in range(g_hi + 1):
            k0 = g * rk
            Sraw = _mm(Qf[:, r0:r0 + BM], Kf[:, k0:k0 + rk], acc)
            dsc = (qs * Ks[:, g, None] * l2)[..., None]
            P = _phat(Sraw, dsc, lse2[:, r0:r0 + BM, None])
            if causal:
                keys = torch.arange(k0, k0 + rk)
                P = P.masked_fill(keys[None, None, :] > rows[None, :, None], 0.0)
            dP = _mm(dOf[:, r0:r0 + BM], Vf[:, k0:k0 + rk], acc) * (dos * Vs[:, g, None])[..., None]
            pd = P * dP
            for h0 in range(0, rk, 32):            # 32-key halves, each an fp32 partial folded into fp64
                a = pd[..., h0:h0 + 32].sum(dim=-1) * _f32(1.0 / 256.0)
                accd += a.to(torch.float64)
        out[:, r0:r0 + BM] = accd.to(F32)
    return out


def bwd_pass1(Q8, Q8s, K8, K8s, V8, V8s, dO8, dO8s, LSE, delta, H, Hk, causal=True, acc=F32, debug=False):
    """Pass 1 (mainloop_bwd_sm90_fp8r.hpp:695-952, D=128 geometry; D=256 uses 64-key blocks with 32-key scale groups).
    Returns dK, dV per QUERY head [BH, N, D] fp32 (before the bf16 store), dS' codes [BH, N/64, N/kb, 64, kb] e4m3,
    psi [BH, N/64, N/kb] fp32, and with debug the row sums / abs row sums of P-hat*(dP - delta) in true units."""
    BH, N, D = Q8.shape
    rq, rk = blocks(D)
    KB = 128 if D == 128 else 64          # keys per CTA / dS' tile width
    BM = 64
    kv = _kv_index(BH, H, Hk)
    Qf, Kf, Vf, dOf = Q8.to(F32), K8.to(F32)[kv], V8.to(F32)[kv], dO8.to(F32)
    Ks, Vs = K8s[kv], V8s[kv]
    l2 = _f32(LOG2E)
    lse2 = LSE * l2
    nbm, nbn = N // BM, N // KB
    dS8 = torch.zeros(BH, nbm, nbn, BM, KB, dtype=E4M3)
    psi_out = torch.zeros(BH, nbm, nbn, dtype=F32)
    dK = torch.zeros(BH, N, D, dtype=F32)
    dV = torch.zeros(BH, N, D, dtype=F32)
    rows_sum = torch.zeros(BH, N, dtype=torch.float64) if debug else None
    rows_abs = torch.zeros(BH, N, dtype=torch.float64) if debug else None
    gpb = KB // rk
    for J in range(nbn):
        k0 = J * KB
        ksg = Ks[:, k0 // rk:(k0 + KB) // rk].repeat_interleave(rk, dim=1)            # [BH, KB] per-key scales
        vsg = Vs[:, k0 // rk:(k0 + KB) // rk].repeat_interleave(rk, dim=1)
        keys = torch.arange(k0, k0 + KB)
        g_max = torch.zeros(BH, dtype=F32)
        dKacc = torch.zeros(BH, KB, D, dtype=F32)
        dVacc = torch.zeros(BH, KB, D, dtype=F32)
        m_lo = (k0 // BM) if causal else 0
        for mb in range(m_lo, nbm):
            r0 = mb * BM
            rows = torch.arange(r0, r0 + BM)
            qs = Q8s[:, r0 // rq]
            dos = dO8s[:, r0 // rq]
            Sraw = _mm(Qf[:, r0:r0 + BM], Kf[:, k0:k0 + KB], acc)
            dsc = (qs[:, None] * ksg * l2)[:, None, :]
            P = _phat(Sraw, dsc, lse2[:, r0:r0 + BM, None])
            if causal:
                P = P.masked_fill(keys[None, None, :] > rows[None, :, None], 0.0)
            dPr = _mm(dOf[:, r0:r0 + BM], Vf[:, k0:k0 + KB], acc)
            dlt_k = delta[:, r0:r0 + BM, None] * ksg[:, None, :]
            dS = P * (dPr * (dos[:, None] * vsg * ksg)[:, None, :] - dlt_k)
            if debug:
                t = (P * (dPr * (dos[:, None] * vsg)[:, None, :] - delta[:, r0:r0 + BM, None])).to(torch.float64) / 256.0
                rows_sum[:, r0:r0 + BM] += t.sum(-1)
                rows_abs[:, r0:r0 + BM] += t.abs().sum(-1)
            amax = dS.abs().amax(dim=(-1, -2))
            tile_zero = amax * _f32(1.0 / 448.0) < _f32(TINY)
            psi_raw = torch.maximum(amax * _f32(1.0 / 448.0), _f32(TINY))
            psi = torch.maximum(psi_raw, g_max * _f32(256.0 * 1e-8) / qs)
            psi_inv = torch.where(tile_zero, torch.zeros_like(psi), 1.0 / psi)
            psi_out[:, mb, J] = torch.where(tile_zero, torch.zeros_like(psi), psi)
            P8 = to_e4m3(P).to(F32)
            dS8t = to_e4m3(dS * psi_inv[:, None, None])
            dS8[:, mb, J] = dS8t
            f = dos * _f32(1.0 / 256.0)
            dVacc = dVacc + _mm(P8.transpose(-1, -2), dOf[:, r0:r0 + BM].transpose(-1, -2), acc) * f[:, None, None]
            g_cur = torch.where(tile_zero, torch.zeros_like(psi), psi * _f32(1.0 / 256.0) * qs)
            dKacc = dKacc + _mm(dS8t.to(F32).transpose(-1, -2), Qf[:, r0:r0 + BM].transpose(-1, -2), acc) * g_cur[:, None, None]
            g_max = torch.maximum(g_max, g_cur)
        dK[:, k0:k0 + KB] = dKacc * (1.0 / ksg)[..., None]
        dV[:, k0:k0 + KB] = dVacc
    if debug:
        return dK, dV, dS8, psi_out, rows_sum, rows_abs
    return dK, dV, dS8, psi_out


def bwd_pass2(dS8, psi, K8, H, Hk, causal=True, acc=F32):
    """Pass 2: dQ[bh, rows] = D^-0.5 / 256 * sum_tiles psi * (dS'8 @ K8), key tiles ascending, tiles with psi == 0 or
    psi < 1e-8 * running psi max skipped (fq8_dq_pass2_hd128.h:286-395).  Returns [BH, N, D] fp32 before the bf16 store.
    The reference folds psi through a 4-tile rescaled window; the sum is the same, the rounding order differs."""
    BH, nbm, nbn, BM, KB = dS8.shape
    N = nbm * BM
    D = K8.shape[-1]
    kv = _kv_index(BH, H, Hk)
    Kf = K8.to(F32)[kv]
    dQ = torch.zeros(BH, N, D, dtype=F32)
    for mb in range(nbm):
        nb_end = (((mb + 1) * BM - 1) // KB + 1) if causal else nbn
        accq = torch.zeros(BH, BM, D, dtype=F32)
        psi_max = torch.zeros(BH, dtype=F32)
        for nb in range(nb_end):
            pc = psi[:, mb, nb]
            take = (pc != 0) & ~(pc < psi_max * _f32(1e-8))
            t = torch.matmul(dS8[:, mb, nb].to(acc), Kf[:, nb * KB:(nb + 1) * KB].to(acc)).to(F32)
            accq = accq + torch.where(take, pc, torch.zeros_like(pc))[:, None, None] * t
            psi_max = torch.where(take, torch.maximum(psi_max, pc), psi_max)
        dQ[:, mb * BM:(mb + 1) * BM] = accq * _f32((D ** -0.5) / 256.0)
    return dQ


def gqa_fold(x_bh_nd: torch.Tensor, B, H, Hk):
    """[B*H, N, D] fp32 per-query-head grads -> (B, N, Hk, D) bf16: bf16 store per query head, then the sum over the
    rep query heads of a KV head in fp32, one bf16 rounding (attn.py:111-118)."""
    BH, N, D = x_bh_nd.shape
    xb = x_bh_nd.to(torch.bfloat16).view(B, Hk, H // Hk, N, D)
    if H == Hk:
        return xb[:, :, 0].permute(0, 2, 1, 3).contiguous()
    return xb.to(F32).sum(2).to(torch.bfloat16).permute(0, 2, 1, 3).contiguous()


def attention_fwd_bwd(q, k, v, dO, causal=True, mode="matched", acc=F32, fwd_tile_keys=None, pv="chain", debug=False):
    """q (B, N, H, D), k / v (B, N, Hk, D), dO (B, N, H, D) bf16 on CPU -> dict with O, dQ, dK, dV (flash layout, bf16)
    plus LSE, delta and, with debug, the pass-1 row-sum residuals and every intermediate."""
    B, N, H, D = q.shape
    Hk = k.shape[2]
    Q8, Q8s = quant_q(q.transpose(1, 2))
    K8, K8s, km = quant_k(k.transpose(1, 2))
    V8, V8s = quant_v(v.transpose(1, 2))
    O, LSE = forward(Q8, Q8s, K8, K8s, V8, V8s, H, Hk, causal, fwd_tile_keys, pv, acc)
    dO8, dO8s = quant_do(dO)
    if mode == "matched":
        delta = matched_delta(Q8, Q8s, K8, K8s, V8, V8s, dO8, dO8s, LSE, H, Hk, causal, acc)
    else:
        delta = stale_delta(dO, O)
    r = bwd_pass1(Q8, Q8s, K8, K8s, V8, V8s, dO8, dO8s, LSE, delta, H, Hk, causal, acc, debug)
    dKh, dVh, dS8, psi = r[:4]
    dQh = bwd_pass2(dS8, psi, K8, H, Hk, causal, acc)
    out = {"O": O, "LSE": LSE, "delta": delta,
           "dQ": dQh.to(torch.bfloat16).view(B, H, N, D).permute(0, 2, 1, 3).contiguous(),
           "dK": gqa_fold(dKh, B, H, Hk), "dV": gqa_fold(dVh, B, H, Hk)}
    if debug:
        out.update(rows_sum=r[4], rows_abs=r[5], Q8=Q8, Q8s=Q8s, K8=K8, K8s=K8s, km=km, V8=V8, V8s=V8s, dO8=dO8, dO8s=dO8s,
                   dS8=dS8, psi=psi, dKh=dKh, dVh=dVh, dQh=dQh)
    return out


def fp32_reference(q, k, v, dO, causal=True):
    """Plain fp32 attention with autograd on the same bf16 inputs (the reference tests' `_reference`,
    tests/test_dm_attn.py:35-50); returns O, dQ, dK, dV in the flash layout, fp32."""
    B, N, H, D = q.shape
    Hk = k.shape[2]
    qf = q.float().transpose(1, 2).requires_grad_(True)
    kf = k.float().transpose(1, 2).requires_grad_(True)
    vf = v.float().transpose(1, 2).requires_grad_(True)
    kr = kf.repeat_interleave(H // Hk, dim=1)
    vr = vf.repeat_interleave(H // Hk, dim=1)
    s = (qf @ kr.transpose(-1, -2)) * (D ** -0.5)
    if causal:
        s = s.masked_fill(~torch.ones(N, N, dtype=torch.bool).tril(), float("-inf"))
    o = torch.softmax(s, dim=-1) @ vr
    o.backward(dO.float().transpose(1, 2))
    return o.detach().transpose(1, 2), qf.grad.transpose(1, 2), kf.grad.transpose(1, 2), vf.grad.transpose(1, 2)


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


def make_inputs(B, N, H, Hk, D, seed):
    """The synthetic workload: CPU generator, q, k, v, dO drawn in that order as fp32 N(0,1) -> bf16."""
    g = torch.Generator("cpu").manual_seed(seed)
    q = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, N, Hk, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, N, Hk, D, generator=g).to(torch.bfloat16)
    dO = torch.randn(B, N, H, D, generator=g).to(torch.bfloat16)
    return q, k, v, dO
