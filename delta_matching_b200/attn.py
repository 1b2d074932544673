"""The API route: dm_attn_func_bhnd(q, k, v, causal, softmax_scale, delta_mode) on (B, H, N, D) inputs, returning
(B, N, H, D).  Forward: the CUDA quantizers (codes and scales; no transposed twins exist in this build), then the fwd_fp8
op.  Backward: the dO quantizer (with the stale delta rowsum(dO * O) only in the stale mode; the matched mode never reads
O), the matched delta from pass 0, then pass 1 and pass 2, split per head group at long context (split.py), then the GQA
fold.  Saved for the backward: the fp8 codes, their scales, O and the LSE.  Mirrors delta_matching/attn.py:37-127 of the
reference."""
from __future__ import annotations

import torch

from . import ops
from .core import _check_inputs


class _DMAttn(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, causal, delta_mode):
        B, H, N, D = q.shape
        Hk = k.shape[1]
        fwd = ops.attn_fwd if torch.compiler.is_compiling() else ops.attn_fwd_eager
        O, Lse, Q8, Q8s, K8, K8s, V8, V8s = fwd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal)
        ctx.save_for_backward(Q8, Q8s, K8, K8s, V8, V8s, O, Lse)
        ctx.dims = (B, H, Hk, N, D)
        ctx.causal = causal
        ctx.delta_mode = delta_mode
        return O

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dO):
        B, H, Hk, N, D = ctx.dims
        Q8, Q8s, K8, K8s, V8, V8s, O, Lse = ctx.saved_tensors
        if dO.stride(-1) != 1:          # e.g. the expanded gradient of o.sum(): the quantizer reads rows with a unit lane stride
            dO = dO.contiguous()
        bwd = ops.attn_bwd if torch.compiler.is_compiling() else ops.attn_bwd_eager
        dq, dk, dv = bwd(dO, O, Lse, Q8, Q8s, K8, K8s, V8, V8s, B, H, Hk, ctx.causal, ctx.delta_mode == "matched")
        return dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3), None, None


def dm_attn_func_bhnd(q, k, v, causal=True, softmax_scale=None, delta_mode="stale"):
    """Attention on (B, H, N, D) inputs: q (B, H, N, D), k / v (B, Hk, N, D) bf16 on CUDA (any strides; H % Hk == 0) ->
    O (B, N, H, D) bf16 contiguous (the kernel's native output layout).  delta_mode: "stale" (delta = rowsum(dO * O)) or
    "matched" (the Delta-Matching backward; needs causal=True).  Input errors raise ValueError / TypeError /
    NotImplementedError (core._check_inputs)."""
    _check_inputs(q, k, v, causal, softmax_scale, delta_mode)
    return _DMAttn.apply(q, k, v, causal, delta_mode)


class _DMAttnPlain(torch.autograd.Function):
    """The plain route: the same kernels driven op by op without the head-group split, always taking the stale delta in
    the dO quantizer pass and replacing it by the pass-0 delta in the matched mode (the shape of the reference's
    core._DMAttnPlain, delta_matching/core.py:178-261).  Bitwise the API route; kept as a cross-check of it."""

    @staticmethod
    def forward(ctx, q, k, v, causal, delta_mode):
        from . import _lib
        B, H, N, D = q.shape
        Hk = k.shape[1]
        qf, kf, vf = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        Q8, Q8s = _lib.quant(0, qf)
        K8, K8s = _lib.quant(1, kf, _lib.kmean(kf))
        V8, V8s = _lib.quant(2, vf)
        O, Lse = _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal)
        ctx.save_for_backward(Q8, Q8s, K8, K8s, V8, V8s, O, Lse)
        ctx.dims = (B, H, Hk, N, D)
        ctx.causal = causal
        ctx.delta_mode = delta_mode
        return O

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dO):
        from . import _lib
        B, H, Hk, N, D = ctx.dims
        Q8, Q8s, K8, K8s, V8, V8s, O, Lse = ctx.saved_tensors
        dO8, dO8s, Dlt = _lib.quant_do(dO.contiguous(), O)
        if ctx.delta_mode == "matched":
            Dlt = _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, Lse, B, H, Hk, ctx.causal)
        dk, dv, ws = _lib.bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, Lse, Dlt, B, H, Hk, ctx.causal)
        dq = _lib.bwd_pass2(ws, K8, B, H, Hk, N, D, ctx.causal)
        dk, dv = _lib.gqa_fold(dk, Hk), _lib.gqa_fold(dv, Hk)
        return dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3), None, None


def dm_attn_func_plain(q, k, v, causal=True, softmax_scale=None, delta_mode="stale"):
    """The plain route on (B, H, N, D) inputs; returns O (B, N, H, D) bf16 contiguous.  Same contract as
    dm_attn_func_bhnd."""
    _check_inputs(q, k, v, causal, softmax_scale, delta_mode)
    return _DMAttnPlain.apply(q, k, v, causal, delta_mode)
