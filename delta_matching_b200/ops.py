"""The op layer: torch.library custom ops in the `dm_b200` namespace over the C ABI (delta_matching_b200._lib).

Replaces the reference's TORCH_LIBRARY(delta_matching) block (csrc/delta_matching_api.cpp:684-736): the ops allocate
their outputs and workspaces with torch on the inputs' device, run on that device's current stream, mutate nothing and
have fake (meta) implementations so torch.compile can trace through them.  Code tensors are [B*heads, N, D] e4m3,
scales [B*heads, N / rows_per_scale] fp32, O / dQ / dK / dV (B, N, H, D) bf16, LSE / delta [B*H, N] fp32.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib

E4M3 = torch.float8_e4m3fn


def _lane(t):
    return t if t.stride(-1) == 1 else t.contiguous()


@torch.library.custom_op("dm_b200::quant_qkv", mutates_args=())
def quant_qkv(q: Tensor, k: Tensor, v: Tensor) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """q (B, N, H, D), k / v (B, N, Hk, D) bf16 (any dense strides with unit head_dim stride) -> Q8, Q8s, K8, K8s, V8, V8s.
    K is centred by its per-head mean; the softmax scale D^-0.5 is baked into the Q codes."""
    Q8, Q8s = _lib.quant(0, q)
    km = _lib.kmean(k)
    K8, K8s = _lib.quant(1, k, km)
    V8, V8s = _lib.quant(2, v)
    return Q8, Q8s, K8, K8s, V8, V8s


@quant_qkv.register_fake
def _(q, k, v):
    B, N, H, D = q.shape
    Hk = k.shape[2]
    rq, rk = _lib.blocks(D)
    f = lambda *s, dt: q.new_empty(s, dtype=dt)
    return (f(B * H, N, D, dt=E4M3), f(B * H, N // rq, dt=torch.float32), f(B * Hk, N, D, dt=E4M3), f(B * Hk, N // rk, dt=torch.float32),
            f(B * Hk, N, D, dt=E4M3), f(B * Hk, N // rk, dt=torch.float32))


@torch.library.custom_op("dm_b200::quant_do", mutates_args=())
def quant_do(dO: Tensor, o: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor]:
    """dO (B, N, H, D) bf16 -> dO8, dO8s and, when `o` is given, the stale delta rowsum(dO * O) (else an empty tensor)."""
    c, s, d = _lib.quant_do(dO, o)
    if d is None:
        d = dO.new_empty((0,), dtype=torch.float32)
    return c, s, d


@quant_do.register_fake
def _(dO, o):
    B, N, H, D = dO.shape
    rq = _lib.blocks(D)[0]
    return (dO.new_empty((B * H, N, D), dtype=E4M3), dO.new_empty((B * H, N // rq), dtype=torch.float32),
            dO.new_empty((B * H, N) if o is not None else (0,), dtype=torch.float32))


@torch.library.custom_op("dm_b200::fwd_fp8", mutates_args=())
def fwd_fp8(Q8: Tensor, K8: Tensor, V8: Tensor, Q8s: Tensor, K8s: Tensor, V8s: Tensor, B: int, H: int, Hk: int,
            causal: bool) -> Tuple[Tensor, Tensor]:
    return _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal)


@fwd_fp8.register_fake
def _(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal):
    BH, N, D = Q8.shape
    return Q8.new_empty((B, N, H, D), dtype=torch.bfloat16), Q8.new_empty((BH, N), dtype=torch.float32)


@torch.library.custom_op("dm_b200::delta_fp8", mutates_args=())
def delta_fp8(Q8: Tensor, K8: Tensor, V8: Tensor, dO8: Tensor, Q8s: Tensor, K8s: Tensor, V8s: Tensor, dO8s: Tensor, lse: Tensor,
              B: int, H: int, Hk: int, causal: bool) -> Tensor:
    return _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal)


@delta_fp8.register_fake
def _(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal):
    return lse.new_empty(lse.shape)


@torch.library.custom_op("dm_b200::bwd_fp8", mutates_args=())
def bwd_fp8(Q8: Tensor, K8: Tensor, V8: Tensor, dO8: Tensor, Q8s: Tensor, K8s: Tensor, V8s: Tensor, dO8s: Tensor, lse: Tensor,
            delta: Optional[Tensor], B: int, H: int, Hk: int, causal: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """dQ, dK, dV (B, N, H, D) bf16 with dK / dV per QUERY head.  delta None = matched mode with the delta taken per
    head group inside the split.  Splits the heads when the dS' workspace would exceed the limit (split.py)."""
    from .split import backward_all_heads
    return backward_all_heads(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal)


@bwd_fp8.register_fake
def _(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal):
    BH, N, D = Q8.shape
    e = lambda: Q8.new_empty((B, N, H, D), dtype=torch.bfloat16)
    return e(), e(), e()


@torch.library.custom_op("dm_b200::gqa_fold", mutates_args=())
def gqa_fold(x: Tensor, Hk: int) -> Tensor:
    out = _lib.gqa_fold(x, Hk)
    return out if out is not x else x.clone()


@gqa_fold.register_fake
def _(x, Hk):
    B, N, H, D = x.shape
    return x.new_empty((B, N, Hk, D))


def attn_fwd_eager(q: Tensor, k: Tensor, v: Tensor, causal: bool):
    """The whole forward as plain calls into the library: q (B, N, H, D), k / v (B, N, Hk, D) bf16 ->
    O, LSE, Q8, Q8s, K8, K8s, V8, V8s.  The autograd route calls this directly in eager mode (the torch.library dispatcher
    costs more host time per call than all the kernel launches together) and the custom op below under torch.compile."""
    return _lib.attn_forward(q, k, v, causal)


@torch.library.custom_op("dm_b200::attn_fwd", mutates_args=())
def attn_fwd(q: Tensor, k: Tensor, v: Tensor, causal: bool) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor]:
    """attn_fwd_eager as one traceable op."""
    return attn_fwd_eager(q, k, v, causal)


@attn_fwd.register_fake
def _(q, k, v, causal):
    B, N, H, D = q.shape
    Hk = k.shape[2]
    rq, rk = _lib.blocks(D)
    f = lambda *s, dt: q.new_empty(s, dtype=dt)
    return (f(B, N, H, D, dt=torch.bfloat16), f(B * H, N, dt=torch.float32), f(B * H, N, D, dt=E4M3), f(B * H, N // rq, dt=torch.float32),
            f(B * Hk, N, D, dt=E4M3), f(B * Hk, N // rk, dt=torch.float32), f(B * Hk, N, D, dt=E4M3), f(B * Hk, N // rk, dt=torch.float32))


def attn_bwd_eager(dO: Tensor, O: Tensor, lse: Tensor, Q8: Tensor, Q8s: Tensor, K8: Tensor, K8s: Tensor, V8: Tensor, V8s: Tensor,
                   B: int, H: int, Hk: int, causal: bool, matched: bool):
    """The whole backward as plain calls into the library: dO quantizer (with the stale delta only in the stale mode),
    pass 0 / 1 / 2 with the head-group split, GQA fold.  Returns dQ (B, N, H, D), dK / dV (B, N, Hk, D) bf16."""
    from .split import backward_all_heads, _bwd_heads_per_call
    if _bwd_heads_per_call(B, H, Hk, H // Hk, Q8.shape[1]) >= H:      # no head-group split: one library call
        return _lib.attn_backward(dO, O, lse, Q8, Q8s, K8, K8s, V8, V8s, B, H, Hk, causal, matched)
    with torch.cuda.device(dO.device):
        dO8, dO8s, delta = _lib.quant_do(dO, None if matched else O)
        dq, dk, dv = backward_all_heads(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal)
        if Hk < H:
            dk, dv = _lib.gqa_fold(dk, Hk), _lib.gqa_fold(dv, Hk)
    return dq, dk, dv


@torch.library.custom_op("dm_b200::attn_bwd", mutates_args=())
def attn_bwd(dO: Tensor, O: Tensor, lse: Tensor, Q8: Tensor, Q8s: Tensor, K8: Tensor, K8s: Tensor, V8: Tensor, V8s: Tensor, B: int,
             H: int, Hk: int, causal: bool, matched: bool) -> Tuple[Tensor, Tensor, Tensor]:
    """attn_bwd_eager as one traceable op."""
    return attn_bwd_eager(dO, O, lse, Q8, Q8s, K8, K8s, V8, V8s, B, H, Hk, causal, matched)


@attn_bwd.register_fake
def _(dO, O, lse, Q8, Q8s, K8, K8s, V8, V8s, B, H, Hk, causal, matched):
    BH, N, D = Q8.shape
    return (Q8.new_empty((B, N, H, D), dtype=torch.bfloat16), Q8.new_empty((B, N, Hk, D), dtype=torch.bfloat16),
            Q8.new_empty((B, N, Hk, D), dtype=torch.bfloat16))
