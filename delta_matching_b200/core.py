"""The input contract, the block-scale contract and the library identity of the B200 build.

Mirrors delta_matching/core.py of the reference (`blocks` :26-29, `_check_inputs` :112-154, `_ops` / `loaded_library`
:81-109): same checks in the same order, same exception classes and message keywords; the capability check asks for
sm_100 (B200) instead of sm_90.
"""
from __future__ import annotations

import torch

from . import _lib

blocks = _lib.blocks


def loaded_library():
    """The path of the loaded shared library (None before the first kernel call)."""
    return _lib.loaded_library()


def _check_inputs(q, k, v, causal, softmax_scale, mode):
    """The input contract on (B, H, N, D) views: raises ValueError / TypeError / NotImplementedError naming the violated
    constraint (explicit checks, so they also hold under `python -O`)."""
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v)):
        raise TypeError("delta_matching: q, k, v must be torch tensors")
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError(f"delta_matching: q, k, v must be 4-D (got {q.dim()}-D, {k.dim()}-D, {v.dim()}-D)")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError(f"delta_matching: q, k, v must be CUDA tensors (got {q.device}, {k.device}, {v.device})")
    if not (q.device == k.device == v.device):
        raise ValueError(f"delta_matching: q, k, v must be on one device (got {q.device}, {k.device}, {v.device})")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise TypeError(f"delta_matching: q, k, v must be torch.bfloat16 (got {q.dtype}, {k.dtype}, {v.dtype})")
    if mode not in ("matched", "stale"):
        raise ValueError(f"delta_matching: mode must be 'matched' or 'stale' (got {mode!r})")
    if mode == "matched" and not causal:
        raise ValueError("delta_matching: mode='matched' needs causal=True (the matched delta is built for causal attention); "
                         "use mode='stale' for non-causal attention")
    B, H, N, D = q.shape
    if k.shape != v.shape:
        raise ValueError(f"delta_matching: k and v must have the same shape (got {tuple(k.shape)} and {tuple(v.shape)})")
    Bk, Hk, Nk, Dk = k.shape
    if Bk != B or Dk != D:
        raise ValueError(f"delta_matching: k and v must match q's batch size and head_dim (q {tuple(q.shape)}, k {tuple(k.shape)})")
    if Nk != N:
        raise ValueError(f"delta_matching: q, k, v must have the same seqlen (self-attention only; got {N} and {Nk})")
    if Hk == 0 or H % Hk:
        raise ValueError(f"delta_matching: nheads ({H}) must be a positive multiple of nheads_k ({Hk})")
    if D not in (128, 256):
        raise ValueError(f"delta_matching: head_dim must be 128 or 256 (got {D})")
    mult = 256 if D == 128 else 128
    if N == 0 or N % mult:
        raise ValueError(f"delta_matching: seqlen must be a positive multiple of {mult} at head_dim {D} (got {N})")
    if B == 0:
        raise ValueError("delta_matching: empty batch")
    if B * H > 65535:
        raise ValueError(f"delta_matching: batch * nheads must be at most 65535 (got {B * H})")
    if softmax_scale is not None and abs(softmax_scale - D ** -0.5) > 1e-12:
        raise NotImplementedError(f"delta_matching: softmax_scale is fixed at head_dim ** -0.5 = {D ** -0.5!r} (it is baked "
                                  f"into the Q codes); got {softmax_scale!r}")
    major, minor = torch.cuda.get_device_capability(q.device)
    if (major, minor) != (10, 0):
        raise ValueError(f"delta_matching: needs a Blackwell B200 GPU (sm100); {q.device} is sm{major}{minor}")
