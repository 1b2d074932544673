"""delta_matching_b200: Delta-Matching fp8 attention for training, B200 (sm_100a) build.

A drop-in for the `delta_matching` package's attention API (same names, defaults, layouts, exceptions):

    from delta_matching_b200 import dm_attn_func
    o = dm_attn_func(q, k, v, causal=True, mode="matched")     # GQA: k, v carry nheads_k with nheads % nheads_k == 0
    o = dm_attn_func(q, k, v, causal=True, mode="stale")

Tensors (batch, seqlen, nheads, headdim), bf16, CUDA, B200.  The forward keeps the attention core in fp8 (e4m3 Q, K, V
codes with per-block scales, a faithful per-row, per-key-group P basis); the backward keeps all five backward matmuls in
fp8 and, in the "matched" mode, forms the softmax-gradient centring term delta from the backward's own fp8 P / dP pair
(pass 0), so that rowsum(dS) = 0 holds to fp32 round-off.  The "stale" mode is the conventional delta = rowsum(dO * O).
Constraints: self-attention; head_dim 128 (seqlen % 256 == 0) or 256 (seqlen % 128 == 0); bf16; softmax_scale =
head_dim ** -0.5; mode "matched" needs causal=True.  Violations raise ValueError / TypeError / NotImplementedError.
All compute runs in hand-written sm_100a CUDA kernels behind a C ABI (include/dm_b200.h); there is no fallback path.
"""
from __future__ import annotations

import torch

from .attn import dm_attn_func_bhnd, dm_attn_func_plain
from . import split  # noqa: F401  (DM_BWD_* environment knobs live there)
from .core import blocks
from .cp import dm_attn_func_cp, zigzag_shard, zigzag_unshard

__version__ = "0.1.0"
KERNEL_NUMERICS = {"128": "Delta-Matching-128 v3", "256": "Delta-Matching-256 v1"}
__all__ = ["dm_attn_func", "dm_attn_func_bhnd", "dm_attn_func_plain", "flash_attn_func", "dm_attn_func_cp", "zigzag_shard",
           "zigzag_unshard", "blocks", "kernel_version", "__version__", "KERNEL_NUMERICS"]


def dm_attn_func(q, k, v, softmax_scale=None, causal=False, mode="matched"):
    """Attention in the flash-attention layout: q (B, N, H, D), k / v (B, N, Hk, D) bf16 on CUDA -> o (B, N, H, D) bf16.
    mode: "matched" (the Delta-Matching backward; needs causal=True) or "stale" (delta = rowsum(dO * O))."""
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or t.dim() != 4:
            raise ValueError(f"delta_matching: {name} must be a 4-D tensor (batch, seqlen, nheads, headdim)")
    return dm_attn_func_bhnd(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal,
                             softmax_scale=softmax_scale, delta_mode=mode)


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False, mode="matched"):
    """flash_attn.flash_attn_func's signature for one-line ports; the arguments this kernel does not implement must be at
    their defaults.  `mode` selects the delta ("matched" or "stale"); `deterministic` is accepted and ignored, since every
    output is deterministic."""
    if dropout_p != 0.0:
        raise NotImplementedError("delta_matching: dropout is not implemented (dropout_p must be 0)")
    if tuple(window_size) != (-1, -1):
        raise NotImplementedError("delta_matching: sliding windows are not implemented (window_size must be (-1, -1))")
    if softcap != 0.0:
        raise NotImplementedError("delta_matching: softcap is not implemented")
    if alibi_slopes is not None:
        raise NotImplementedError("delta_matching: alibi_slopes are not implemented")
    if return_attn_probs:
        raise NotImplementedError("delta_matching: return_attn_probs is not implemented")
    return dm_attn_func(q, k, v, softmax_scale=softmax_scale, causal=causal, mode=mode)


def kernel_version():
    """A stamp for training logs: the package version, a content hash of the kernel sources, the numerics tags and, once
    the library is loaded, its path and build string."""
    from . import _lib
    from .build import code_sha
    info = {"version": __version__, "code_sha": code_sha(), "numerics": KERNEL_NUMERICS, "arch": "sm_100a", "bf16_dp": False}
    try:
        info["build"] = _lib.build_info()
        info["library"] = _lib.loaded_library()
    except Exception:
        pass
    return info
