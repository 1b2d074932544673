"""delta_matching_b200 -- Delta-Matching fp8 attention for training on B200 (sm_100a).

Public surface (a drop-in for the `delta_matching` package: same callables, defaults, tensor layouts and exception types):

    dm_attn_func(q, k, v, softmax_scale=None, causal=False, mode="matched")      flash layout (B, N, H, D)
    dm_attn_func_bhnd(q, k, v, causal=False, softmax_scale=None, delta_mode=...)  head-major layout (B, H, N, D)
    flash_attn_func(...)                                                         flash_attn's signature
    dm_attn_func_plain(...)                                                      the cross-check route
    dm_attn_func_cp(...)                                                         sequence split over a process group

What runs underneath: Q, K, V (K minus its per-head mean) become e4m3 codes with per-block fp32 scales; the forward keeps a
per-row, per-key-group basis for P; the backward runs its five matmuls in fp8 and, in "matched" mode, takes the centring
term delta of the softmax gradient from the backward's own fp8 P and dP (so every row of dS sums to zero up to fp32
round-off), while "stale" mode uses rowsum(dO * O).  Limits: self-attention, bf16 CUDA tensors on a B200, head_dim 128
(seqlen a multiple of 256) or 256 (a multiple of 128), softmax_scale fixed at head_dim ** -0.5, "matched" only with
causal=True.  Anything else is refused with ValueError / TypeError / NotImplementedError before a kernel is launched.
Every kernel is hand-written sm_100a CUDA behind the C ABI of include/dm_b200.h; nothing falls back to another path.
"""
from __future__ import annotations

import torch

from .attn import dm_attn_func_bhnd, dm_attn_func_plain
from . import split  # noqa: F401  (the DM_BWD_* environment knobs are read there)
from .core import blocks
from .cp import dm_attn_func_cp, zigzag_shard, zigzag_unshard

__version__ = "0.1.0"
KERNEL_NUMERICS = {"128": "Delta-Matching-128 v3", "256": "Delta-Matching-256 v1"}
__all__ = ["dm_attn_func", "dm_attn_func_bhnd", "dm_attn_func_plain", "flash_attn_func", "dm_attn_func_cp", "zigzag_shard",
           "zigzag_unshard", "blocks", "kernel_version", "__version__", "KERNEL_NUMERICS"]


def _head_major(name, t):
    if not (isinstance(t, torch.Tensor) and t.dim() == 4):
        raise ValueError(f"delta_matching: {name} has to be a 4-D tensor laid out (batch, seqlen, nheads, headdim)")
    return t.transpose(1, 2)


def dm_attn_func(q, k, v, softmax_scale=None, causal=False, mode="matched"):
    """q (B, N, H, D) and k, v (B, N, Hk, D), bf16 on a B200, give o (B, N, H, D) bf16; H must be a multiple of Hk.
    `mode` picks the backward's delta: "matched" (needs causal=True) or "stale"."""
    qh, kh, vh = _head_major("q", q), _head_major("k", k), _head_major("v", v)
    return dm_attn_func_bhnd(qh, kh, vh, causal=causal, softmax_scale=softmax_scale, delta_mode=mode)


# flash_attn_func arguments this kernel has no implementation for: (name, the only accepted value, what to say)
_FLASH_ONLY_DEFAULTS = (
    ("dropout_p", 0.0, "attention dropout is outside this kernel: pass dropout_p=0"),
    ("window_size", (-1, -1), "a sliding window_size is outside this kernel: pass (-1, -1)"),
    ("softcap", 0.0, "logit softcap is outside this kernel: pass softcap=0"),
    ("alibi_slopes", None, "alibi_slopes (ALiBi bias) is outside this kernel: pass None"),
    ("return_attn_probs", False, "return_attn_probs=True is outside this kernel: the probabilities are never materialised"),
)


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1), softcap=0.0,
                    alibi_slopes=None, deterministic=False, return_attn_probs=False, mode="matched"):
    """The call `flash_attn.flash_attn_func` takes, so a model switches by changing one import.  Features outside this kernel
    (dropout, windows, softcap, alibi, returned probabilities) must stay at their defaults; `deterministic` may be anything,
    the outputs are deterministic regardless; `mode` is the extra keyword that selects the delta."""
    given = {"dropout_p": dropout_p, "window_size": window_size, "softcap": softcap, "alibi_slopes": alibi_slopes,
             "return_attn_probs": return_attn_probs}
    for name, accepted, complaint in _FLASH_ONLY_DEFAULTS:
        value = given[name]
        if isinstance(accepted, tuple) and value is not None:
            value = tuple(value)        # a list [-1, -1] is the same window as the tuple
        if (value is not None) if accepted is None else (value != accepted):
            raise NotImplementedError("delta_matching: " + complaint)
    return dm_attn_func(q, k, v, softmax_scale=softmax_scale, causal=causal, mode=mode)


def kernel_version():
    """What to print into a training log: package version, a hash over the kernel sources and the C header, the numerics
    tags per head dim and, when the shared library can be loaded, its build string and path."""
    from . import _lib
    from .build import code_sha
    stamp = dict(version=__version__, code_sha=code_sha(), numerics=KERNEL_NUMERICS, arch="sm_100a", bf16_dp=False)
    try:
        stamp.update(build=_lib.build_info(), library=_lib.loaded_library())
    except Exception:       # not built yet, or no loadable library on this machine: the stamp stays partial
        pass
    return stamp
