"""The input contract, the block-scale contract and the library identity of the B200 build.

The contract is the reference's (delta_matching/core.py:112-154: which exception class each violation raises, and the word
each message must contain, as its tests/test_api.py:117-143 match on them); the capability rule asks for sm_100 (B200)
instead of sm_90.  Here it is a table of rules evaluated in order on a small record of the call.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

from . import _lib

blocks = _lib.blocks
_SEQLEN_MULTIPLE = {128: 256, 256: 128}       # the forward walks 128-key tiles in pairs at head_dim 128


def loaded_library():
    """Path of the shared library the kernels come from; None until the first call has loaded it."""
    return _lib.loaded_library()


@dataclass(frozen=True)
class _Call:
    q: object
    k: object
    v: object
    causal: bool
    scale: Optional[float]
    mode: object

    @property
    def qkv(self):
        return (self.q, self.k, self.v)

    def each(self, attr):
        return ", ".join(str(getattr(t, attr)() if callable(getattr(t, attr)) else getattr(t, attr)) for t in self.qkv)


@dataclass(frozen=True)
class _Rule:
    broken: Callable[[_Call], bool]
    error: type
    text: Callable[[_Call], str]


def _dims(c):
    return c.q.shape, c.k.shape, c.v.shape


_RULES = (
    _Rule(lambda c: any(not isinstance(t, torch.Tensor) for t in c.qkv), TypeError, lambda c: "q, k, v must be torch tensors"),
    _Rule(lambda c: any(t.dim() != 4 for t in c.qkv), ValueError,
          lambda c: "q, k, v must be 4-D (got " + ", ".join(f"{t.dim()}-D" for t in c.qkv) + ")"),
    _Rule(lambda c: any(not t.is_cuda for t in c.qkv), ValueError, lambda c: f"q, k, v must be CUDA tensors (got {c.each('device')})"),
    _Rule(lambda c: len({t.device for t in c.qkv}) != 1, ValueError, lambda c: f"q, k, v must be on one device (got {c.each('device')})"),
    _Rule(lambda c: any(t.dtype != torch.bfloat16 for t in c.qkv), TypeError,
          lambda c: f"q, k, v must be torch.bfloat16 (got {c.each('dtype')})"),
    _Rule(lambda c: c.mode not in ("matched", "stale"), ValueError, lambda c: f"mode must be 'matched' or 'stale' (got {c.mode!r})"),
    _Rule(lambda c: c.mode == "matched" and not c.causal, ValueError,
          lambda c: "mode='matched' needs causal=True (the matched delta is built for causal attention); use mode='stale' for "
                    "non-causal attention"),
    _Rule(lambda c: c.k.shape != c.v.shape, ValueError,
          lambda c: f"k and v must have the same shape (got {tuple(c.k.shape)} and {tuple(c.v.shape)})"),
    _Rule(lambda c: c.k.shape[0] != c.q.shape[0] or c.k.shape[3] != c.q.shape[3], ValueError,
          lambda c: f"k and v must match q's batch size and head_dim (q {tuple(c.q.shape)}, k {tuple(c.k.shape)})"),
    _Rule(lambda c: c.k.shape[2] != c.q.shape[2], ValueError,
          lambda c: f"q, k, v must have the same seqlen (self-attention only; got {c.q.shape[2]} and {c.k.shape[2]})"),
    _Rule(lambda c: c.k.shape[1] == 0 or c.q.shape[1] % c.k.shape[1] != 0, ValueError,
          lambda c: f"nheads ({c.q.shape[1]}) must be a positive multiple of nheads_k ({c.k.shape[1]})"),
    _Rule(lambda c: c.q.shape[3] not in _SEQLEN_MULTIPLE, ValueError, lambda c: f"head_dim must be 128 or 256 (got {c.q.shape[3]})"),
    _Rule(lambda c: c.q.shape[2] == 0 or c.q.shape[2] % _SEQLEN_MULTIPLE[c.q.shape[3]] != 0, ValueError,
          lambda c: f"seqlen must be a positive multiple of {_SEQLEN_MULTIPLE[c.q.shape[3]]} at head_dim {c.q.shape[3]} "
                    f"(got {c.q.shape[2]})"),
    _Rule(lambda c: c.q.shape[0] == 0, ValueError, lambda c: "empty batch"),
    _Rule(lambda c: c.q.shape[0] * c.q.shape[1] > 65535, ValueError,
          lambda c: f"batch * nheads must be at most 65535 (got {c.q.shape[0] * c.q.shape[1]})"),
    _Rule(lambda c: c.scale is not None and abs(c.scale - c.q.shape[3] ** -0.5) > 1e-12, NotImplementedError,
          lambda c: f"softmax_scale is fixed at head_dim ** -0.5 = {c.q.shape[3] ** -0.5!r} (it is baked into the Q codes); "
                    f"got {c.scale!r}"),
    _Rule(lambda c: torch.cuda.get_device_capability(c.q.device) != (10, 0), ValueError,
          lambda c: "needs a Blackwell B200 GPU (sm100); {} is sm{}{}".format(c.q.device, *torch.cuda.get_device_capability(c.q.device))),
)


def _check_inputs(q, k, v, causal, softmax_scale, mode):
    """Validate a call on (B, H, N, D) views before any device work.  The first broken rule raises its exception
    (ValueError, TypeError or NotImplementedError) with a message that names the constraint.  Plain `raise`, never
    `assert`, so the checks survive `python -O`."""
    call = _Call(q, k, v, causal, softmax_scale, mode)
    for rule in _RULES:
        if rule.broken(call):
            raise rule.error("delta_matching: " + rule.text(call))
