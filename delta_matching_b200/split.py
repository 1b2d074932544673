"""The backward on head groups (long context).  Pass 1 materializes its dS' code tiles in e4m3 over
[batch * heads, N, N] bytes (1 GiB at batch 1, 16 heads, N = 8192; 4 GiB per head at N = 65536), so the call is split per
KV-head group or per query head when that workspace would exceed DM_BWD_WS_LIMIT_GB.  Heads are independent inside every
kernel (per-query-head dK / dV, fixed-order per-head reductions), so the split result is bitwise the single call's; in the
matched mode the delta is taken per group as well.  Mirrors delta_matching/split.py:17-92 of the reference: the same
environment variables and decision rule.  Unlike the reference nothing is sliced or concatenated: the kernels take a
head range and write into the full-size outputs.

DM_BWD_HEAD_GROUPS = auto (default) | off | kv | head;  DM_BWD_WS_LIMIT_GB (default 8);  DM_BWD_STREAMS = K (default 1)
runs the groups round-robin on K CUDA streams, each with its own workspace, so pass 2 of one group (bound by the dS' read)
overlaps pass 0 / pass 1 of another.
"""
from __future__ import annotations

import os as _os

import torch

from . import _lib

def _knob(name, default):
    return _os.environ.get(name, default).strip()


# The three knobs keep the reference's names and meanings; tests override the module attributes directly.
_BWD_GROUPS = _knob("DM_BWD_HEAD_GROUPS", "auto").lower()          # auto | off (also 0, 1) | kv | head
_BWD_WS_LIMIT = float(_knob("DM_BWD_WS_LIMIT_GB", "8")) * (1 << 30)   # bytes of dS' codes one call may hold
_BWD_STREAMS = max(int(_knob("DM_BWD_STREAMS", "1")), 1)
_bwd_stream_pool = {}       # (device type, index) -> side streams, made on first use and kept


def _bwd_streams(device):
    """The side streams of `device`, at least _BWD_STREAMS of them."""
    have = _bwd_stream_pool.setdefault((device.type, device.index), [])
    while len(have) < _BWD_STREAMS:
        have.append(torch.cuda.Stream(device=device))
    return have


def _bwd_heads_per_call(B, H, Hkv, n_rep, N):
    """How many query heads one backward call covers.  A forced setting answers directly (off: all H heads, kv: the n_rep
    heads that share a KV head, head: one); "auto" takes the widest of those three whose dS' codes, B * heads * N * N
    bytes, stay within the limit, and one head when none does."""
    forced = {"off": H, "0": H, "1": H, "kv": n_rep, "head": 1}.get(_BWD_GROUPS)
    if forced is not None:
        return forced
    bytes_per_head = float(B) * N * N
    return next((heads for heads in (H, n_rep) if heads * bytes_per_head <= _BWD_WS_LIMIT), 1)


def backward_all_heads(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal):
    """Pass 0 (when delta is None), pass 1 and pass 2 for every head, split into head groups when needed.
    Returns dq, dk, dv (B, N, H, D) bf16, dk / dv per query head."""
    BH, N, D = Q8.shape
    dev = Q8.device
    n_rep = H // Hk
    hp = _bwd_heads_per_call(B, H, Hk, n_rep, N)
    with torch.cuda.device(dev):
        dq = torch.empty(B, N, H, D, device=dev, dtype=torch.bfloat16)
        dk = torch.empty_like(dq)
        dv = torch.empty_like(dq)
        if delta is None and hp >= H:
            delta = _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal)
        if hp >= H:
            _, _, ws = _lib.bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal, out=(dk, dv))
            _lib.bwd_pass2(ws, K8, B, H, Hk, N, D, causal, out=dq)
            return dq, dk, dv
        per_group_delta = delta is None
        if per_group_delta:
            delta = torch.empty(BH, N, device=dev, dtype=torch.float32)
        groups = list(range(0, H, hp))
        K = min(_BWD_STREAMS, len(groups))
        cur = torch.cuda.current_stream(dev)
        streams = _bwd_streams(dev)[:K] if K > 1 else [cur]
        nb_ds, nb_psi = _lib.bwd_workspace_bytes(B, H, Hk, N, D, causal, hp)
        wss = [(torch.empty(nb_ds, device=dev, dtype=torch.uint8), torch.empty(nb_psi // 4, device=dev, dtype=torch.float32))
               for _ in range(K)]
        if K > 1:
            ready = torch.cuda.Event()
            ready.record(cur)
            for s in streams:
                s.wait_event(ready)
        for i, h0 in enumerate(groups):
            assert (h0 + hp - 1) // n_rep == h0 // n_rep, "a call must stay inside one KV group"
            s, ws = streams[i % K], wss[i % K]
            with torch.cuda.stream(s):
                if per_group_delta:
                    _lib.delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal, h0=h0, hcount=hp, out=delta)
                _lib.bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal, h0=h0, hcount=hp, out=(dk, dv), ws=ws)
                _lib.bwd_pass2(ws, K8, B, H, Hk, N, D, causal, h0=h0, hcount=hp, out=dq)
        if K > 1:
            for s in streams:
                cur.wait_stream(s)
            for t in (dq, dk, dv, delta, *[w for ws in wss for w in ws]):
                t.record_stream(cur)
        return dq, dk, dv
