"""Host-side logic that needs no GPU: the library loads and exports every symbol declared in include/dm_b200.h, the C ABI
validates shapes before touching the device, the head-group split decision, and the argument checks of the public API
that precede any device work."""
import ctypes as C
import os
import re

import pytest
import torch

import delta_matching_b200 as dm
from delta_matching_b200 import _lib, split

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "dm_b200.h")).read()
    declared = set(re.findall(r"\b(dm_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    handle = C.CDLL(_lib.library_path())
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared in include/dm_b200.h but not exported"
    assert set(_lib.EXPORTS) == declared, (set(_lib.EXPORTS) ^ declared)
    assert "sm_100a" in _lib.build_info()


def test_shape_validation_happens_before_any_device_work():
    lib = _lib.lib()
    err = C.create_string_buffer(256)
    bad = [(_lib.DmShape(1, 4, 4, 1000, 128, 1), "seqlen"), (_lib.DmShape(1, 4, 3, 512, 128, 1), "nheads"),
           (_lib.DmShape(1, 4, 4, 512, 64, 1), "head_dim"), (_lib.DmShape(0, 4, 4, 512, 128, 1), "empty"),
           (_lib.DmShape(70000, 1, 1, 512, 128, 1), "65535")]
    for shp, word in bad:
        rc = lib.dm_fwd_fp8(None, None, None, None, None, None, shp, 0, shp.H, None, None, None, err, len(err))
        assert rc == -1 and word in err.value.decode(), (rc, err.value)
    rc = lib.dm_fwd_fp8(None, None, None, None, None, None, _lib.DmShape(1, 4, 4, 512, 128, 1), 2, 4, None, None, None, err, len(err))
    assert rc == -1 and "head range" in err.value.decode()
    a, b = C.c_size_t(0), C.c_size_t(0)
    assert lib.dm_bwd_workspace_bytes(_lib.DmShape(1, 16, 16, 8192, 128, 1), 16, C.byref(a), C.byref(b)) == 0
    assert a.value == 2 ** 30 and b.value == 16 * 128 * 64 * 4          # 1 GiB at batch 1, 16 heads, N = 8192
    assert lib.dm_kmean_scratch_bytes(4, 8, 4096, 128) == 4 * 8 * 64 * 128 * 4


def test_register_pool_rule():
    """Kernels whose roles trade registers with setmaxnreg are refused unless the compiled register count times the
    thread count covers what the roles request: pass 1 (768 threads: 16 x 32 x 64 + 128 x 184 + 128 x 40 = 768 x 80) and
    the forward (512 threads: 256 x 128 + 128 x 208 + 128 x 40 = 512 x 128)."""
    ok = _lib.lib().dm_register_pool_ok
    assert ok(80, 768, 16 * 32 * 64 + 128 * 184 + 128 * 40) == 1
    assert ok(72, 768, 16 * 32 * 64 + 128 * 184 + 128 * 40) == 0       # a compiler that found a tighter allocation
    assert ok(128, 512, 256 * 128 + 128 * 208 + 128 * 40) == 1
    assert ok(120, 512, 256 * 128 + 128 * 208 + 128 * 40) == 0
    assert ok(0, 256, 1) == 0 and ok(128, 0, 1) == 0


def test_head_group_split_decision(monkeypatch):
    monkeypatch.setattr(split, "_BWD_GROUPS", "auto")
    monkeypatch.setattr(split, "_BWD_WS_LIMIT", 8 * 2 ** 30)
    assert split._bwd_heads_per_call(1, 16, 4, 4, 8192) == 16            # 1 GiB: no split
    assert split._bwd_heads_per_call(4, 32, 8, 4, 4096) == 32            # config 3: 2 GiB
    assert split._bwd_heads_per_call(1, 32, 8, 4, 65536) == 1            # config 5: 4 GiB per head
    assert split._bwd_heads_per_call(1, 32, 8, 4, 32768) == 4            # 1 GiB per head: per KV group
    monkeypatch.setattr(split, "_BWD_GROUPS", "kv")
    assert split._bwd_heads_per_call(1, 16, 4, 4, 1024) == 4
    monkeypatch.setattr(split, "_BWD_GROUPS", "head")
    assert split._bwd_heads_per_call(1, 16, 4, 4, 1024) == 1
    monkeypatch.setattr(split, "_BWD_GROUPS", "off")
    assert split._bwd_heads_per_call(1, 32, 8, 4, 65536) == 32


def test_argument_checks_that_precede_device_work():
    q = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError, match="dropout"):
        dm.flash_attn_func(q, q, q, 0.1, causal=True)
    with pytest.raises(NotImplementedError, match="window"):
        dm.flash_attn_func(q, q, q, causal=True, window_size=(128, 0))
    with pytest.raises(NotImplementedError, match="softcap"):
        dm.flash_attn_func(q, q, q, causal=True, softcap=30.0)
    with pytest.raises(NotImplementedError, match="alibi"):
        dm.flash_attn_func(q, q, q, causal=True, alibi_slopes=torch.zeros(2))
    with pytest.raises(NotImplementedError, match="return_attn_probs"):
        dm.flash_attn_func(q, q, q, causal=True, return_attn_probs=True)
    with pytest.raises(ValueError, match="4-D"):
        dm.dm_attn_func(q[0], q[0], q[0], causal=True)
    with pytest.raises(ValueError, match="4-D"):
        dm.dm_attn_func(None, q, q, causal=True)
    with pytest.raises(TypeError, match="tensors"):
        dm.dm_attn_func_bhnd(None, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        dm.dm_attn_func(q, q, q, causal=True)
    assert dm.blocks(128) == (128, 64) and dm.blocks(256) == (64, 32)
    s = dm.kernel_version()
    assert len(s["code_sha"]) == 12 and s["numerics"]["128"]


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("DM_SO", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="does not exist"):
        _lib.library_path()


def _snake_items(total, ctas):
    """The walk of the persistent kernels (bwd1_item in dm_bwd1.cu, fwd_item in dm_fwd.cu): CTA c takes position c of the
    even rounds and ctas - 1 - c of the odd ones and stops at its first position past the end of the list."""
    taken = []
    for c in range(ctas):
        mine, r = [], 0
        while True:
            idx = r * ctas + (ctas - 1 - c if r & 1 else c)
            if idx >= total:
                break
            mine.append(idx)
            r += 1
        taken.append(mine)
    return taken


@pytest.mark.parametrize("heads,blocks,ctas", [(32, 16, 148), (128, 32, 148), (1, 512, 148), (3, 5, 148), (32, 16, 7), (1, 1, 1)])
def test_persistent_walk_covers_every_item_once(heads, blocks, ctas):
    """Stopping at the first invalid position loses nothing (only the last round is partial), every item is taken exactly
    once, and with the causal weights (key block J of a head has blocks - J row pairs, items ordered by J) the heaviest
    CTA carries at most one heaviest item more than the mean."""
    total = heads * blocks
    ctas = min(ctas, total)
    taken = _snake_items(total, ctas)
    flat = sorted(i for mine in taken for i in mine)
    assert flat == list(range(total))
    weight = lambda idx: blocks - idx // heads
    loads = [sum(weight(i) for i in mine) for mine in taken]
    assert max(loads) - sum(loads) / ctas <= blocks
