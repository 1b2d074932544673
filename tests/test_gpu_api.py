"""End-to-end through the public API on the GPU: the reference's own test strategy (tests/test_dm_attn.py and
tests/test_api.py of the reference) -- tolerances against fp32 attention, bitwise determinism, the structural identities
between the two delta modes, the plain route, strided inputs, the head-group split, argument errors -- plus parity of
every output against the CPU oracle on the same seeded inputs."""
import inspect
import math

import pytest
import torch

import delta_matching_b200 as dm
from oracle import dm_oracle as O

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
TOL = {"O": 8e-2, "dV": 8e-2, "dQ": 1.2e-1, "dK": 1.2e-1}     # the reference's bounds (tests/test_dm_attn.py:15)
SHAPES = {"mha": (1, 4, 4, 2048), "gqa": (1, 8, 2, 2048)}      # (B, H, Hk, N)


def _inputs(B, H, Hk, N, D, seed):
    return O.make_inputs(B, N, H, Hk, D, seed)


def _run(q, k, v, do, mode, causal=True, fn=None):
    fn = fn or dm.dm_attn_func
    q, k, v = (t.cuda().clone().requires_grad_(True) for t in (q, k, v))
    o = fn(q, k, v, causal=causal, mode=mode)
    o.backward(do.cuda())
    return o.detach(), q.grad, k.grad, v.grad


@pytest.mark.parametrize("shape", sorted(SHAPES))
@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_matches_fp32_reference(shape, mode):
    B, H, Hk, N = SHAPES[shape]
    q, k, v, do = _inputs(B, H, Hk, N, 128, 0)
    ref = O.fp32_reference(q, k, v, do)
    got = _run(q, k, v, do, mode)
    assert got[0].shape == q.shape and got[1].shape == q.shape and got[2].shape == k.shape and got[3].shape == v.shape
    for name, a, b in zip(("O", "dQ", "dK", "dV"), got, ref):
        e = O.rel(a.cpu(), b)
        assert math.isfinite(e) and e < TOL[name], f"{name} relative error {e:.4f} exceeds {TOL[name]} ({shape}, {mode})"


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_stale_noncausal_matches_fp32_reference(shape):
    B, H, Hk, N = SHAPES[shape]
    q, k, v, do = _inputs(B, H, Hk, N, 128, 4)
    ref = O.fp32_reference(q, k, v, do, causal=False)
    got = _run(q, k, v, do, "stale", causal=False)
    for name, a, b in zip(("O", "dQ", "dK", "dV"), got, ref):
        assert O.rel(a.cpu(), b) < TOL[name], name


@pytest.mark.parametrize("cfg", [(1, 2, 2, 256, True, "matched"), (2, 4, 2, 512, True, "matched"), (1, 4, 1, 512, True, "stale"),
                                 (1, 2, 2, 512, False, "stale")])
def test_every_output_matches_the_oracle(cfg):
    """BASELINE config 1 and small relatives: O, dQ, dK, dV against the CPU oracle on identical bits."""
    B, H, Hk, N, causal, mode = cfg
    q, k, v, do = _inputs(B, H, Hk, N, 128, 1001)
    r = O.attention_fwd_bwd(q, k, v, do, causal, mode, fwd_tile_keys=128, pv="group")
    got = _run(q, k, v, do, mode, causal)
    for name, a in zip(("O", "dQ", "dK", "dV"), got):
        e = O.rel(a.cpu(), r[name])
        assert e < 4e-3, f"{name}: relative difference to the oracle {e:.2e}"


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_deterministic(mode):
    B, H, Hk, N = SHAPES["gqa"]
    q, k, v, do = _inputs(B, H, Hk, N, 128, 1)
    a = _run(q, k, v, do, mode)
    b = _run(q, k, v, do, mode)
    for x, y, name in zip(a, b, ("O", "dQ", "dK", "dV")):
        assert torch.equal(x, y), f"{name} differs between two identical calls ({mode})"


def test_modes_share_forward_and_dv():
    B, H, Hk, N = SHAPES["gqa"]
    q, k, v, do = _inputs(B, H, Hk, N, 128, 2)
    om, dqm, dkm, dvm = _run(q, k, v, do, "matched")
    os_, dqs, dks, dvs = _run(q, k, v, do, "stale")
    assert torch.equal(om, os_) and torch.equal(dvm, dvs)
    assert not torch.equal(dqm, dqs) and not torch.equal(dkm, dks), "the two deltas must give different dQ / dK"


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_plain_route_is_bitwise(mode):
    B, H, Hk, N = SHAPES["gqa"]
    q, k, v, do = _inputs(B, H, Hk, N, 128, 3)
    a = _run(q, k, v, do, mode)

    def plain(q, k, v, causal, mode):
        return dm.dm_attn_func_plain(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal, delta_mode=mode)
    b = _run(q, k, v, do, mode, fn=plain)
    for x, y, name in zip(a, b, ("O", "dQ", "dK", "dV")):
        assert torch.equal(x, y), f"{name}: the plain route differs from the API route ({mode})"


def test_flash_attn_alias_and_argument_checks():
    B, H, Hk, N = SHAPES["gqa"]
    q, k, v, do = (t.cuda() for t in _inputs(B, H, Hk, N, 128, 5))
    a = dm.flash_attn_func(q, k, v, causal=True)
    b = dm.dm_attn_func(q, k, v, causal=True, mode="matched")
    assert torch.equal(a, b)
    with pytest.raises(NotImplementedError):
        dm.flash_attn_func(q, k, v, dropout_p=0.1, causal=True)
    with pytest.raises(NotImplementedError):
        dm.flash_attn_func(q, k, v, causal=True, window_size=(128, 0))
    with pytest.raises(ValueError, match="causal"):
        dm.dm_attn_func(q, k, v, causal=False, mode="matched")
    with pytest.raises(ValueError, match="mode"):
        dm.dm_attn_func(q, k, v, causal=True, mode="other")
    with pytest.raises(ValueError, match="seqlen"):
        dm.dm_attn_func(q[:, :1000], k[:, :1000], v[:, :1000], causal=True)
    with pytest.raises(TypeError, match="bfloat16"):
        dm.dm_attn_func(q.float(), k.float(), v.float(), causal=True)


def _leaf(*ts):
    return [t.detach().clone().requires_grad_(True) for t in ts]


def _api_inputs(B=2, N=1024, H=8, Hk=2, D=128, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [torch.randn(B, N, h, D, generator=g).to("cuda", BF) for h in (H, Hk, Hk)]


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_backward_accepts_an_expanded_grad(mode):
    q, k, v = _api_inputs()
    a = _leaf(q, k, v)
    dm.dm_attn_func(*a, causal=True, mode=mode).sum().backward()
    b = _leaf(q, k, v)
    o = dm.dm_attn_func(*b, causal=True, mode=mode)
    o.backward(torch.ones_like(o))
    for x, y in zip(a, b):
        assert torch.equal(x.grad, y.grad)


@pytest.mark.parametrize("mode", ["matched", "stale"])
def test_non_contiguous_inputs_match_contiguous(mode):
    B, N, H, Hk, D = 2, 1024, 8, 2, 128
    g = torch.Generator(device="cpu").manual_seed(9)
    qkv = torch.randn(B, N, H + 2 * Hk, D, generator=g).to("cuda", BF)
    go = torch.randn(B, N, H, D, generator=g).to("cuda", BF)
    views = [t.detach().requires_grad_(True) for t in qkv.split([H, Hk, Hk], dim=2)]
    copies = [t.detach().contiguous().requires_grad_(True) for t in views]
    oa = dm.dm_attn_func(*views, causal=True, mode=mode)
    oa.backward(go)
    ob = dm.dm_attn_func(*copies, causal=True, mode=mode)
    ob.backward(go)
    assert torch.equal(oa, ob)
    for x, y in zip(views, copies):
        assert torch.equal(x.grad, y.grad)


@pytest.mark.parametrize("mode", ["matched", "stale"])
@pytest.mark.parametrize("groups,streams", [("kv", 1), ("head", 1), ("kv", 2)])
def test_head_group_split_is_bitwise(mode, groups, streams, monkeypatch):
    import delta_matching_b200.split as S
    q, k, v = _api_inputs(B=2, N=1024, H=8, Hk=2, seed=7)
    go = torch.randn(q.shape, generator=torch.Generator("cpu").manual_seed(8)).to("cuda", BF)

    def fb():
        a = _leaf(q, k, v)
        o = dm.dm_attn_func(*a, causal=True, mode=mode)
        o.backward(go)
        return [o.detach()] + [x.grad for x in a]
    monkeypatch.setattr(S, "_BWD_GROUPS", "off")
    ref = fb()
    monkeypatch.setattr(S, "_BWD_GROUPS", groups)
    monkeypatch.setattr(S, "_BWD_STREAMS", streams)
    monkeypatch.setattr(S, "_bwd_stream_pool", {})
    got = fb()
    torch.cuda.synchronize()
    for name, x, y in zip(("O", "dQ", "dK", "dV"), ref, got):
        assert torch.equal(x, y), f"{name}: split {groups} x{streams} differs from the single call ({mode})"


def test_flash_attn_func_signature_matches_flash_attention():
    flash_attn = pytest.importorskip("flash_attn")
    ours = list(inspect.signature(dm.flash_attn_func).parameters)
    theirs = list(inspect.signature(flash_attn.flash_attn_func).parameters)
    assert ours[:len(theirs)] == theirs


def _raises(exc, match, fn):
    with pytest.raises(exc, match=match):
        fn()


def test_input_errors_are_clear_exceptions():
    q, k, v = _api_inputs(B=1)
    f, fa = dm.dm_attn_func, dm.flash_attn_func
    _raises(ValueError, "causal", lambda: f(q, k, v))
    _raises(ValueError, "causal", lambda: fa(q, k, v))
    _raises(ValueError, "mode", lambda: f(q, k, v, causal=True, mode="match"))
    _raises(TypeError, "bfloat16", lambda: f(q.half(), k.half(), v.half(), causal=True))
    _raises(ValueError, "head_dim", lambda: f(q[..., :64], k[..., :64], v[..., :64], causal=True))
    _raises(ValueError, "256", lambda: f(q[:, :384], k[:, :384], v[:, :384], causal=True))
    _raises(ValueError, "nheads", lambda: f(q[:, :, :7], k, v, causal=True))
    _raises(ValueError, "seqlen", lambda: f(q[:, :512], k, v, causal=True))
    _raises(ValueError, "CUDA", lambda: f(q.cpu(), k.cpu(), v.cpu(), causal=True))
    _raises(ValueError, "4-D", lambda: f(q[0], k[0], v[0], causal=True))
    _raises(ValueError, "shape", lambda: f(q, k, v[:, :, :1], causal=True))
    _raises(NotImplementedError, "softmax_scale", lambda: f(q, k, v, causal=True, softmax_scale=0.05))
    _raises(NotImplementedError, "dropout", lambda: fa(q, k, v, 0.1, causal=True))
    _raises(NotImplementedError, "window", lambda: fa(q, k, v, causal=True, window_size=(128, 0)))
    _raises(NotImplementedError, "softcap", lambda: fa(q, k, v, causal=True, softcap=30.0))
    _raises(TypeError, "unexpected keyword", lambda: fa(q, k, v, causal=True, bogus=1))
    qb, kb, vb = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    _raises(ValueError, "causal", lambda: dm.dm_attn_func_bhnd(qb, kb, vb, causal=False, delta_mode="matched"))
    _raises(ValueError, "seqlen", lambda: dm.dm_attn_func_plain(qb[:, :, :384], kb[:, :, :384], vb[:, :, :384], causal=True))
    f(q, k, v, causal=True, softmax_scale=q.shape[-1] ** -0.5)


def test_library_checks_its_inputs():
    """The C ABI refuses invalid inputs with an error code and message (RuntimeError here) before any launch."""
    from delta_matching_b200 import _lib
    q, k, v = _api_inputs(B=1, N=512, H=4, Hk=2)
    Q8, Q8s, K8, K8s, V8, V8s = dm.ops.quant_qkv(q, k, v)
    o, lse = _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, 1, 4, 2, True)
    assert o.shape == q.shape and lse.dtype == torch.float32
    _raises(RuntimeError, "CUDA", lambda: _lib.fwd_fp8(Q8.cpu(), K8, V8, Q8s, K8s, V8s, 1, 4, 2, True))
    _raises(RuntimeError, "CUDA", lambda: _lib.fwd_fp8(Q8, K8, V8, Q8s.cpu(), K8s, V8s, 1, 4, 2, True))
    buf = torch.empty(Q8.numel() + 16, dtype=torch.uint8, device="cuda")
    shifted = buf[1:1 + Q8.numel()].view(torch.float8_e4m3fn).view(Q8.shape)
    _raises(RuntimeError, "aligned", lambda: _lib.fwd_fp8(shifted, K8, V8, Q8s, K8s, V8s, 1, 4, 2, True))
    _raises(RuntimeError, "seqlen", lambda: _lib.delta_fp8(Q8[:, :192], K8, V8, Q8, Q8s, K8s, V8s, Q8s, lse, 1, 4, 2, True))
    _raises(RuntimeError, "nheads", lambda: _lib.fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, 1, 4, 3, True))
    assert _lib.device_status() == 0


def test_kernel_version_reports_the_loaded_library():
    import os
    s = dm.kernel_version()
    assert len(s["code_sha"]) == 12 and s["numerics"]["128"] and s["library"] and os.path.isfile(s["library"]) and s["bf16_dp"] is False


def test_torch_compile_matches_eager():
    q, k, v = _api_inputs(B=1, N=1024, H=8, Hk=2, seed=11)
    go = torch.randn(1, 1024, 8, 128, generator=torch.Generator("cpu").manual_seed(12)).to("cuda", BF)

    def f(q, k, v):
        return dm.dm_attn_func(q * 1.0, k, v, causal=True, mode="matched")
    qa, ka, va = _leaf(q, k, v)
    oa = torch.compile(f)(qa, ka, va)
    oa.backward(go)
    qb, kb, vb = _leaf(q, k, v)
    ob = f(qb, kb, vb)
    ob.backward(go)
    assert torch.equal(oa, ob) and torch.equal(qa.grad, qb.grad) and torch.equal(ka.grad, kb.grad) and torch.equal(va.grad, vb.grad)


def test_cuda_graph_capture_of_the_forward():
    q, k, v = _api_inputs(B=1, N=1024, H=8, Hk=2, seed=12)
    dm.dm_attn_func(q, k, v, causal=True)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        o = dm.dm_attn_func(q, k, v, causal=True)
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(o, dm.dm_attn_func(q, k, v, causal=True))


def test_logit_range_regime():
    """q and k scaled by 3 and by 10 (BASELINE config 3's probe): the forward error grows as the reference documents
    (about 0.12 and 0.28) and everything stays finite."""
    q, k, v, do = _inputs(1, 4, 2, 1024, 128, 21)
    for scale, bound in ((3.0, 0.2), (10.0, 0.45)):
        qs, ks = (q.float() * scale).to(BF), (k.float() * scale).to(BF)
        ref = O.fp32_reference(qs, ks, v, do)
        got = _run(qs, ks, v, do, "matched")
        assert all(torch.isfinite(t.float()).all() for t in got)
        assert O.rel(got[0].cpu(), ref[0]) < bound
