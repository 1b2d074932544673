"""ctypes binding of libdm_b200.so (the C ABI declared in include/dm_b200.h) and thin tensor-level wrappers.

The library is the only compute path: if it is missing or fails to load, every call raises (there is no fallback).
Wrappers allocate outputs with torch (the caching allocator, the tensors' device) and pass raw pointers plus the
current CUDA stream of that device; a non-zero return code becomes a RuntimeError carrying the library's message.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_LIB_PATH = None

E4M3 = torch.float8_e4m3fn


class DmShape(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("Hk", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("causal", C.c_int32)]


class DmStrides(C.Structure):
    _fields_ = [("b", C.c_int64), ("n", C.c_int64), ("h", C.c_int64)]


class DmCp(C.Structure):
    """Row map of a rank's Q-side tensors under a sequence split: nq local rows = half_blocks 128-row blocks starting at
    global block off0, then the rest starting at global block off1."""
    _fields_ = [("nq", C.c_int32), ("half_blocks", C.c_int32), ("off0", C.c_int32), ("off1", C.c_int32)]


_ERR = (C.c_char_p, C.c_size_t)
_P = C.c_void_p
_SIGNATURES = {
    "dm_build_info": (C.c_char_p, []),
    "dm_kmean_scratch_bytes": (C.c_size_t, [C.c_int32] * 4),
    "dm_kmean": (C.c_int, [_P, DmStrides, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, *_ERR]),
    "dm_kmean_noalloc_max_bytes": (C.c_size_t, []),
    "dm_kmean_noalloc": (C.c_int, [_P, DmStrides, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_quant": (C.c_int, [C.c_int32, _P, DmStrides, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, *_ERR]),
    "dm_quant_do": (C.c_int, [_P, DmStrides, _P, DmStrides, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, *_ERR]),
    "dm_fwd_fp8": (C.c_int, [_P] * 6 + [DmShape, C.c_int32, C.c_int32, _P, _P, _P, *_ERR]),
    "dm_delta_fp8": (C.c_int, [_P] * 9 + [DmShape, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_bwd_workspace_bytes": (C.c_int, [DmShape, C.c_int32, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "dm_bwd_fp8_pass1": (C.c_int, [_P] * 10 + [DmShape, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, *_ERR]),
    "dm_bwd_fp8_pass2": (C.c_int, [_P] * 3 + [DmShape, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_gqa_fold": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_attn_forward": (C.c_int, [_P, DmStrides, _P, DmStrides, _P, DmStrides, DmShape] + [_P] * 10 + [_P, *_ERR]),
    "dm_attn_backward": (C.c_int, [_P, DmStrides, _P, DmStrides] + [_P] * 7 + [DmShape, C.c_int32] + [_P] * 10 + [_P, *_ERR]),
    "dm_bwd_dbg_rowsum": (C.c_int, [_P] * 10 + [DmShape, _P, _P, _P, *_ERR]),
    "dm_probe_mma": (C.c_int, [_P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, *_ERR]),
    "dm_device_status": (C.c_int, [C.POINTER(C.c_int32), *_ERR]),
    "dm_selftest_wait_timeout": (C.c_int, [_P, _P, *_ERR]),
    "dm_init": (C.c_int, [*_ERR]),
    "dm_register_pool_ok": (C.c_int, [C.c_int32] * 3),
    "dm_quant_qv_kpartials": (C.c_int, [_P, DmStrides, _P, DmStrides, _P, DmStrides, DmShape] + [_P] * 5 + [_P, *_ERR]),
    "dm_kmean_partials": (C.c_int, [_P, DmStrides, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_kmean_fold": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_fold_f32": (C.c_int, [_P, C.c_int64, C.c_int32, C.c_int64, C.c_int32, _P, _P, *_ERR]),
    "dm_fold_to_owners": (C.c_int, [_P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_fwd_fp8_cp": (C.c_int, [_P] * 6 + [DmShape, DmCp, C.c_int32, C.c_int32, _P, _P, _P, *_ERR]),
    "dm_delta_fp8_cp": (C.c_int, [_P] * 9 + [DmShape, DmCp, C.c_int32, C.c_int32, _P, _P, *_ERR]),
    "dm_bwd_workspace_bytes_cp": (C.c_int, [DmShape, DmCp, C.c_int32, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "dm_bwd_fp8_pass1_cp": (C.c_int, [_P] * 10 + [DmShape, DmCp, C.c_int32, C.c_int32, C.c_int32, _P, _P, _P, _P, _P, *_ERR]),
    "dm_bwd_fp8_pass2_cp": (C.c_int, [_P] * 3 + [DmShape, DmCp, C.c_int32, C.c_int32, _P, _P, *_ERR]),
}
EXPORTS = tuple(_SIGNATURES)


def library_path() -> str:
    """The shared library this package loads: DM_SO if set, else the in-tree libdm_b200.so."""
    so = os.environ.get("DM_SO")
    if so:
        if not os.path.isfile(so):
            raise RuntimeError(f"DM_SO={so!r} does not exist")
        return so
    so = os.path.join(_HERE, "libdm_b200.so")
    if not os.path.isfile(so):
        raise RuntimeError("delta_matching_b200: libdm_b200.so is not built; run `python -m delta_matching_b200.build` "
                           "in the checkout, or point DM_SO at a built library")
    return so


def lib():
    """Load the library on first use and bind the signatures; missing symbols are an error."""
    global _LIB, _LIB_PATH
    if _LIB is None:
        path = library_path()
        handle = C.CDLL(path)
        for name, (res, args) in _SIGNATURES.items():
            try:
                fn = getattr(handle, name)
            except AttributeError as e:
                raise RuntimeError(f"delta_matching_b200: {path} does not export {name}; rebuild the library") from e
            fn.restype = res
            fn.argtypes = args
        _LIB, _LIB_PATH = handle, path
    return _LIB


def loaded_library():
    return _LIB_PATH


def build_info() -> str:
    return lib().dm_build_info().decode()


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _call(name, *args):
    err = C.create_string_buffer(512)
    rc = getattr(lib(), name)(*args, err, len(err))
    if rc != 0:
        raise RuntimeError(f"delta_matching_b200.{name}: {err.value.decode(errors='replace')} (code {rc})")


def _strides_bnhd(t):
    """Element strides (batch, seqlen, head) of a (B, N, H, D) view with unit head_dim stride."""
    return DmStrides(t.stride(0), t.stride(1), t.stride(2))


def _shape(B, H, Hk, N, D, causal):
    return DmShape(B, H, Hk, N, D, 1 if causal else 0)


def blocks(D: int):
    """Rows per Q / dO scale and keys per K / V scale: (64, 32) at head_dim 256, (128, 64) at head_dim 128."""
    return (64, 32) if D >= 256 else (128, 64)


def _device_of(*ts):
    """The CUDA device the call runs on: the first CUDA tensor's; host tensors are left for the library to refuse."""
    for t in ts:
        if t is not None and t.is_cuda:
            return t.device
    return torch.device("cuda", torch.cuda.current_device())


def _unit_lane(t):
    return t if t.stride(-1) == 1 else t.contiguous()


# ----------------------------------------------------------------------------------------------------------------------
# tensor-level wrappers; all take flash-layout (B, N, heads, D) bf16 views and code tensors [B*heads, N, D]
# ----------------------------------------------------------------------------------------------------------------------
def kmean(k_bnhd):
    B, N, Hk, D = k_bnhd.shape
    k_bnhd = _unit_lane(k_bnhd)
    with torch.cuda.device(k_bnhd.device):
        km = torch.empty(B * Hk, D, device=k_bnhd.device, dtype=torch.float32)
        scratch = torch.empty(lib().dm_kmean_scratch_bytes(B, Hk, N, D) // 4, device=k_bnhd.device, dtype=torch.float32)
        _call("dm_kmean", _ptr(k_bnhd), _strides_bnhd(k_bnhd), B, Hk, N, D, _ptr(km), _ptr(scratch), _stream(k_bnhd.device))
    return km


def kmean_noalloc(k_bnhd, out):
    """The K mean through the entry point that allocates nothing: for callers whose own arena owns all device memory (or
    that cannot take cudaMalloc's device-wide synchronisation), the partial sums live in a 4 MiB array inside the library.
    `out` is the caller's [B*Hk, D] fp32 result tensor; the input must already have a unit head_dim stride.  Calls on one
    device share that array, so do not let two of them overlap on the GPU."""
    B, N, Hk, D = k_bnhd.shape
    with torch.cuda.device(k_bnhd.device):
        _call("dm_kmean_noalloc", _ptr(k_bnhd), _strides_bnhd(k_bnhd), B, Hk, N, D, _ptr(out), _stream(k_bnhd.device))
    return out


def quant(mode, x_bnhd, km=None):
    """mode 0 = Q, 1 = K (needs km), 2 = V.  Returns (codes [B*heads, N, D] e4m3, scales [B*heads, N/blk] fp32)."""
    B, N, Hh, D = x_bnhd.shape
    x_bnhd = _unit_lane(x_bnhd)
    blk = blocks(D)[0 if mode == 0 else 1]
    with torch.cuda.device(x_bnhd.device):
        codes = torch.empty(B * Hh, N, D, device=x_bnhd.device, dtype=E4M3)
        scales = torch.empty(B * Hh, max(N // blk, 1), device=x_bnhd.device, dtype=torch.float32)
        _call("dm_quant", mode, _ptr(x_bnhd), _strides_bnhd(x_bnhd), B, Hh, N, D, _ptr(km), _ptr(codes), _ptr(scales),
              _stream(x_bnhd.device))
    return codes, scales


def quant_do(dO_bnhd, o_bnhd=None):
    """dO codes / scales and, when o is given, the stale delta [B*H, N] fp32."""
    B, N, H, D = dO_bnhd.shape
    dO_bnhd = _unit_lane(dO_bnhd)
    with torch.cuda.device(dO_bnhd.device):
        codes = torch.empty(B * H, N, D, device=dO_bnhd.device, dtype=E4M3)
        scales = torch.empty(B * H, max(N // blocks(D)[0], 1), device=dO_bnhd.device, dtype=torch.float32)
        delta = None
        os_ = DmStrides(0, 0, 0)
        if o_bnhd is not None:
            o_bnhd = _unit_lane(o_bnhd)
            delta = torch.empty(B * H, N, device=dO_bnhd.device, dtype=torch.float32)
            os_ = _strides_bnhd(o_bnhd)
        _call("dm_quant_do", _ptr(dO_bnhd), _strides_bnhd(dO_bnhd), _ptr(o_bnhd), os_, B, H, N, D, _ptr(codes), _ptr(scales),
              _ptr(delta), _stream(dO_bnhd.device))
    return codes, scales, delta


def fwd_fp8(Q8, K8, V8, Q8s, K8s, V8s, B, H, Hk, causal, h0=0, hcount=None, out=None, cp=None):
    """O (B, N, H, D) bf16 and LSE [B*H, N] fp32; with a head range only those heads are written.  With a row map `cp`
    (sequence split) Q8 holds the rank's nq local rows, K8 / V8 the whole sequence, and O / LSE are local."""
    BH, nq, D = Q8.shape
    N = nq if cp is None else K8.shape[1]      # whole sequence: the Q-side tensors carry it
    hcount = H if hcount is None else hcount
    dev = _device_of(Q8, K8, V8)
    with torch.cuda.device(dev):
        if out is None:
            o = torch.empty(B, nq, H, D, device=dev, dtype=torch.bfloat16)
            lse = torch.empty(B * H, nq, device=dev, dtype=torch.float32)
        else:
            o, lse = out
        if cp is None:
            _call("dm_fwd_fp8", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _shape(B, H, Hk, N, D, causal), h0,
                  hcount, _ptr(o), _ptr(lse), _stream(dev))
        else:
            _call("dm_fwd_fp8_cp", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _shape(B, H, Hk, N, D, causal), cp,
                  h0, hcount, _ptr(o), _ptr(lse), _stream(dev))
    return o, lse


def delta_fp8(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, B, H, Hk, causal, h0=0, hcount=None, out=None, cp=None):
    BH, nq, D = Q8.shape
    N = nq if cp is None else K8.shape[1]      # whole sequence: the Q-side tensors carry it
    hcount = H if hcount is None else hcount
    dev = _device_of(Q8, K8, V8)
    with torch.cuda.device(dev):
        delta = torch.empty(B * H, nq, device=dev, dtype=torch.float32) if out is None else out
        if cp is None:
            _call("dm_delta_fp8", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(dO8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _ptr(dO8s), _ptr(lse),
                  _shape(B, H, Hk, N, D, causal), h0, hcount, _ptr(delta), _stream(dev))
        else:
            _call("dm_delta_fp8_cp", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(dO8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _ptr(dO8s), _ptr(lse),
                  _shape(B, H, Hk, N, D, causal), cp, h0, hcount, _ptr(delta), _stream(dev))
    return delta


def bwd_workspace_bytes(B, H, Hk, N, D, causal, hcount, cp=None):
    a, b = C.c_size_t(0), C.c_size_t(0)
    if cp is None:
        rc = lib().dm_bwd_workspace_bytes(_shape(B, H, Hk, N, D, causal), hcount, C.byref(a), C.byref(b))
    else:
        rc = lib().dm_bwd_workspace_bytes_cp(_shape(B, H, Hk, N, D, causal), cp, hcount, C.byref(a), C.byref(b))
    if rc != 0:
        raise RuntimeError(f"delta_matching_b200.dm_bwd_workspace_bytes failed (code {rc})")
    return a.value, b.value


def bwd_pass1(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal, h0=0, hcount=None, out=None, ws=None, cp=None,
              out_fp32=False):
    """dK, dV (B, N, H, D) per query head (bf16, or fp32 partials with out_fp32) plus the dS' / psi workspace for pass 2.
    With a row map `cp` the Q-side inputs and the workspace hold the rank's local rows; dK / dV span the whole sequence."""
    BH, nq, D = Q8.shape
    N = nq if cp is None else K8.shape[1]      # whole sequence: the Q-side tensors carry it
    hcount = H if hcount is None else hcount
    dev = _device_of(Q8, K8, V8)
    with torch.cuda.device(dev):
        if out is None:
            dt = torch.float32 if out_fp32 else torch.bfloat16
            dk = torch.empty(B, N, H, D, device=dev, dtype=dt)
            dv = torch.empty(B, N, H, D, device=dev, dtype=dt)
        else:
            dk, dv = out
        if ws is None:
            nb_ds, nb_psi = bwd_workspace_bytes(B, H, Hk, N, D, causal, hcount, cp)
            ws = (torch.empty(nb_ds, device=dev, dtype=torch.uint8), torch.empty(nb_psi // 4, device=dev, dtype=torch.float32))
        if cp is None and not out_fp32:
            _call("dm_bwd_fp8_pass1", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(dO8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _ptr(dO8s), _ptr(lse),
                  _ptr(delta), _shape(B, H, Hk, N, D, causal), h0, hcount, _ptr(dk), _ptr(dv), _ptr(ws[0]), _ptr(ws[1]), _stream(dev))
        else:
            cpm = cp if cp is not None else DmCp(N, N // 128, 0, 0)
            _call("dm_bwd_fp8_pass1_cp", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(dO8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _ptr(dO8s),
                  _ptr(lse), _ptr(delta), _shape(B, H, Hk, N, D, causal), cpm, h0, hcount, 1 if out_fp32 else 0, _ptr(dk), _ptr(dv),
                  _ptr(ws[0]), _ptr(ws[1]), _stream(dev))
    return dk, dv, ws


def bwd_pass2(ws, K8, B, H, Hk, N, D, causal, h0=0, hcount=None, out=None, cp=None):
    hcount = H if hcount is None else hcount
    dev = K8.device
    nq = N if cp is None else cp.nq
    with torch.cuda.device(dev):
        dq = torch.empty(B, nq, H, D, device=dev, dtype=torch.bfloat16) if out is None else out
        if cp is None:
            _call("dm_bwd_fp8_pass2", _ptr(ws[0]), _ptr(ws[1]), _ptr(K8), _shape(B, H, Hk, N, D, causal), h0, hcount, _ptr(dq),
                  _stream(dev))
        else:
            _call("dm_bwd_fp8_pass2_cp", _ptr(ws[0]), _ptr(ws[1]), _ptr(K8), _shape(B, H, Hk, N, D, causal), cp, h0, hcount, _ptr(dq),
                  _stream(dev))
    return dq


def kmean_partials(k_bnhd):
    """Per-64-row-chunk column sums [B*Hk, N_local/64, D] fp32 of a rank's local keys."""
    B, N, Hk, D = k_bnhd.shape
    k_bnhd = _unit_lane(k_bnhd)
    with torch.cuda.device(k_bnhd.device):
        part = torch.empty(B * Hk, N // 64, D, device=k_bnhd.device, dtype=torch.float32)
        _call("dm_kmean_partials", _ptr(k_bnhd), _strides_bnhd(k_bnhd), B, Hk, N, D, _ptr(part), _stream(k_bnhd.device))
    return part


def kmean_fold(partials, B, Hk, N, D):
    """The K mean [B*Hk, D] from all chunk sums of the sequence, [B*Hk, N/64, D] in sequence order."""
    partials = partials.contiguous()
    with torch.cuda.device(partials.device):
        km = torch.empty(B * Hk, D, device=partials.device, dtype=torch.float32)
        _call("dm_kmean_fold", _ptr(partials), B, Hk, N, D, _ptr(km), _stream(partials.device))
    return km


def fold_f32(x, count_dim, out_dtype=torch.float32):
    """Sum a contiguous fp32 tensor over dimension `count_dim` in ascending order; the result (that dimension removed) is
    rounded once to out_dtype (fp32 or bf16)."""
    assert x.dtype == torch.float32 and out_dtype in (torch.float32, torch.bfloat16)
    x = x.contiguous()
    shape = list(x.shape)
    outer = 1
    for s_ in shape[:count_dim]:
        outer *= s_
    inner = 1
    for s_ in shape[count_dim + 1:]:
        inner *= s_
    with torch.cuda.device(x.device):
        out = torch.empty(shape[:count_dim] + shape[count_dim + 1:], device=x.device, dtype=out_dtype)
        _call("dm_fold_f32", _ptr(x), outer, shape[count_dim], inner, 1 if out_dtype == torch.bfloat16 else 0, _ptr(out),
              _stream(x.device))
    return out


def fold_to_owners(dkp, dvp, Hk, world):
    """fp32 partials (B, N, H, D) of dK and dV over all keys -> [world, 2, B, N / world, Hk, D] fp32: summed over the query
    heads of each KV group in head order, slice d holding the rows rank d owns under the zig-zag split."""
    assert dkp.dtype == torch.float32 and dkp.is_contiguous() and dvp.is_contiguous() and dkp.shape == dvp.shape
    B, N, H, D = dkp.shape
    with torch.cuda.device(dkp.device):
        out = torch.empty(world, 2, B, N // world, Hk, D, device=dkp.device, dtype=torch.float32)
        _call("dm_fold_to_owners", _ptr(dkp), _ptr(dvp), B, N, H, Hk, D, world, _ptr(out), _stream(dkp.device))
    return out


def gqa_fold(x_bnhd, Hk):
    B, N, H, D = x_bnhd.shape
    if H == Hk:
        return x_bnhd
    x_bnhd = x_bnhd.contiguous()
    with torch.cuda.device(x_bnhd.device):
        out = torch.empty(B, N, Hk, D, device=x_bnhd.device, dtype=torch.bfloat16)
        _call("dm_gqa_fold", _ptr(x_bnhd), B, N, H, Hk, D, _ptr(out), _stream(x_bnhd.device))
    return out


def attn_forward(q, k, v, causal):
    """Quantizers + forward in one library call.  q (B, N, H, D), k / v (B, N, Hk, D) bf16 views (unit head_dim stride).
    Returns O, LSE, Q8, Q8s, K8, K8s, V8, V8s."""
    B, N, H, D = q.shape
    Hk = k.shape[2]
    q, k, v = _unit_lane(q), _unit_lane(k), _unit_lane(v)
    dev = q.device
    rq, rk = blocks(D)
    f32, bf = torch.float32, torch.bfloat16
    with torch.cuda.device(dev):
        e = lambda shape, dt: torch.empty(shape, device=dev, dtype=dt)
        Q8, K8, V8 = e((B * H, N, D), E4M3), e((B * Hk, N, D), E4M3), e((B * Hk, N, D), E4M3)
        Q8s, K8s, V8s = e((B * H, N // rq), f32), e((B * Hk, N // rk), f32), e((B * Hk, N // rk), f32)
        km, part = e((B * Hk, D), f32), e((B * Hk * (N // 64) * D,), f32)
        O, lse = e((B, N, H, D), bf), e((B * H, N), f32)
        _call("dm_attn_forward", _ptr(q), _strides_bnhd(q), _ptr(k), _strides_bnhd(k), _ptr(v), _strides_bnhd(v),
              _shape(B, H, Hk, N, D, causal), _ptr(Q8), _ptr(Q8s), _ptr(K8), _ptr(K8s), _ptr(V8), _ptr(V8s), _ptr(km), _ptr(part),
              _ptr(O), _ptr(lse), _stream(dev))
    return O, lse, Q8, Q8s, K8, K8s, V8, V8s


def attn_backward(dO, O, lse, Q8, Q8s, K8, K8s, V8, V8s, B, H, Hk, causal, matched):
    """dO quantizer + pass 0 / 1 / 2 + GQA fold for all heads in one library call.  Returns dq (B, N, H, D), dk / dv
    (B, N, Hk, D) bf16."""
    BH, N, D = Q8.shape
    dO = _unit_lane(dO)
    dev = Q8.device
    f32, bf = torch.float32, torch.bfloat16
    with torch.cuda.device(dev):
        e = lambda shape, dt: torch.empty(shape, device=dev, dtype=dt)
        dO8, dO8s, delta = e((BH, N, D), E4M3), e((BH, N // blocks(D)[0]), f32), e((BH, N), f32)
        nb_ds, nb_psi = bwd_workspace_bytes(B, H, Hk, N, D, causal, H)
        ws_ds, ws_psi = e((nb_ds,), torch.uint8), e((nb_psi // 4,), f32)
        dq = e((B, N, H, D), bf)
        dk, dv = e((B, N, Hk, D), bf), e((B, N, Hk, D), bf)
        dkh = e((B, N, H, D), bf) if Hk < H else None
        dvh = e((B, N, H, D), bf) if Hk < H else None
        os_ = _strides_bnhd(O) if not matched else DmStrides(0, 0, 0)
        _call("dm_attn_backward", _ptr(dO), _strides_bnhd(dO), _ptr(O) if not matched else C.c_void_p(0), os_, _ptr(Q8), _ptr(K8),
              _ptr(V8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _ptr(lse), _shape(B, H, Hk, N, D, causal), 1 if matched else 0, _ptr(dO8),
              _ptr(dO8s), _ptr(delta), _ptr(dkh), _ptr(dvh), _ptr(ws_ds), _ptr(ws_psi), _ptr(dq), _ptr(dk), _ptr(dv), _stream(dev))
    return dq, dk, dv


def bwd_dbg_rowsum(Q8, K8, V8, dO8, Q8s, K8s, V8s, dO8s, lse, delta, B, H, Hk, causal):
    BH, N, D = Q8.shape
    dev = _device_of(Q8, K8, V8)
    with torch.cuda.device(dev):
        rows = torch.empty(B * H, N, device=dev, dtype=torch.float32)
        rabs = torch.empty(B * H, N, device=dev, dtype=torch.float32)
        _call("dm_bwd_dbg_rowsum", _ptr(Q8), _ptr(K8), _ptr(V8), _ptr(dO8), _ptr(Q8s), _ptr(K8s), _ptr(V8s), _ptr(dO8s), _ptr(lse),
              _ptr(delta), _shape(B, H, Hk, N, D, causal), _ptr(rows), _ptr(rabs), _stream(dev))
    return rows, rabs


def probe_mma(a_tile, b_tile, a_mn, b_mn, n_cols=128, via_st=0):
    """via_st: 0 = A by TMA, 1 = A written by threads into the swizzled tile (and echoed back by a TMA store), 2 / 3 / 4 = A
    in tensor memory (contiguous / one K step per 32 columns / overwritten by a second product, returned as rows 128..255)."""
    dev = a_tile.device
    with torch.cuda.device(dev):
        c = torch.empty(256 if int(via_st) == 4 else 128, n_cols, device=dev, dtype=torch.float32)
        echo = torch.zeros(128, 128, device=dev, dtype=torch.uint8)
        _call("dm_probe_mma", _ptr(a_tile), _ptr(b_tile), int(a_mn), int(b_mn), n_cols, int(via_st), _ptr(c), _ptr(echo), _stream(dev))
    return c, echo


def init(device=None) -> None:
    """One-time set-up of a device (status word, kernel attributes, register-pool checks): call before capturing CUDA graphs."""
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _call("dm_init")


def selftest_wait_timeout(device=None):
    """Runs the bounded-wait self-test kernel; returns the two per-warp flags (1 = the wait was satisfied)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        out = torch.full((2,), -1, device=dev, dtype=torch.int32)
        _call("dm_selftest_wait_timeout", _ptr(out), _stream(dev))
    return out


def device_status(device=None) -> int:
    """Synchronise the device and read-and-clear the status word the kernels' bounded waits write (0 = clean)."""
    v = C.c_int32(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _call("dm_device_status", C.byref(v))
    return v.value
