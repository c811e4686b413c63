"""ctypes binding of the CPU oracle (oracle/liboracle.so) for the tests.

Only tests, the smoke check and the benchmark's CPU-baseline leg load this.
"""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent.parent / "oracle"

F32, F16, BF16 = 0, 1, 2
_NP_DT = {F32: np.float32, F16: np.float16, BF16: np.uint16}


class AttnParams(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "q_batch_stride", "k_batch_stride", "v_batch_stride", "o_batch_stride",
        "q_row_stride", "k_row_stride", "v_row_stride", "o_row_stride",
        "q_head_stride", "k_head_stride", "v_head_stride", "o_head_stride",
        "b", "h", "h_k", "d", "seqlen_q", "seqlen_k")] + [
        ("softmax_scale", C.c_float), ("window_left", C.c_int64), ("window_right", C.c_int64)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        so = ORACLE_DIR / "liboracle.so"
        if not so.exists() or so.stat().st_mtime < (ORACLE_DIR / "oracle.cc").stat().st_mtime:
            subprocess.check_call(["make", "-C", str(ORACLE_DIR), "liboracle.so"])
        _lib = C.CDLL(str(so))
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return C.c_void_p(a.ctypes.data)


def dtype_code(a):
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float16:
        return F16
    if a.dtype == np.uint16:
        return BF16
    raise TypeError(a.dtype)


def f32_to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_bf16(_p(x), _p(out), C.c_int64(x.size))
    return out


def bf16_to_f32(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, np.float32)
    lib().oracle_bf16_to_f32(_p(x), _p(out), C.c_int64(x.size))
    return out


def to_f32(a):
    return bf16_to_f32(a) if a.dtype == np.uint16 else a.astype(np.float32)


def reduce_abc(shape, dims):
    """A, B, C collapse of reduce_impl.h:28-59 (size-1 dims are dropped from
    `dims`; the rest must be consecutive)."""
    dims = sorted(d for d in dims if shape[d] != 1)
    if not dims:
        return 0, 0, int(np.prod(shape, dtype=np.int64))
    assert all(b - a == 1 for a, b in zip(dims, dims[1:])), "non-consecutive dims"
    A = int(np.prod(shape[:dims[0]], dtype=np.int64))
    B = int(np.prod([shape[d] for d in dims], dtype=np.int64))
    Cc = int(np.prod(shape[dims[-1] + 1:], dtype=np.int64))
    return A, B, Cc


def reduce(op, x, A, B, Cc):
    x = np.ascontiguousarray(x)
    if A == 0 and B == 0:  # nothing to reduce: the reference copies (reduce_impl.h:70-73)
        return x.reshape(-1).copy()
    out = np.empty(A * Cc, x.dtype)
    fn = lib().oracle_reduce_sum if op == "sum" else lib().oracle_reduce_max
    rc = fn(dtype_code(x), _p(x), _p(out), C.c_int64(A), C.c_int64(B), C.c_int64(Cc))
    assert rc == 0
    return out


def reduce_sum_f64(x, A, B, Cc):
    x = np.ascontiguousarray(x)
    out = np.empty(A * Cc, np.float64)
    rc = lib().oracle_reduce_sum_f64(dtype_code(x), _p(x), _p(out), C.c_int64(A), C.c_int64(B), C.c_int64(Cc))
    assert rc == 0
    return out


def index_select(x, idx, dim):
    x = np.ascontiguousarray(x)
    idx = np.ascontiguousarray(idx)
    shape = x.shape
    A = int(np.prod(shape[:dim], dtype=np.int64))
    IB = shape[dim]
    Cc = int(np.prod(shape[dim + 1:], dtype=np.int64))
    OB = idx.shape[0]
    out = np.empty(shape[:dim] + (OB,) + shape[dim + 1:], x.dtype)
    rc = lib().oracle_index_select(x.itemsize, idx.itemsize, _p(x), _p(idx), _p(out),
                                   C.c_int64(A), C.c_int64(IB), C.c_int64(OB), C.c_int64(Cc))
    return out, rc


def index_put_add(x, idx, upd, dim=0):
    x = np.ascontiguousarray(x)
    upd = np.ascontiguousarray(upd)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    rows = int(np.prod(x.shape[:dim + 1], dtype=np.int64))
    feat = int(np.prod(x.shape[dim + 1:], dtype=np.int64))
    out = np.empty_like(x)
    rc = lib().oracle_index_put_add(dtype_code(x), _p(x), _p(idx), _p(upd), _p(out),
                                    C.c_int64(rows), C.c_int64(idx.size), C.c_int64(feat))
    return out, rc


def index_put_add_seq_f32(x, idx, upd, dim=0):
    x = np.ascontiguousarray(x, dtype=np.float32)
    upd = np.ascontiguousarray(upd, dtype=np.float32)
    idx = np.ascontiguousarray(idx, dtype=np.int64)
    rows = int(np.prod(x.shape[:dim + 1], dtype=np.int64))
    feat = int(np.prod(x.shape[dim + 1:], dtype=np.int64))
    out = np.empty_like(x)
    rc = lib().oracle_index_put_add_seq_f32(_p(x), _p(idx), _p(upd), _p(out),
                                            C.c_int64(rows), C.c_int64(idx.size), C.c_int64(feat))
    return out, rc


def transpose(x, perm):
    x = np.ascontiguousarray(x)
    shape = (C.c_int64 * x.ndim)(*x.shape)
    p = (C.c_int64 * x.ndim)(*perm)
    out = np.empty(tuple(x.shape[i] for i in perm), x.dtype)
    rc = lib().oracle_transpose(x.itemsize, _p(x), _p(out), x.ndim, shape, p)
    assert rc == 0
    return out


def attn_params(b, sq, sk, h, hk, d, scale, causal=True, window=(-1, -1)):
    """Contiguous [B, S, H, D] layout, as the reference's custom call gets it."""
    p = AttnParams()
    p.q_batch_stride = p.o_batch_stride = sq * h * d
    p.k_batch_stride = p.v_batch_stride = sk * hk * d
    p.q_row_stride = p.o_row_stride = h * d
    p.k_row_stride = p.v_row_stride = hk * d
    p.q_head_stride = p.k_head_stride = p.v_head_stride = p.o_head_stride = d
    p.b, p.h, p.h_k, p.d, p.seqlen_q, p.seqlen_k = b, h, hk, d, sq, sk
    p.softmax_scale = scale
    p.window_left = window[0]
    p.window_right = 0 if causal else window[1]
    return p


def flash_attn_fwd(q, k, v, scale, causal=True, round_p=False, window=(-1, -1)):
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    q, k, v = (np.ascontiguousarray(t) for t in (q, k, v))
    p = attn_params(b, sq, sk, h, hk, d, scale, causal, window)
    out = np.empty_like(q)
    lse = np.empty((b, h, sq), np.float32)
    rc = lib().oracle_flash_attn_fwd(dtype_code(q), _p(q), _p(k), _p(v), _p(out), _p(lse),
                                     C.byref(p), int(round_p))
    assert rc == 0
    return out, lse


class KvNewStrides(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "knew_batch_stride", "vnew_batch_stride", "knew_row_stride", "vnew_row_stride",
        "knew_head_stride", "vnew_head_stride", "seqlen_knew")]


def flash_attn_kvcache(q, kcache, vcache, knew, vnew, seqlens_k, scale, causal=True, window=(-1, -1)):
    """One decode step on contiguous arrays.  kcache / vcache are updated in place (pass copies).
    Returns (out, lse)."""
    b, sq, h, d = q.shape
    cap, hk = kcache.shape[1], kcache.shape[2]
    for t in (q, kcache, vcache):
        assert t.flags.c_contiguous
    p = attn_params(b, sq, cap, h, hk, d, scale, causal, window)
    n = KvNewStrides()
    if knew is not None:
        knew, vnew = np.ascontiguousarray(knew), np.ascontiguousarray(vnew)
        s_new = knew.shape[1]
        n.knew_batch_stride = n.vnew_batch_stride = s_new * hk * d
        n.knew_row_stride = n.vnew_row_stride = hk * d
        n.knew_head_stride = n.vnew_head_stride = d
        n.seqlen_knew = s_new
    if seqlens_k is not None:
        seqlens_k = np.ascontiguousarray(seqlens_k, dtype=np.int32)
    out = np.empty_like(q)
    lse = np.empty((b, h, sq), np.float32)
    ptr = lambda a: _p(a) if a is not None else None
    rc = lib().oracle_flash_attn_kvcache(dtype_code(q), _p(q), _p(kcache), _p(vcache), ptr(knew), ptr(vnew),
                                         ptr(seqlens_k), _p(out), _p(lse), C.byref(p), C.byref(n))
    assert rc == 0
    return out, lse


def flash_attn_bwd(dout, q, k, v, out, lse, scale, causal=True, window=(-1, -1)):
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    dout, q, k, v, out = (np.ascontiguousarray(t) for t in (dout, q, k, v, out))
    lse = np.ascontiguousarray(lse, dtype=np.float32)
    p = attn_params(b, sq, sk, h, hk, d, scale, causal, window)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    rc = lib().oracle_flash_attn_bwd(dtype_code(q), _p(dout), _p(q), _p(k), _p(v), _p(out), _p(lse),
                                     _p(dq), _p(dk), _p(dv), C.byref(p))
    assert rc == 0
    return dq, dk, dv
