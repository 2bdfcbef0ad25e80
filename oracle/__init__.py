"""ctypes front end of the CPU oracle (oracle/oracle.c).

Test infrastructure only: nothing in the shipped package imports this module.
It may be used by tests/, by the smoke check and by the benchmark's CPU
baseline leg.  Every function takes and returns float32 numpy arrays; the
arithmetic inside is float64 (see oracle.c for the reference citations).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i64 = ctypes.c_int64
_dbl = ctypes.c_double


def build(force: bool = False) -> str:
    """Compile oracle.c into liboracle.so next to it (gcc + OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.orc_cross_entropy_dense.restype = _dbl
        _lib.orc_cross_entropy_index.restype = _dbl
    return _lib


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a, a.ctypes.data_as(_i64p)


def round_bf16(x):
    """float32 -> nearest-even bfloat16 -> float32."""
    x, xp = _f(x)
    y = np.empty_like(x)
    lib().orc_round_bf16(xp, y.ctypes.data_as(_f32p), _i64(x.size))
    return y


def matmul_bias_bt(a, w, bias=None):
    a, ap = _f(a)
    w, wp = _f(w)
    M, K = a.shape
    N = w.shape[0]
    y = np.empty((M, N), np.float32)
    bp = None
    if bias is not None:
        bias, bp = _f(bias)
    lib().orc_matmul_bias_bt(ap, wp, bp, y.ctypes.data_as(_f32p), _i64(M), _i64(N), _i64(K), _i64(K), _i64(K),
                             _i64(N))
    return y


def matmul_bias_bt_bwd(dy, x, w, need_db=True):
    """Returns (dX, dW, db) for Y = X @ W.T + b."""
    dy, dyp = _f(dy)
    x, xp = _f(x)
    w, wp = _f(w)
    M, N = dy.shape
    K = x.shape[1]
    dx = np.empty((M, K), np.float32)
    dw = np.empty((N, K), np.float32)
    db = np.empty((N,), np.float32) if need_db else None
    lib().orc_matmul_bias_bt_bwd(dyp, xp, wp, dx.ctypes.data_as(_f32p), dw.ctypes.data_as(_f32p),
                                 db.ctypes.data_as(_f32p) if need_db else None, _i64(M), _i64(N), _i64(K), _i64(N),
                                 _i64(K), _i64(K), _i64(K), _i64(K))
    return dx, dw, db


def layer_norm_fwd(x, gamma, beta, eps=1e-5):
    x, xp = _f(x)
    gamma, gp = _f(gamma)
    beta, bp = _f(beta)
    cols = x.shape[-1]
    rows = x.size // cols
    y = np.empty_like(x)
    mean = np.empty((rows,), np.float32)
    rstd = np.empty((rows,), np.float32)
    lib().orc_layer_norm_fwd(xp, gp, bp, y.ctypes.data_as(_f32p), mean.ctypes.data_as(_f32p),
                             rstd.ctypes.data_as(_f32p), _i64(rows), _i64(cols), _dbl(eps))
    return y, mean, rstd


def layer_norm_bwd(dy, x, gamma, eps=1e-5):
    dy, dyp = _f(dy)
    x, xp = _f(x)
    gamma, gp = _f(gamma)
    cols = x.shape[-1]
    rows = x.size // cols
    dx = np.empty_like(x)
    dg = np.empty((cols,), np.float32)
    db = np.empty((cols,), np.float32)
    lib().orc_layer_norm_bwd(dyp, xp, gp, dx.ctypes.data_as(_f32p), dg.ctypes.data_as(_f32p),
                             db.ctypes.data_as(_f32p), _i64(rows), _i64(cols), _dbl(eps))
    return dx, dg, db


def cross_entropy_dense(logits, labels, upstream=1.0, want_grad=True):
    """Returns (loss, dlogits) with dense float labels of the logits' shape."""
    logits, lp = _f(logits)
    labels, tp = _f(labels)
    N, C = logits.shape
    d = np.empty_like(logits) if want_grad else None
    loss = lib().orc_cross_entropy_dense(lp, tp, d.ctypes.data_as(_f32p) if want_grad else None, _i64(N), _i64(C),
                                         _i64(C), _i64(C), _i64(C), _dbl(upstream))
    return float(loss), d


def cross_entropy_index(logits, idx, upstream=1.0, want_grad=True):
    """Returns (loss, dlogits, row_lse) with one class index per row."""
    logits, lp = _f(logits)
    idx, ip = _i(idx)
    N, C = logits.shape
    d = np.empty_like(logits) if want_grad else None
    lse = np.empty((N,), np.float32)
    loss = lib().orc_cross_entropy_index(lp, ip, d.ctypes.data_as(_f32p) if want_grad else None,
                                         lse.ctypes.data_as(_f32p), _i64(N), _i64(C), _i64(C), _i64(C),
                                         _dbl(upstream))
    return float(loss), d, lse


def sdpa_fwd(q, k, v, scale, causal, mask=None):
    """q,k,v BSHD -> (O BHSD, LSE (B,H,S))."""
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    B, S, H, D = q.shape
    out = np.empty((B, H, S, D), np.float32)
    lse = np.empty((B, H, S), np.float32)
    mp = None
    if mask is not None:
        mask, mp = _f(mask)
    lib().orc_sdpa_fwd(qp, kp, vp, mp, out.ctypes.data_as(_f32p), lse.ctypes.data_as(_f32p), _i64(B), _i64(S),
                       _i64(H), _i64(D), _dbl(scale), ctypes.c_int(int(causal)))
    return out, lse


def sdpa_bwd(q, k, v, dy, scale, causal, mask=None, o_saved=None):
    """q,k,v BSHD, dy BHSD -> (dQ, dK, dV) BSHD.  o_saved: stored forward output (BHSD) to take delta from."""
    q, qp = _f(q)
    k, kp = _f(k)
    v, vp = _f(v)
    dy, dp = _f(dy)
    B, S, H, D = q.shape
    dq = np.empty_like(q)
    dk = np.empty_like(q)
    dv = np.empty_like(q)
    mp = None
    if mask is not None:
        mask, mp = _f(mask)
    op = None
    if o_saved is not None:
        o_saved, op = _f(o_saved)
    lib().orc_sdpa_bwd(qp, kp, vp, dp, mp, op, dq.ctypes.data_as(_f32p), dk.ctypes.data_as(_f32p),
                       dv.ctypes.data_as(_f32p), _i64(B), _i64(S), _i64(H), _i64(D), _dbl(scale),
                       ctypes.c_int(int(causal)))
    return dq, dk, dv


def relu(x):
    x, xp = _f(x)
    y = np.empty_like(x)
    lib().orc_relu(xp, y.ctypes.data_as(_f32p), _i64(x.size))
    return y


def relu_grad(x, dy):
    x, xp = _f(x)
    dy, dp = _f(dy)
    dx = np.empty_like(x)
    lib().orc_relu_grad(xp, dp, dx.ctypes.data_as(_f32p), _i64(x.size))
    return dx


def embedding_fwd(table, idx):
    table, tp = _f(table)
    idx, ip = _i(idx)
    d = table.shape[1]
    out = np.empty((idx.size, d), np.float32)
    lib().orc_embedding_fwd(tp, ip, out.ctypes.data_as(_f32p), _i64(idx.size), _i64(d))
    return out


def embedding_bwd(dout, idx, V):
    dout, dp = _f(dout)
    idx, ip = _i(idx)
    d = dout.shape[1]
    dt = np.empty((V, d), np.float32)
    lib().orc_embedding_bwd(dp, ip, dt.ctypes.data_as(_f32p), _i64(idx.size), _i64(V), _i64(d))
    return dt
