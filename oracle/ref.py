"""ctypes/numpy front end of the CPU oracle (``libcleave_ref.so``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this module;
the shipped package never does.  Every function maps one-to-one onto a function of
``cleave_ref.cpp``, which cites the reference source lines it restates.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libcleave_ref.so")

_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i64 = ctypes.c_int64


def build(force: bool = False) -> str:
    """Compile the oracle with the flags stated in ``oracle/Makefile``; returns the .so path."""
    src = os.path.join(_HERE, "cleave_ref.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "libcleave_ref.so"])
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        sig = {
            "ref_matmul_ijk_f32": (None, [_f32p, _f32p, _f32p, _i64, _i64, _i64]),
            "ref_matmul_f32": (None, [_f32p, _f32p, _f32p, _i64, _i64, _i64]),
            "ref_matmul_rows_f32": (None, [_f32p, _f32p, _f32p, _i64, _i64, _i64, _i64, _i64]),
            "ref_matmul_f64acc": (None, [_f32p, _f32p, _f64p, _i64, _i64, _i64]),
            "ref_matmul_absdot_f64": (None, [_f32p, _f32p, _f64p, _i64, _i64, _i64]),
            "ref_matmul_tn_f32": (None, [_f32p, _f32p, _f32p, _i64, _i64, _i64]),
            "ref_matmul_nt_f32": (None, [_f32p, _f32p, _f32p, _i64, _i64, _i64]),
            "ref_sum_f32": (ctypes.c_float, [_f32p, _i64]),
            "ref_mean_f32": (ctypes.c_float, [_f32p, _i64]),
            "ref_max_f32": (ctypes.c_float, [_f32p, _i64]),
            "ref_sum_f64acc": (ctypes.c_double, [_f32p, _i64]),
            "ref_sum_abs_f64": (ctypes.c_double, [_f32p, _i64]),
            "ref_bias_add_f32": (None, [_f32p, _f32p, _f32p, _i64, _i64]),
            "ref_colsum_f32": (None, [_f32p, _f32p, _i64, _i64]),
            "ref_mse_f32": (ctypes.c_float, [_f32p, _f32p, _f32p, _i64]),
            "ref_mse_f64acc": (ctypes.c_double, [_f32p, _f32p, _i64]),
            "ref_sgd_f32": (None, [_f32p, _f32p, ctypes.c_float, _i64]),
            "ref_linreg_step_f32": (ctypes.c_float, [_f32p, _f32p, _f32p, _f32p, _f32p, _i64, _i64]),
            "ref_linreg_step_f64": (ctypes.c_double, [_f32p, _f32p, _f32p, _f64p, _i64, _i64]),
            "ref_mlp2_fwd_bwd_f32": (
                ctypes.c_float,
                [_f32p] * 6 + [_i64] * 4 + [ctypes.c_int] * 3 + [_f32p] * 11,
            ),
            "ref_num_threads": (ctypes.c_int, []),
            "ref_set_num_threads": (None, [ctypes.c_int]),
        }
        for name in ("add", "sub", "mul", "div"):
            sig[f"ref_{name}_f32"] = (None, [_f32p, _f32p, _f32p, _i64])
        for name in ("neg", "relu", "exp", "sigmoid", "tanh"):
            sig[f"ref_{name}_f32"] = (None, [_f32p, _f32p, _i64])
        for name in ("tanh_bwd", "sigmoid_bwd", "relu_bwd"):
            sig[f"ref_{name}_f32"] = (None, [_f32p, _f32p, _f32p, _i64])
        sig["ref_matmul_f64"] = (None, [_f64p, _f64p, _f64p, _i64, _i64, _i64])
        for name in ("add", "sub", "mul", "div"):
            sig[f"ref_{name}_f64"] = (None, [_f64p, _f64p, _f64p, _i64])
        for name in ("neg", "relu", "exp", "sigmoid", "tanh"):
            sig[f"ref_{name}_f64"] = (None, [_f64p, _f64p, _i64])
        for name in ("sum", "mean", "max"):
            sig[f"ref_{name}_f64"] = (ctypes.c_double, [_f64p, _i64])
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _c(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(_f32p)


def _pd(a: np.ndarray):
    return a.ctypes.data_as(_f64p)


def num_threads() -> int:
    return int(lib().ref_num_threads())


def set_num_threads(n: int) -> None:
    lib().ref_set_num_threads(int(n))


# ------------------------------------------------------------------ matmul
def matmul(a, b, faithful_loop_order: bool = False) -> np.ndarray:
    a, b = _c(a), _c(b)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), np.float32)
    fn = lib().ref_matmul_ijk_f32 if faithful_loop_order else lib().ref_matmul_f32
    fn(_p(a), _p(b), _p(c), m, k, n)
    return c


def matmul_rows(a, b, row0: int, rows: int) -> np.ndarray:
    a, b = _c(a), _c(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((rows, n), np.float32)
    lib().ref_matmul_rows_f32(_p(a), _p(b), _p(c), m, k, n, row0, rows)
    return c


def matmul_f64(a, b) -> np.ndarray:
    a, b = _c(a), _c(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float64)
    lib().ref_matmul_f64acc(_p(a), _p(b), _pd(c), m, k, n)
    return c


def matmul_absdot(a, b) -> np.ndarray:
    a, b = _c(a), _c(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float64)
    lib().ref_matmul_absdot_f64(_p(a), _p(b), _pd(c), m, k, n)
    return c


def matmul_tn(a, b) -> np.ndarray:
    """a stored [k, m], b stored [k, n] -> a^T b."""
    a, b = _c(a), _c(b)
    k, m = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().ref_matmul_tn_f32(_p(a), _p(b), _p(c), m, k, n)
    return c


def matmul_nt(a, b) -> np.ndarray:
    """a stored [m, k], b stored [n, k] -> a b^T."""
    a, b = _c(a), _c(b)
    m, k = a.shape
    n = b.shape[0]
    c = np.empty((m, n), np.float32)
    lib().ref_matmul_nt_f32(_p(a), _p(b), _p(c), m, k, n)
    return c


# ------------------------------------------------------------------ elementwise
def _binary(name):
    def f(a, b):
        a, b = _c(a), _c(b)
        assert a.shape == b.shape
        o = np.empty_like(a)
        getattr(lib(), f"ref_{name}_f32")(_p(a), _p(b), _p(o), a.size)
        return o

    f.__name__ = name
    return f


def _unary(name):
    def f(a):
        a = _c(a)
        o = np.empty_like(a)
        getattr(lib(), f"ref_{name}_f32")(_p(a), _p(o), a.size)
        return o

    f.__name__ = name
    return f


add, sub, mul, div = (_binary(n) for n in ("add", "sub", "mul", "div"))
neg, relu, exp, sigmoid, tanh = (_unary(n) for n in ("neg", "relu", "exp", "sigmoid", "tanh"))
tanh_bwd, sigmoid_bwd, relu_bwd = (_binary(n) for n in ("tanh_bwd", "sigmoid_bwd", "relu_bwd"))


# ------------------------------------------------------------------ reductions
def sum(v) -> np.float32:  # noqa: A001 - mirrors the reference name
    v = _c(v).ravel()
    return np.float32(lib().ref_sum_f32(_p(v), v.size))


def mean(v) -> np.float32:
    v = _c(v).ravel()
    return np.float32(lib().ref_mean_f32(_p(v), v.size))


def max_of(v) -> np.float32:
    v = _c(v).ravel()
    return np.float32(lib().ref_max_f32(_p(v), v.size))


def sum_f64(v) -> float:
    v = _c(v).ravel()
    return float(lib().ref_sum_f64acc(_p(v), v.size))


def sum_abs_f64(v) -> float:
    v = _c(v).ravel()
    return float(lib().ref_sum_abs_f64(_p(v), v.size))


# ------------------------------------------------------------------ compositions
def bias_add(x, b) -> np.ndarray:
    x, b = _c(x), _c(b)
    o = np.empty_like(x)
    lib().ref_bias_add_f32(_p(x), _p(b), _p(o), x.shape[0], x.shape[1])
    return o


def colsum(x) -> np.ndarray:
    x = _c(x)
    o = np.empty(x.shape[1], np.float32)
    lib().ref_colsum_f32(_p(x), _p(o), x.shape[0], x.shape[1])
    return o


def mse(p, t):
    """Returns (loss, dloss/dp) with loss = mean((p - t)^2)."""
    p, t = _c(p), _c(t)
    dp = np.empty_like(p)
    loss = lib().ref_mse_f32(_p(p), _p(t), _p(dp), p.size)
    return np.float32(loss), dp


def mse_f64(p, t) -> float:
    p, t = _c(p), _c(t)
    return float(lib().ref_mse_f64acc(_p(p), _p(t), p.size))


def sgd(w, g, lr) -> np.ndarray:
    w = _c(w).copy()
    g = _c(g)
    lib().ref_sgd_f32(_p(w), _p(g), ctypes.c_float(lr), w.size)
    return w


def linreg_step(X, y, w):
    """Returns (loss, pred, grad) for loss = mean((X w - y)^2)."""
    X, y, w = _c(X), _c(y), _c(w)
    rows, feat = X.shape
    pred = np.empty(rows, np.float32)
    grad = np.empty(feat, np.float32)
    loss = lib().ref_linreg_step_f32(_p(X), _p(y), _p(w), _p(pred), _p(grad), rows, feat)
    return np.float32(loss), pred, grad


def linreg_step_f64(X, y, w):
    X, y, w = _c(X), _c(y), _c(w)
    rows, feat = X.shape
    grad = np.empty(feat, np.float64)
    loss = lib().ref_linreg_step_f64(_p(X), _p(y), _p(w), _pd(grad), rows, feat)
    return float(loss), grad


ACT = {"identity": 0, "relu": 1, "sigmoid": 2, "tanh": 3}


def mlp2_fwd_bwd(X, W1, b1, W2, b2, T, act1="tanh", act2="sigmoid", mean_loss=True) -> dict:
    """Two-layer perceptron forward + backward; returns every intermediate and gradient."""
    X, W1, b1, W2, b2, T = (_c(a) for a in (X, W1, b1, W2, b2, T))
    batch, d_in = X.shape
    d_hid = W1.shape[1]
    d_out = W2.shape[1]
    f = lambda *s: np.empty(s, np.float32)  # noqa: E731
    r = dict(
        Z1=f(batch, d_hid), H=f(batch, d_hid), Z2=f(batch, d_out), Y=f(batch, d_out),
        dZ2=f(batch, d_out), dH=f(batch, d_hid), dZ1=f(batch, d_hid),
        dW1=f(d_in, d_hid), db1=f(d_hid), dW2=f(d_hid, d_out), db2=f(d_out),
    )
    loss = lib().ref_mlp2_fwd_bwd_f32(
        _p(X), _p(W1), _p(b1), _p(W2), _p(b2), _p(T), batch, d_in, d_hid, d_out,
        ACT[act1], ACT[act2], 1 if mean_loss else 0,
        *(_p(r[k]) for k in ("Z1", "H", "Z2", "Y", "dZ2", "dH", "dZ1", "dW1", "db1", "dW2", "db2")),
    )
    r["loss"] = np.float32(loss)
    return r


# ------------------------------------------------------------------ f64 instances
def _c64(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float64)


def matmul64(a, b) -> np.ndarray:
    a, b = _c64(a), _c64(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float64)
    lib().ref_matmul_f64(_pd(a), _pd(b), _pd(c), m, k, n)
    return c


def binary64(name: str, a, b) -> np.ndarray:
    a, b = _c64(a), _c64(b)
    o = np.empty_like(a)
    getattr(lib(), f"ref_{name}_f64")(_pd(a), _pd(b), _pd(o), a.size)
    return o


def unary64(name: str, a) -> np.ndarray:
    a = _c64(a)
    o = np.empty_like(a)
    getattr(lib(), f"ref_{name}_f64")(_pd(a), _pd(o), a.size)
    return o


def reduce64(name: str, v) -> float:
    v = _c64(v).ravel()
    return float(getattr(lib(), f"ref_{name}_f64")(_pd(v), v.size))
