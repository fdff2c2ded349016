"""Seeded synthetic inputs for the benchmark configurations.

The reference measures on no public data set; each configuration is defined by shapes and value
distributions, so seeded synthetic inputs ARE the workload.  Generation uses numpy's Philox
counter-based generator with a fixed seed per tensor, on the host, so the oracle and the device
see identical bits.
"""
from __future__ import annotations

import math

import numpy as np


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(seed))


def uniform_pm1(seed: int, *shape) -> np.ndarray:
    """iid uniform on [-1, 1) in float32."""
    r = _rng(seed).random(shape, dtype=np.float32)
    r *= 2.0
    r -= 1.0
    return r


def uniform01(seed: int, *shape) -> np.ndarray:
    return _rng(seed).random(shape, dtype=np.float32)


def normal(seed: int, *shape, sigma: float = 1.0) -> np.ndarray:
    r = _rng(seed).standard_normal(shape, dtype=np.float32)
    if sigma != 1.0:
        r *= np.float32(sigma)
    return r


def xavier_uniform(seed: int, fan_in: int, fan_out: int) -> np.ndarray:
    a = math.sqrt(6.0 / (fan_in + fan_out))
    return (uniform_pm1(seed, fan_in, fan_out) * np.float32(a)).astype(np.float32)


def gemm_inputs(m: int, n: int, k: int, seed_a: int = 1, seed_b: int = 2):
    """Configuration 0 / 3: A [m,k], B [k,n] iid U[-1,1)."""
    return uniform_pm1(seed_a, m, k), uniform_pm1(seed_b, k, n)


def linreg_inputs(rows: int = 1 << 20, feat: int = 16):
    """Configuration 1: X ~ N(0,1), w* ~ N(0,1), y = X w* + noise, noise ~ N(0, 0.01) read as
    variance 0.01 (sigma 0.1)."""
    X = normal(3, rows, feat)
    w_true = normal(4, feat)
    y = (X.astype(np.float64) @ w_true.astype(np.float64)).astype(np.float32) + normal(5, rows, sigma=0.1)
    return X, y.astype(np.float32), w_true


def mlp_inputs(batch: int = 4096, d_in: int = 1024, d_hid: int = 4096, d_out: int = 1024, seed_shift: int = 0):
    """Configuration 2: X ~ N(0,1); W1, W2 Xavier-uniform; zero biases; targets U[0,1)."""
    X = normal(6 + seed_shift, batch, d_in)
    W1 = xavier_uniform(7, d_in, d_hid)
    W2 = xavier_uniform(8, d_hid, d_out)
    b1 = np.zeros(d_hid, np.float32)
    b2 = np.zeros(d_out, np.float32)
    T = uniform01(9 + seed_shift, batch, d_out)
    return X, W1, b1, W2, b2, T
