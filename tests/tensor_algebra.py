"""Definition-level truncated tensor algebra in numpy float64 (tests only).

Independent of both the oracle's per-word recursions and the CUDA kernels: levels are dense
arrays of shape (d,)*k, products are explicit outer products.  Used to pin the oracle on
small cases (src/pathsig semantics restated from the mathematical definition:
S = prod_t exp(dx_t), log S = sum_m (-1)^(m+1) (S-1)^m / m).
"""
from __future__ import annotations

import math

import numpy as np


def one(d, depth):
    return [np.ones(())] + [np.zeros((d,) * k) for k in range(1, depth + 1)]


def mul(a, b, depth):
    out = []
    for k in range(depth + 1):
        acc = 0
        for j in range(k + 1):
            acc = acc + np.multiply.outer(a[j], b[k - j])
        out.append(acc)
    return out


def exp_inc(dx, depth):
    out = [np.ones(())]
    cur = np.ones(())
    for k in range(1, depth + 1):
        cur = np.multiply.outer(cur, dx)
        out.append(cur / math.factorial(k))
    return out


def signature_levels(path, depth):
    """path (L, d) -> list of level arrays, index 0 = scalar 1."""
    d = path.shape[1]
    s = one(d, depth)
    for t in range(path.shape[0] - 1):
        s = mul(s, exp_inc(path[t + 1] - path[t], depth), depth)
    return s


def flatten(levels):
    return np.concatenate([lv.reshape(-1) for lv in levels[1:]])


def signature(path, depth):
    return flatten(signature_levels(path, depth))


def log_levels(levels, depth):
    d = levels[1].shape[0]
    x = [np.zeros(())] + [lv.copy() for lv in levels[1:]]
    power = one(d, depth)
    out = [np.zeros(())] + [np.zeros((d,) * k) for k in range(1, depth + 1)]
    for m in range(1, depth + 1):
        power = mul(power, x, depth)
        coeff = (1.0 if m % 2 == 1 else -1.0) / m
        for k in range(1, depth + 1):
            out[k] = out[k] + coeff * power[k]
    return out


def logsignature(path, depth):
    return flatten(log_levels(signature_levels(path, depth), depth))
