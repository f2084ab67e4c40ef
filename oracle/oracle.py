"""ctypes front end of the CPU oracle (``libpathsig_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``.  The shipped package never imports this module.

All functions take and return CPU ``torch`` tensors (float32 or float64) and mirror the four
operators of the reference (``src/pathsig/bindings.cpp:9-63``):

* :func:`sig_forward`       ~ ``pathsig::compute_signature``
* :func:`sig_backward`      ~ ``pathsig::signature_backward``
* :func:`sig_to_logsig`     ~ ``pathsig::sig_to_logsig``
* :func:`logsig_backward`   ~ ``pathsig::logsig_backward``

plus :func:`logsignature`, which chains them the way ``LogSignature.forward`` does
(``src/pathsig/modules.py:112-135``), and :func:`chen_product`, a definition-level statement (torch
outer products, no native code) of the one operator of the package that the reference does not have.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import threading
from typing import Optional, Sequence

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libpathsig_oracle.so")
_lock = threading.Lock()
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file; returns the library path."""
    if force or not os.path.isfile(_LIB_PATH):
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            build()
            lib = ctypes.CDLL(_LIB_PATH)
            p, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
            for sfx in ("_f32", "_f64"):
                getattr(lib, "oracle_sig_forward" + sfx).argtypes = [p, i64, i64, i32, i32, p, p, p, i64, p]
                getattr(lib, "oracle_sig_backward" + sfx).argtypes = [p, p, p, i64, i64, i32, i32, p, p, p, i64, p]
                getattr(lib, "oracle_sig_to_logsig" + sfx).argtypes = [p, i64, i32, i32, p, p, p, p]
                getattr(lib, "oracle_logsig_backward" + sfx).argtypes = [p, p, p, i64, i32, i32, p, p, p]
                for name in ("oracle_sig_forward", "oracle_sig_backward", "oracle_sig_to_logsig",
                             "oracle_logsig_backward"):
                    getattr(lib, name + sfx).restype = ctypes.c_int
            _lib = lib
    return _lib


def set_threads(n: int) -> None:
    """Number of OpenMP threads used by the oracle (``omp_set_num_threads``)."""
    gomp = ctypes.CDLL("libgomp.so.1")
    gomp.omp_set_num_threads(int(n))


def _sfx(t: torch.Tensor) -> str:
    if t.dtype == torch.float32:
        return "_f32"
    if t.dtype == torch.float64:
        return "_f64"
    raise TypeError("oracle supports float32 and float64")


def _cpu(t: torch.Tensor, dtype=None) -> torch.Tensor:
    t = t.detach().to("cpu")
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous()


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else ctypes.c_void_p(t.data_ptr())


def _levels(level_sizes: Optional[Sequence[int]], depth: int):
    if level_sizes is None or len(level_sizes) == 0:
        return None
    if len(level_sizes) < depth + 1:
        raise ValueError("level_sizes must cover depth + 1 entries")
    return torch.tensor(list(level_sizes[: depth + 1]), dtype=torch.int64)


def sig_size(d: int, depth: int, level_sizes: Optional[Sequence[int]] = None) -> int:
    if level_sizes is None or len(level_sizes) == 0:
        return sum(d ** k for k in range(1, depth + 1))
    return int(sum(level_sizes[1: depth + 1]))


def sig_forward(path, depth, encoded_words=None, level_sizes=None, windows=None):
    """Signature of ``path`` (B, L, d); ``level_sizes=None`` means all levels dense."""
    path = _cpu(path)
    B, L, d = path.shape
    ls = _levels(level_sizes, depth)
    ew = _cpu(encoded_words, torch.int64) if (ls is not None and encoded_words is not None) else None
    win = _cpu(windows, torch.int32) if windows is not None else None
    W = 0 if win is None else win.shape[0]
    D = sig_size(d, depth, level_sizes)
    out = torch.zeros((B, D) if win is None else (B, W, D), dtype=path.dtype)
    rc = getattr(_load(), "oracle_sig_forward" + _sfx(path))(
        _ptr(path), B, L, d, depth, _ptr(ew), _ptr(ls), _ptr(win), W, _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle_sig_forward failed ({rc})")
    return out


def sig_backward(path, sig, grad_sig, depth, encoded_words=None, level_sizes=None, windows=None):
    """Gradient wrt ``path`` of ``sum(sig * grad_sig)``; ``sig`` is the forward output."""
    path = _cpu(path)
    sig = _cpu(sig, path.dtype)
    grad_sig = _cpu(grad_sig, path.dtype)
    B, L, d = path.shape
    ls = _levels(level_sizes, depth)
    ew = _cpu(encoded_words, torch.int64) if (ls is not None and encoded_words is not None) else None
    win = _cpu(windows, torch.int32) if windows is not None else None
    W = 0 if win is None else win.shape[0]
    out = torch.zeros_like(path)
    rc = getattr(_load(), "oracle_sig_backward" + _sfx(path))(
        _ptr(path), _ptr(sig), _ptr(grad_sig), B, L, d, depth, _ptr(ew), _ptr(ls), _ptr(win), W, _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle_sig_backward failed ({rc})")
    return out


def _rows(t: torch.Tensor) -> int:
    n = 1
    for s in t.shape[:-1]:
        n *= s
    return n


def sig_to_logsig(sig, depth, d, top_words=None, level_sizes=None):
    """(logsig, P) for a signature in the hybrid layout (dense below the top level)."""
    sig = _cpu(sig)
    ls = _levels(level_sizes, depth) if top_words is not None else None
    tw = _cpu(top_words, torch.int64) if ls is not None else None
    logsig = torch.zeros_like(sig)
    P = torch.zeros(sig.shape[:-1] + (sig.shape[-1] * depth,), dtype=sig.dtype)
    rc = getattr(_load(), "oracle_sig_to_logsig" + _sfx(sig))(
        _ptr(sig), _rows(sig), depth, d, _ptr(tw), _ptr(ls), _ptr(logsig), _ptr(P))
    if rc != 0:
        raise RuntimeError(f"oracle_sig_to_logsig failed ({rc})")
    return logsig, P


def logsig_backward(sig, P, grad_logsig, depth, d, top_words=None, level_sizes=None):
    sig = _cpu(sig)
    P = _cpu(P, sig.dtype)
    grad_logsig = _cpu(grad_logsig, sig.dtype)
    ls = _levels(level_sizes, depth) if top_words is not None else None
    tw = _cpu(top_words, torch.int64) if ls is not None else None
    out = torch.zeros_like(sig)
    rc = getattr(_load(), "oracle_logsig_backward" + _sfx(sig))(
        _ptr(sig), _ptr(P), _ptr(grad_logsig), _rows(sig), depth, d, _ptr(tw), _ptr(ls), _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle_logsig_backward failed ({rc})")
    return out


def logsignature(path, depth, *, top_words=None, ext_level_sizes=None, indices=None, windows=None,
                 grad_out=None):
    """Log-signature the way ``LogSignature.forward`` composes it (src/pathsig/modules.py:112-135).

    ``top_words`` / ``ext_level_sizes`` / ``indices`` are the module's ``_top_words``,
    ``_ext_level_sizes`` and ``_indices_from_sig``; all ``None`` for the un-projected case.
    With ``grad_out`` also returns the gradient wrt ``path``.
    """
    path = _cpu(path)
    d = path.shape[-1]
    projected = ext_level_sizes is not None
    sig = sig_forward(path, depth, top_words if projected else None,
                      ext_level_sizes if projected else None, windows)
    logsig, P = sig_to_logsig(sig, depth, d, top_words if projected else None,
                              ext_level_sizes if projected else None)
    out = logsig if indices is None else logsig.index_select(-1, _cpu(indices, torch.int64))
    if grad_out is None:
        return out
    g = _cpu(grad_out, path.dtype)
    if indices is not None:
        gl = torch.zeros_like(logsig)
        gl.index_add_(-1, _cpu(indices, torch.int64), g)
    else:
        gl = g
    gsig = logsig_backward(sig, P, gl, depth, d, top_words if projected else None,
                           ext_level_sizes if projected else None)
    gpath = sig_backward(path, sig, gsig, depth, top_words if projected else None,
                         ext_level_sizes if projected else None, windows)
    return out, gpath


def chen_product(sig_a, sig_b, d: int, depth: int):
    """Truncated tensor product of two dense signatures ``(..., D)`` (degree-0 coordinate 1 implied):
    ``out_n = a_n + b_n + sum_{0<k<n} a_k (x) b_{n-k}``, level by level with explicit outer products.

    Not an operator of the reference (it never combines signatures); the definition is Chen's identity
    for the signature of a concatenation, which the reference's forward recurrence applies one
    increment at a time (``src/pathsig/forward/sig_kernels.cu:138-152``).  Returns
    ``(out, grad_fn)`` where ``grad_fn(g)`` gives ``(dL/da, dL/db)`` for ``dL/dout = g``.
    """
    a, b = _cpu(sig_a, torch.float64), _cpu(sig_b, torch.float64)
    lead = a.shape[:-1]
    off = [0]
    for k in range(1, depth + 1):
        off.append(off[-1] + d ** k)
    if a.shape[-1] != off[-1] or b.shape != a.shape:
        raise ValueError("signatures must be dense rows of equal shape")
    al = [a[..., off[k - 1]: off[k]].reshape(-1, d ** k) for k in range(1, depth + 1)]
    bl = [b[..., off[k - 1]: off[k]].reshape(-1, d ** k) for k in range(1, depth + 1)]

    def product(xl, yl, bilinear_only=False):
        out = []
        for n in range(1, depth + 1):
            acc = torch.zeros_like(xl[n - 1]) if bilinear_only else xl[n - 1] + yl[n - 1]
            for k in range(1, n):
                acc = acc + (xl[k - 1].unsqueeze(2) * yl[n - k - 1].unsqueeze(1)).reshape(acc.shape)
            out.append(acc)
        return out

    out = torch.cat(product(al, bl), dim=1).reshape(lead + (off[-1],))

    def grad_fn(g):
        gl = [_cpu(g, torch.float64)[..., off[k - 1]: off[k]].reshape(-1, d ** k) for k in range(1, depth + 1)]
        ga = [x.clone() for x in gl]
        gb = [x.clone() for x in gl]
        for n in range(1, depth + 1):
            for k in range(1, n):
                gn = gl[n - 1].reshape(-1, d ** k, d ** (n - k))
                ga[k - 1] += (gn * bl[n - k - 1].unsqueeze(1)).sum(2)
                gb[n - k - 1] += (gn * al[k - 1].unsqueeze(2)).sum(1)
        return (torch.cat(ga, dim=1).reshape(lead + (off[-1],)), torch.cat(gb, dim=1).reshape(lead + (off[-1],)))

    return out, grad_fn
