"""Operator layer: the reference's four operators, served by the B200 CUDA library.

Host-side mirror of ``src/pathsig/ops.py`` and ``src/pathsig/bindings.cpp`` of the reference:
the same four schemas (``bindings.cpp:9-63``), the same fake (meta) shape functions
(``ops.py:59-84, 101-123, 152-179, 197-227``) and the same autograd wiring
(``ops.py:231-297``).  The CUDA implementations validate like the reference launchers
(``forward/sig_launch.cu:84-121``, ``backward/sig_backward_launch.cu:94-155``), allocate the
outputs with torch's caching allocator and hand raw pointers plus the current stream to the
C ABI (``include/pathsig_b200.h``).  torch is used for memory, streams and dispatch only.

The operators are registered in the namespace ``pathsig_b200`` so that this package and a
build of the reference (namespace ``pathsig``) can live in one process, which is how the
parity tests compare them.  :func:`register_namespace` registers the same operators under
another namespace (``pathsig_b200.install_as_pathsig`` uses it for ``pathsig``).
"""
from __future__ import annotations

import collections
import ctypes
from typing import List, Optional, Sequence, Tuple

import torch
from torch import Tensor

from . import _load

__all__ = ["compute_signature", "sig_to_logsig", "signature_backward", "logsig_backward",
           "logsig_projected", "logsig_projected_backward", "logsig_projected_supported",
           "chen_product", "chen_product_backward", "register_namespace", "NAMESPACE"]

NAMESPACE = "pathsig_b200"

_SCHEMAS = {
    "compute_signature": "(Tensor path_in, int depth, bool alternative_projection, Tensor encoded_words, "
                         "int[] level_sizes, bool use_windows, Tensor windows) -> Tensor",
    "signature_backward": "(Tensor path_in, Tensor signature_in, Tensor grad_signature_in, int depth, "
                          "bool alternative_projection, Tensor encoded_words, int[] level_sizes, "
                          "bool use_windows, Tensor windows) -> Tensor",
    "sig_to_logsig": "(Tensor signature_in, int depth, int d, bool alternative_projection, "
                     "Tensor encoded_words, int[] level_sizes) -> (Tensor, Tensor)",
    "logsig_backward": "(Tensor signature_in, Tensor P_in, Tensor grad_logsig_in, int depth, "
                       "bool alternative_projection, Tensor encoded_words, int[] level_sizes) -> Tensor",
    # not in the reference, where a stock index_select follows the logarithm (src/pathsig/modules.py:134-135):
    # logarithm and column selection as one kernel.  The output row is the words of the degrees below `depth`
    # listed in lower_columns (positions in a dense row of those degrees) followed by the whole top degree.
    "logsig_projected": "(Tensor signature_in, int depth, int d, Tensor top_words, int[] level_sizes, "
                        "Tensor lower_columns) -> Tensor",
    "logsig_projected_backward": "(Tensor signature_in, Tensor grad_out, int depth, int d, Tensor top_words, "
                                 "int[] level_sizes, Tensor lower_columns) -> Tensor",
    # not in the reference: Chen product of two dense truncated signatures and its adjoint
    "chen_product": "(Tensor sig_a, Tensor sig_b, int depth, int d) -> Tensor",
    "chen_product_backward": "(Tensor sig_a, Tensor sig_b, Tensor grad_out, int depth, int d) -> (Tensor, Tensor)",
}

# Kernel family used by the signature operators: _load.ALGO_AUTO / ALGO_GENERIC / ALGO_TILED.
# Tests flip it to compare the register-tiled kernels with the generic ones.
_algo = _load.ALGO_AUTO


def set_algorithm(name: str) -> None:
    """Select the signature kernel family: "auto", "generic", "tiled" or "closure"."""
    global _algo
    _algo = {"auto": _load.ALGO_AUTO, "generic": _load.ALGO_GENERIC, "tiled": _load.ALGO_TILED,
             "closure": _load.ALGO_CLOSURE}[name]


# Host copies of word-code tensors.  The prefix-closure kernels are generated from the word set, so the
# library wants the codes in host memory; reading them back on every call would synchronise, so the
# copy is made once per (storage, version) and kept while the device tensor is alive.  An entry holds a
# reference to its device tensor, which keeps the address from being reused by another tensor.
_HOST_WORDS_LIMIT = 64
_host_words_cache: "collections.OrderedDict" = collections.OrderedDict()


def _host_words(words: Tensor) -> Optional[Tensor]:
    key = (words.data_ptr(), words._version, words.numel(), words.device.index)
    hit = _host_words_cache.get(key)
    if hit is not None:
        _host_words_cache.move_to_end(key)
        return hit[1]
    if torch.cuda.is_current_stream_capturing():
        return None  # no device read inside a graph capture; the library then uses another kernel family
    host = words.detach().cpu().contiguous()
    _host_words_cache[key] = (words, host)
    while len(_host_words_cache) > _HOST_WORDS_LIMIT:
        _host_words_cache.popitem(last=False)
    return host


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------

def _dtype_id(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return _load.PSIG_F32
    if t.dtype == torch.float64:
        return _load.PSIG_F64
    raise RuntimeError("path must be float32 or float64")


def _stream_ptr(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _ptr(t: Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr() if t.numel() > 0 else 0)


def _check_same_device(anchor: Tensor, **operands: Tensor) -> None:
    """Every tensor operand must live on the device the kernels are launched on (the anchor's).  The
    dispatcher does not check this for operators registered from Python, and a pointer into another
    GPU's memory would fault there (or be read silently over a peer mapping)."""
    for name, t in operands.items():
        if t.device != anchor.device:
            raise RuntimeError(f"{name} must be on the same device as the path/signature "
                               f"({name} is on {t.device}, expected {anchor.device})")


def _check_words_cuda(encoded_words: Tensor) -> None:
    if not encoded_words.is_cuda:
        raise RuntimeError("encoded_words must be CUDA")
    if encoded_words.dtype != torch.int64:
        raise RuntimeError("encoded_words must be int64")
    if not encoded_words.is_contiguous():
        raise RuntimeError("encoded_words must be contiguous")
    if encoded_words.dim() != 1:
        raise RuntimeError("encoded_words must be 1D")


def _sig_desc(path: Tensor, depth: int, alt: bool, encoded_words: Tensor, level_sizes: Sequence[int],
              use_windows: bool, windows: Tensor) -> Tuple[_load.SigDesc, list]:
    """Validated ``PsigSigDesc`` plus the tensors that must stay alive during the call."""
    if not path.is_cuda:
        raise RuntimeError("path must be CUDA")
    if path.dim() != 3:
        raise RuntimeError("path must be [B,T,d]")
    depth = int(depth)
    if not (1 <= depth <= _load.MAX_DEPTH):
        raise RuntimeError("depth must be in [1,12]")
    B, L, d = path.shape
    if L < 2:
        raise RuntimeError("path must have at least 2 time steps")
    keep = []
    desc = _load.SigDesc()
    desc.dtype = _dtype_id(path)
    desc.d, desc.depth, desc.B, desc.L = d, depth, B, L
    desc.projected = 1 if alt else 0
    desc.algo = _algo
    if alt:
        _check_words_cuda(encoded_words)
        _check_same_device(path, encoded_words=encoded_words)
        if len(level_sizes) < depth + 1:
            raise RuntimeError("level_sizes must cover at least depth + 1 entries")
        need = 0
        for k in range(1, depth + 1):
            size = int(level_sizes[k])
            desc.level_sizes[k] = size
            if size != d ** k:
                need += size
        if encoded_words.numel() < need:
            raise RuntimeError("encoded_words holds fewer codes than level_sizes requires")
        desc.words = encoded_words.data_ptr() if encoded_words.numel() > 0 else None
        keep.append(encoded_words)
        if encoded_words.numel() > 0:
            host = _host_words(encoded_words)
            if host is not None:
                desc.words_host = host.data_ptr()
                keep.append(host)
    if use_windows:
        if not windows.is_cuda:
            raise RuntimeError("windows must be CUDA")
        if windows.dim() != 2 or windows.size(1) != 2:
            raise RuntimeError("windows must be [W,2]")
        if windows.dtype not in (torch.int32, torch.int64):
            raise RuntimeError("windows must be int32")
        _check_same_device(path, windows=windows)
        win = windows.to(torch.int32).contiguous()
        keep.append(win)
        desc.W = win.size(0)
        desc.windows = win.data_ptr() if win.numel() > 0 else None
    return desc, keep


def _log_desc(signature: Tensor, depth: int, d: int, alt: bool, encoded_words: Tensor,
              level_sizes: Sequence[int], fake: bool = False) -> _load.LogDesc:
    """``PsigLogDesc`` for these arguments; with ``fake`` no device pointer is read (shape queries only)."""
    depth, d = int(depth), int(d)
    if not (1 <= depth <= _load.MAX_DEPTH):
        raise RuntimeError("depth must be in [1,12]")
    if d < 1:
        raise RuntimeError("d must be >= 1")
    if signature.dim() not in (2, 3):
        raise RuntimeError("signature must be [B,S] or [B,W,S]")
    desc = _load.LogDesc()
    desc.dtype = _dtype_id(signature)
    desc.d, desc.depth = d, depth
    desc.algo = _algo
    desc.rows = 0 if fake else (signature.numel() // signature.size(-1) if signature.size(-1) > 0 else 0)
    desc.top_size = d ** depth
    if alt:
        if not fake:
            _check_words_cuda(encoded_words)
            _check_same_device(signature, encoded_words=encoded_words)
        if len(level_sizes) < depth + 1:
            raise RuntimeError("level_sizes must have entries up to depth")
        desc.top_size = int(level_sizes[depth])
        if desc.top_size != d ** depth:
            if encoded_words.numel() < desc.top_size:
                raise RuntimeError("encoded_words holds fewer codes than level_sizes[depth]")
            if fake:
                desc.top_words = 1 if encoded_words.numel() > 0 else None  # non-null marker, never read
            else:
                desc.top_words = encoded_words.data_ptr() if encoded_words.numel() > 0 else None
    return desc


def _projected_log_desc(signature: Tensor, depth: int, d: int, top_words: Tensor, level_sizes: Sequence[int],
                        lower_columns: Tensor, fake: bool = False) -> _load.LogDesc:
    """``PsigLogDesc`` of the fused logarithm + column selection."""
    desc = _log_desc(signature, depth, d, True, top_words, level_sizes, fake=fake)
    if lower_columns.dim() != 1 or lower_columns.dtype != torch.int64:
        raise RuntimeError("lower_columns must be a 1D int64 tensor")
    if not fake:
        if not lower_columns.is_cuda or not lower_columns.is_contiguous():
            raise RuntimeError("lower_columns must be a contiguous CUDA tensor")
        _check_same_device(signature, lower_columns=lower_columns)
    desc.n_lower_columns = lower_columns.numel()
    # a non-null marker is enough for the shape queries; an empty list still selects the projected layout
    desc.lower_columns = (lower_columns.data_ptr() if not fake and lower_columns.numel() > 0 else 1)
    return desc


def logsig_projected_supported(dtype: torch.dtype, depth: int, d: int, level_sizes: Sequence[int]) -> bool:
    """Whether the fused logarithm + column selection has a kernel for this row (it is part of the
    row-in-shared-memory family, so the dense degrees below the top must fit shared memory)."""
    lib = _load.ensure_loaded()
    desc = _load.LogDesc()
    desc.dtype = _load.PSIG_F32 if dtype == torch.float32 else _load.PSIG_F64
    desc.d, desc.depth, desc.algo, desc.rows = int(d), int(depth), _algo, 1
    desc.top_size = int(level_sizes[depth])
    desc.top_words = 1 if desc.top_size != int(d) ** int(depth) else None
    return lib.psig_logsig_cache_size(ctypes.byref(desc)) == 0


def _row_width(d: int, depth: int, alt: bool, level_sizes: Sequence[int]) -> int:
    if alt:
        return int(sum(int(s) for s in level_sizes[1: depth + 1]))
    return int(sum(d ** k for k in range(1, depth + 1)))


# --------------------------------------------------------------------------------------
# CUDA implementations
# --------------------------------------------------------------------------------------

def _compute_signature_cuda(path_in, depth, alternative_projection, encoded_words, level_sizes, use_windows,
                            windows):
    lib = _load.ensure_loaded()
    path = path_in.contiguous()
    desc, keep = _sig_desc(path, depth, alternative_projection, encoded_words, level_sizes, use_windows, windows)
    D = _row_width(desc.d, desc.depth, bool(alternative_projection), level_sizes)
    shape = (desc.B, desc.W, D) if use_windows else (desc.B, D)
    out = torch.empty(shape, dtype=path.dtype, device=path.device)
    if out.numel() == 0:  # no paths, no windows or no requested words: nothing to launch
        return out
    with torch.cuda.device(path.device):
        rc = lib.psig_sig_forward(ctypes.byref(desc), _ptr(path), _ptr(out), _stream_ptr(path.device))
    _load.check(rc, "compute_signature")
    del keep
    return out


def _signature_backward_cuda(path_in, signature_in, grad_signature_in, depth, alternative_projection,
                             encoded_words, level_sizes, use_windows, windows):
    lib = _load.ensure_loaded()
    if not signature_in.is_cuda:
        raise RuntimeError("signature must be CUDA")
    if not grad_signature_in.is_cuda:
        raise RuntimeError("grad_signature must be CUDA")
    if signature_in.dtype != path_in.dtype:
        raise RuntimeError("signature must have same dtype as path")
    if grad_signature_in.dtype != path_in.dtype:
        raise RuntimeError("grad_signature must have same dtype as path")
    if signature_in.shape != grad_signature_in.shape:
        raise RuntimeError("grad_signature must match signature shape")
    _check_same_device(path_in, signature=signature_in, grad_signature=grad_signature_in)
    path = path_in.contiguous()
    sig = signature_in.contiguous()
    grad = grad_signature_in.contiguous()
    desc, keep = _sig_desc(path, depth, alternative_projection, encoded_words, level_sizes, use_windows, windows)
    D = _row_width(desc.d, desc.depth, bool(alternative_projection), level_sizes)
    expect = (desc.B, desc.W, D) if use_windows else (desc.B, D)
    if tuple(sig.shape) != expect:
        if use_windows and sig.dim() == 3 and sig.size(1) != desc.W:
            raise RuntimeError("windows.size(0) must match signature num_windows")
        raise RuntimeError("signature must be [B,S] or [B,W,S]")
    if sig.numel() == 0:  # an empty signature carries no gradient
        return torch.zeros_like(path)
    grad_path = torch.empty_like(path)
    with torch.cuda.device(path.device):
        ws_bytes = lib.psig_sig_backward_workspace(ctypes.byref(desc))
        _load.check(ws_bytes, "signature_backward")
        ws = torch.empty(max(int(ws_bytes), 1), dtype=torch.uint8, device=path.device)
        rc = lib.psig_sig_backward(ctypes.byref(desc), _ptr(path), _ptr(sig), _ptr(grad), _ptr(grad_path),
                                   _ptr(ws), int(ws_bytes), _stream_ptr(path.device))
    _load.check(rc, "signature_backward")
    del keep
    return grad_path


def _sig_to_logsig_cuda(signature_in, depth, d, alternative_projection, encoded_words, level_sizes):
    lib = _load.ensure_loaded()
    if not signature_in.is_cuda:
        raise RuntimeError("signature must be CUDA")
    sig = signature_in.contiguous()
    desc = _log_desc(sig, depth, d, alternative_projection, encoded_words, level_sizes)
    with torch.cuda.device(sig.device):
        S = lib.psig_logsig_size(ctypes.byref(desc))
        _load.check(S, "sig_to_logsig")
        if S != sig.size(-1):
            raise RuntimeError(f"signature width {sig.size(-1)} does not match the layout width {S}")
        logsig = torch.empty_like(sig)
        per_row = lib.psig_logsig_cache_size(ctypes.byref(desc))
        _load.check(per_row, "sig_to_logsig")
        cache = torch.empty(sig.shape[:-1] + (int(per_row),), dtype=sig.dtype, device=sig.device)
        rc = lib.psig_logsig_forward(ctypes.byref(desc), _ptr(sig), _ptr(logsig), _ptr(cache),
                                     _stream_ptr(sig.device))
    _load.check(rc, "sig_to_logsig")
    return logsig, cache


def _logsig_backward_cuda(signature_in, P_in, grad_logsig_in, depth, alternative_projection, encoded_words,
                          level_sizes):
    lib = _load.ensure_loaded()
    if not signature_in.is_cuda:
        raise RuntimeError("sig must be CUDA")
    if not P_in.is_cuda:
        raise RuntimeError("P must be CUDA")
    if not grad_logsig_in.is_cuda:
        raise RuntimeError("grad_logsig must be CUDA")
    if P_in.dtype != signature_in.dtype:
        raise RuntimeError("P must have same dtype as sig")
    if grad_logsig_in.dtype != signature_in.dtype:
        raise RuntimeError("grad_logsig must have same dtype as sig")
    if grad_logsig_in.shape != signature_in.shape:
        raise RuntimeError("grad_logsig must match sig shape")
    _check_same_device(signature_in, P=P_in, grad_logsig=grad_logsig_in)
    if len(level_sizes) <= int(depth):
        raise RuntimeError("level_sizes must have entries up to depth")
    d = int(level_sizes[1])  # the channel count travels in level_sizes[1], as in the reference
    if d < 1:
        raise RuntimeError("level_sizes[1] must be >= 1 (infers path_dim)")
    sig = signature_in.contiguous()
    cache = P_in.contiguous()
    grad = grad_logsig_in.contiguous()
    desc = _log_desc(sig, depth, d, alternative_projection, encoded_words, level_sizes)
    # The cache tells which kernel family produced it: the table of powers (S*depth per row) belongs to
    # the global-memory kernels, an empty one to the row-in-shared-memory kernels.
    if tuple(cache.shape[:-1]) != tuple(sig.shape[:-1]) or cache.size(-1) not in (0, sig.size(-1) * int(depth)):
        raise RuntimeError("P must be [B,(W),S*depth] (or [B,(W),0] as returned by sig_to_logsig)")
    desc.algo = _load.ALGO_GENERIC if cache.size(-1) > 0 else _load.ALGO_AUTO
    if lib.psig_logsig_cache_size(ctypes.byref(desc)) != cache.size(-1):
        raise RuntimeError("P does not belong to a sig_to_logsig call with these arguments")
    grad_sig = torch.empty_like(sig)
    with torch.cuda.device(sig.device):
        ws_bytes = lib.psig_logsig_backward_workspace(ctypes.byref(desc))
        _load.check(ws_bytes, "logsig_backward")
        ws = torch.empty(max(int(ws_bytes), 1), dtype=torch.uint8, device=sig.device)
        rc = lib.psig_logsig_backward(ctypes.byref(desc), _ptr(sig), _ptr(cache), _ptr(grad), _ptr(grad_sig),
                                      _ptr(ws), int(ws_bytes), _stream_ptr(sig.device))
    _load.check(rc, "logsig_backward")
    return grad_sig


def _logsig_projected_cuda(signature_in, depth, d, top_words, level_sizes, lower_columns):
    lib = _load.ensure_loaded()
    if not signature_in.is_cuda:
        raise RuntimeError("signature must be CUDA")
    sig = signature_in.contiguous()
    desc = _projected_log_desc(sig, depth, d, top_words, level_sizes, lower_columns)
    with torch.cuda.device(sig.device):
        S = lib.psig_logsig_size(ctypes.byref(desc))
        _load.check(S, "logsig_projected")
        if S != sig.size(-1):
            raise RuntimeError(f"signature width {sig.size(-1)} does not match the layout width {S}")
        width = lib.psig_logsig_out_size(ctypes.byref(desc))
        _load.check(width, "logsig_projected")
        out = torch.empty(sig.shape[:-1] + (int(width),), dtype=sig.dtype, device=sig.device)
        if out.numel() == 0:
            return out
        rc = lib.psig_logsig_forward(ctypes.byref(desc), _ptr(sig), _ptr(out), None, _stream_ptr(sig.device))
    _load.check(rc, "logsig_projected")
    return out


def _logsig_projected_backward_cuda(signature_in, grad_out, depth, d, top_words, level_sizes, lower_columns):
    lib = _load.ensure_loaded()
    if not signature_in.is_cuda or not grad_out.is_cuda:
        raise RuntimeError("signature and grad_out must be CUDA")
    if grad_out.dtype != signature_in.dtype:
        raise RuntimeError("grad_out must have same dtype as signature")
    _check_same_device(signature_in, grad_out=grad_out)
    sig = signature_in.contiguous()
    grad = grad_out.contiguous()
    desc = _projected_log_desc(sig, depth, d, top_words, level_sizes, lower_columns)
    with torch.cuda.device(sig.device):
        width = lib.psig_logsig_out_size(ctypes.byref(desc))
        _load.check(width, "logsig_projected_backward")
        if tuple(grad.shape) != tuple(sig.shape[:-1]) + (int(width),):
            raise RuntimeError("grad_out must be [B,(W),n_lower_columns + top_size]")
        grad_sig = torch.empty_like(sig)
        if grad_sig.numel() == 0:
            return grad_sig
        rc = lib.psig_logsig_backward(ctypes.byref(desc), _ptr(sig), None, _ptr(grad), _ptr(grad_sig), None, 0,
                                      _stream_ptr(sig.device))
    _load.check(rc, "logsig_projected_backward")
    return grad_sig


def _chen_desc(sig_a: Tensor, sig_b: Tensor, depth: int, d: int) -> _load.ChenDesc:
    depth, d = int(depth), int(d)
    if not sig_a.is_cuda or not sig_b.is_cuda:
        raise RuntimeError("signatures must be CUDA")
    if not (1 <= depth <= _load.MAX_DEPTH):
        raise RuntimeError("depth must be in [1,12]")
    if d < 1:
        raise RuntimeError("d must be >= 1")
    if sig_a.dtype != sig_b.dtype:
        raise RuntimeError("signatures must have the same dtype")
    _check_same_device(sig_a, sig_b=sig_b)
    if sig_a.shape != sig_b.shape or sig_a.dim() < 1:
        raise RuntimeError("signatures must have the same shape (..., D)")
    D = sum(d ** k for k in range(1, depth + 1))
    if sig_a.size(-1) != D:
        raise RuntimeError(f"signature width {sig_a.size(-1)} is not the dense width {D} for d={d}, depth={depth}")
    desc = _load.ChenDesc()
    desc.dtype = _dtype_id(sig_a)
    desc.d, desc.depth = d, depth
    desc.rows = sig_a.numel() // D
    return desc


def _chen_product_cuda(sig_a, sig_b, depth, d):
    lib = _load.ensure_loaded()
    desc = _chen_desc(sig_a, sig_b, depth, d)
    a, b = sig_a.contiguous(), sig_b.contiguous()
    out = torch.empty_like(a)
    if out.numel() == 0:
        return out
    with torch.cuda.device(a.device):
        rc = lib.psig_chen_forward(ctypes.byref(desc), _ptr(a), _ptr(b), _ptr(out), _stream_ptr(a.device))
    _load.check(rc, "chen_product")
    return out


def _chen_product_backward_cuda(sig_a, sig_b, grad_out, depth, d):
    lib = _load.ensure_loaded()
    desc = _chen_desc(sig_a, sig_b, depth, d)
    if not grad_out.is_cuda:
        raise RuntimeError("grad_out must be CUDA")
    if grad_out.dtype != sig_a.dtype or grad_out.shape != sig_a.shape:
        raise RuntimeError("grad_out must match the signatures in dtype and shape")
    _check_same_device(sig_a, grad_out=grad_out)
    a, b, g = sig_a.contiguous(), sig_b.contiguous(), grad_out.contiguous()
    ga, gb = torch.empty_like(a), torch.empty_like(a)
    if ga.numel() == 0:
        return ga, gb
    with torch.cuda.device(a.device):
        rc = lib.psig_chen_backward(ctypes.byref(desc), _ptr(a), _ptr(b), _ptr(g), _ptr(ga), _ptr(gb),
                                    _stream_ptr(a.device))
    _load.check(rc, "chen_product_backward")
    return ga, gb


def _no_cpu(name):
    def impl(*args, **kwargs):
        raise NotImplementedError(
            f"pathsig_b200::{name} has a CUDA (sm_100a) implementation only; move the inputs to a CUDA device.")
    return impl


# --------------------------------------------------------------------------------------
# fake (meta) implementations
# --------------------------------------------------------------------------------------

def _fake_check_path(path: Tensor):
    torch._check(path.device.type in ("cuda", "meta"), lambda: "path must be a CUDA tensor")
    torch._check(path.dtype in (torch.float32, torch.float64), lambda: "path must be float32 or float64")
    torch._check(path.dim() == 3, lambda: "path must have shape (B, L, d)")
    B, L, d = path.shape
    torch._check(L >= 2, lambda: "path length must be at least 2")
    return B, L, d


def _fake_check_windows(windows: Tensor) -> None:
    torch._check(windows.device.type in ("cuda", "meta"), lambda: "windows must be a CUDA tensor")
    torch._check(windows.dtype in (torch.int32, torch.int64), lambda: "windows must be int32 or int64")
    torch._check(windows.dim() == 2 and windows.size(1) == 2, lambda: "windows must have shape (num_windows, 2)")


def _fake_check_projection(encoded_words: Tensor, level_sizes, depth: int) -> None:
    torch._check(encoded_words.device.type in ("cuda", "meta"), lambda: "encoded_words must be a CUDA tensor")
    torch._check(encoded_words.dtype == torch.int64, lambda: "encoded_words must be int64")
    torch._check(encoded_words.dim() == 1, lambda: "encoded_words must be 1D")
    torch._check(len(level_sizes) >= depth + 1, lambda: "level_sizes must cover at least depth + 1 entries")


def _fake_compute_signature(path, depth, alternative_projection, encoded_words, level_sizes, use_windows, windows):
    B, _, d = _fake_check_path(path)
    depth = int(depth)
    torch._check(1 <= depth <= 12, lambda: "depth must satisfy 1 <= depth <= 12")
    if use_windows:
        _fake_check_windows(windows)
    if alternative_projection:
        _fake_check_projection(encoded_words, level_sizes, depth)
    D = _row_width(d, depth, bool(alternative_projection), level_sizes)
    shape = (B, windows.size(0), D) if use_windows else (B, D)
    return path.new_empty(shape)


def _fake_signature_backward(path, signature, grad_signature, depth, alternative_projection, encoded_words,
                             level_sizes, use_windows, windows):
    _fake_check_path(path)
    torch._check(signature.dtype == path.dtype, lambda: "signature must have same dtype as path")
    torch._check(grad_signature.dtype == path.dtype, lambda: "grad_signature must have same dtype as path")
    torch._check(grad_signature.shape == signature.shape, lambda: "grad_signature must match signature shape")
    torch._check(1 <= int(depth) <= 12, lambda: "depth must satisfy 1 <= depth <= 12")
    if use_windows:
        _fake_check_windows(windows)
        torch._check(signature.dim() == 3 and windows.size(0) == signature.size(1),
                     lambda: "windows.size(0) must match signature num_windows")
    else:
        torch._check(signature.dim() == 2, lambda: "signature must be [B,S]")
    if alternative_projection:
        _fake_check_projection(encoded_words, level_sizes, int(depth))
    return torch.empty_like(path)


def _fake_sig_to_logsig(signature, depth, d, alternative_projection, encoded_words, level_sizes):
    torch._check(signature.device.type in ("cuda", "meta"), lambda: "signature must be a CUDA tensor")
    torch._check(signature.dtype in (torch.float32, torch.float64), lambda: "signature must be float32 or float64")
    depth = int(depth)
    torch._check(1 <= depth <= 12, lambda: "depth must satisfy 1 <= depth <= 12")
    torch._check(int(d) >= 1, lambda: "path dimension d must be >= 1")
    torch._check(signature.dim() in (2, 3), lambda: "signature must be 2D or 3D")
    if alternative_projection:
        _fake_check_projection(encoded_words, level_sizes, depth)
    desc = _log_desc(signature, depth, d, alternative_projection, encoded_words, level_sizes, fake=True)
    per_row = _load.ensure_loaded().psig_logsig_cache_size(ctypes.byref(desc))
    _load.check(per_row, "sig_to_logsig")
    cache = signature.new_empty(tuple(signature.shape[:-1]) + (int(per_row),))
    return torch.empty_like(signature), cache


def _fake_logsig_backward(signature, P_arr, grad_logsig, depth, alternative_projection, encoded_words, level_sizes):
    torch._check(signature.dtype in (torch.float32, torch.float64), lambda: "signature must be float32 or float64")
    torch._check(signature.dtype == grad_logsig.dtype, lambda: "signature must have same dtype as grad_logsig")
    torch._check(grad_logsig.dtype == P_arr.dtype, lambda: "grad_logsig must have same dtype as P_arr")
    depth = int(depth)
    torch._check(1 <= depth <= 12, lambda: "depth must satisfy 1 <= depth <= 12")
    torch._check(grad_logsig.shape == signature.shape, lambda: "grad_logsig must match signature shape")
    torch._check(signature.dim() in (2, 3) and P_arr.dim() == signature.dim(), lambda: "P must match signature rank")
    torch._check(tuple(P_arr.shape[:-1]) == tuple(signature.shape[:-1])
                 and P_arr.shape[-1] in (0, signature.shape[-1] * depth), lambda: "P must be [B,(W),S*depth]")
    if alternative_projection:
        _fake_check_projection(encoded_words, level_sizes, depth)
    return torch.empty_like(signature)


def _fake_logsig_projected(signature, depth, d, top_words, level_sizes, lower_columns):
    torch._check(signature.dtype in (torch.float32, torch.float64), lambda: "signature must be float32 or float64")
    torch._check(signature.dim() in (2, 3), lambda: "signature must be 2D or 3D")
    torch._check(1 <= int(depth) <= 12, lambda: "depth must satisfy 1 <= depth <= 12")
    torch._check(len(level_sizes) >= int(depth) + 1, lambda: "level_sizes must have entries up to depth")
    torch._check(lower_columns.dim() == 1, lambda: "lower_columns must be 1D")
    width = lower_columns.shape[0] + int(level_sizes[int(depth)])
    return signature.new_empty(tuple(signature.shape[:-1]) + (width,))


def _fake_logsig_projected_backward(signature, grad_out, depth, d, top_words, level_sizes, lower_columns):
    torch._check(grad_out.dtype == signature.dtype, lambda: "grad_out must have same dtype as signature")
    return torch.empty_like(signature)


def _fake_chen_product(sig_a, sig_b, depth, d):
    torch._check(sig_a.dtype in (torch.float32, torch.float64), lambda: "signatures must be float32 or float64")
    torch._check(sig_a.dtype == sig_b.dtype, lambda: "signatures must have the same dtype")
    torch._check(sig_a.shape == sig_b.shape, lambda: "signatures must have the same shape")
    torch._check(1 <= int(depth) <= 12, lambda: "depth must satisfy 1 <= depth <= 12")
    return torch.empty_like(sig_a)


def _fake_chen_product_backward(sig_a, sig_b, grad_out, depth, d):
    torch._check(grad_out.shape == sig_a.shape, lambda: "grad_out must match the signatures")
    return torch.empty_like(sig_a), torch.empty_like(sig_b)


# --------------------------------------------------------------------------------------
# registration
# --------------------------------------------------------------------------------------

_IMPLS = {
    "compute_signature": (_compute_signature_cuda, _fake_compute_signature),
    "signature_backward": (_signature_backward_cuda, _fake_signature_backward),
    "sig_to_logsig": (_sig_to_logsig_cuda, _fake_sig_to_logsig),
    "logsig_backward": (_logsig_backward_cuda, _fake_logsig_backward),
    "logsig_projected": (_logsig_projected_cuda, _fake_logsig_projected),
    "logsig_projected_backward": (_logsig_projected_backward_cuda, _fake_logsig_projected_backward),
    "chen_product": (_chen_product_cuda, _fake_chen_product),
    "chen_product_backward": (_chen_product_backward_cuda, _fake_chen_product_backward),
}
_libraries = {}  # namespace -> torch.library.Library (kept alive for the life of the process)


def register_namespace(ns: str) -> None:
    """Define and implement the four operators under ``torch.ops.<ns>``."""
    if ns in _libraries:
        return
    lib = torch.library.Library(ns, "FRAGMENT")
    for name, schema in _SCHEMAS.items():
        lib.define(name + schema, tags=(torch.Tag.pt2_compliant_tag,))
        cuda_impl, fake_impl = _IMPLS[name]
        lib.impl(name, cuda_impl, "CUDA")
        lib.impl(name, _no_cpu(name), "CPU")
        torch.library.register_fake(f"{ns}::{name}", fake_impl, lib=lib)

    def setup_sig(ctx, inputs, output):
        path, depth, alt, encoded_words, level_sizes, use_windows, windows = inputs
        ctx.save_for_backward(path, output, windows, encoded_words)
        ctx.depth, ctx.alt = int(depth), bool(alt)
        ctx.level_sizes, ctx.use_windows = level_sizes, bool(use_windows)

    def backward_sig(ctx, grad_out):
        path, signature, windows, encoded_words = ctx.saved_tensors
        grad_path = None
        if ctx.needs_input_grad[0]:
            grad_path = getattr(torch.ops, ns).signature_backward.default(
                path, signature, grad_out, ctx.depth, ctx.alt, encoded_words, ctx.level_sizes, ctx.use_windows,
                windows)
        return grad_path, None, None, None, None, None, None

    def setup_log(ctx, inputs, output):
        signature, depth, d, alt, encoded_words, level_sizes = inputs
        ctx.save_for_backward(signature, output[1], encoded_words)
        ctx.depth, ctx.alt, ctx.level_sizes = int(depth), bool(alt), level_sizes

    def backward_log(ctx, grad_logsig, grad_cache):
        signature, cache, encoded_words = ctx.saved_tensors
        grad_sig = None
        if ctx.needs_input_grad[0]:
            grad_sig = getattr(torch.ops, ns).logsig_backward.default(
                signature, cache, grad_logsig, ctx.depth, ctx.alt, encoded_words, ctx.level_sizes)
        return grad_sig, None, None, None, None, None

    def setup_logproj(ctx, inputs, output):
        signature, depth, d, top_words, level_sizes, lower_columns = inputs
        ctx.save_for_backward(signature, top_words, lower_columns)
        ctx.depth, ctx.d, ctx.level_sizes = int(depth), int(d), level_sizes

    def backward_logproj(ctx, grad_out):
        signature, top_words, lower_columns = ctx.saved_tensors
        grad_sig = None
        if ctx.needs_input_grad[0]:
            grad_sig = getattr(torch.ops, ns).logsig_projected_backward.default(
                signature, grad_out, ctx.depth, ctx.d, top_words, ctx.level_sizes, lower_columns)
        return grad_sig, None, None, None, None, None

    def setup_chen(ctx, inputs, output):
        sig_a, sig_b, depth, d = inputs
        ctx.save_for_backward(sig_a, sig_b)
        ctx.depth, ctx.d = int(depth), int(d)

    def backward_chen(ctx, grad_out):
        sig_a, sig_b = ctx.saved_tensors
        grad_a = grad_b = None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            grad_a, grad_b = getattr(torch.ops, ns).chen_product_backward.default(sig_a, sig_b, grad_out, ctx.depth,
                                                                                  ctx.d)
        return (grad_a if ctx.needs_input_grad[0] else None, grad_b if ctx.needs_input_grad[1] else None, None,
                None)

    def setup_chen_bwd(ctx, inputs, output):
        sig_a, sig_b, grad_out, depth, d = inputs
        ctx.save_for_backward(sig_a, sig_b, grad_out)
        ctx.depth, ctx.d = int(depth), int(d)

    def backward_chen_bwd(ctx, gga, ggb):
        # The product is bilinear, so its adjoint is linear in each of (a, grad_out) and (b, grad_out):
        #   grad_a = adj_a(b, g), grad_b = adj_b(a, g)  with  <adj_a(b, g), x> = <g, x (x) b - b> etc.
        # Second derivatives are composed from the same two operators.
        sig_a, sig_b, grad_out = ctx.saved_tensors
        op = getattr(torch.ops, ns)
        zero = torch.zeros_like(sig_a)
        ga = gb = gg = None
        # d/d(grad_out): grad_a = J_a^T g, so the adjoint wrt g is J_a gga (+ J_b ggb)
        #   J_a x = x (x) b - b  (the part of the product linear in a), J_b y = a (x) y - a
        if ctx.needs_input_grad[2]:
            gg = (op.chen_product.default(gga, sig_b, ctx.depth, ctx.d) - sig_b
                  + op.chen_product.default(sig_a, ggb, ctx.depth, ctx.d) - sig_a)
        # d/db of <gga, adj_a(b, g)> = adj_b(gga, g) - g (the bilinear part only); likewise for a
        if ctx.needs_input_grad[1]:
            gb = op.chen_product_backward.default(gga, zero, grad_out, ctx.depth, ctx.d)[1] - grad_out
        if ctx.needs_input_grad[0]:
            ga = op.chen_product_backward.default(zero, ggb, grad_out, ctx.depth, ctx.d)[0] - grad_out
        return ga, gb, gg, None, None

    torch.library.register_autograd(f"{ns}::chen_product", backward_chen, setup_context=setup_chen, lib=lib)
    torch.library.register_autograd(f"{ns}::chen_product_backward", backward_chen_bwd,
                                    setup_context=setup_chen_bwd, lib=lib)
    torch.library.register_autograd(f"{ns}::compute_signature", backward_sig, setup_context=setup_sig, lib=lib)
    torch.library.register_autograd(f"{ns}::sig_to_logsig", backward_log, setup_context=setup_log, lib=lib)
    torch.library.register_autograd(f"{ns}::logsig_projected", backward_logproj, setup_context=setup_logproj, lib=lib)
    _libraries[ns] = lib


register_namespace(NAMESPACE)
_ops = getattr(torch.ops, NAMESPACE)


def compute_signature(path: Tensor, depth: int, alternative_projection: bool, encoded_words: Tensor,
                      level_sizes: List[int], use_windows: bool, windows: Tensor) -> Tensor:
    """(Windowed / projected) signature of ``path``; differentiable wrt ``path``."""
    return _ops.compute_signature.default(path, depth, alternative_projection, encoded_words, level_sizes,
                                          use_windows, windows)


def sig_to_logsig(signature: Tensor, depth: int, d: int, alternative_projection: bool, encoded_words: Tensor,
                  level_sizes: List[int]) -> Tuple[Tensor, Tensor]:
    """Signature (hybrid layout) -> (log-signature, cache); differentiable wrt ``signature``."""
    return _ops.sig_to_logsig.default(signature, depth, d, alternative_projection, encoded_words, level_sizes)


def signature_backward(path: Tensor, signature: Tensor, grad_signature: Tensor, depth: int,
                       alternative_projection: bool, encoded_words: Tensor, level_sizes: List[int],
                       use_windows: bool, windows: Tensor) -> Tensor:
    """dL/dpath from dL/dsignature."""
    return _ops.signature_backward.default(path, signature, grad_signature, depth, alternative_projection,
                                           encoded_words, level_sizes, use_windows, windows)


def logsig_projected(signature: Tensor, depth: int, d: int, top_words: Tensor, level_sizes: List[int],
                     lower_columns: Tensor) -> Tensor:
    """Signature (hybrid layout) -> projected log-signature: the words of the degrees below ``depth`` at
    ``lower_columns`` followed by the whole top degree, in one kernel.  Differentiable wrt ``signature``."""
    return _ops.logsig_projected.default(signature, depth, d, top_words, level_sizes, lower_columns)


def logsig_projected_backward(signature: Tensor, grad_out: Tensor, depth: int, d: int, top_words: Tensor,
                              level_sizes: List[int], lower_columns: Tensor) -> Tensor:
    """dL/dsignature from the gradient of :func:`logsig_projected`'s output."""
    return _ops.logsig_projected_backward.default(signature, grad_out, depth, d, top_words, level_sizes,
                                                  lower_columns)


def chen_product(sig_a: Tensor, sig_b: Tensor, depth: int, d: int) -> Tensor:
    """Truncated tensor product of two dense signatures ``(..., D)`` of ``d`` channels up to ``depth``:
    the signature of the first path followed by the second (Chen's identity).  Differentiable (twice)
    wrt both arguments.  Not an operator of the reference."""
    return _ops.chen_product.default(sig_a, sig_b, depth, d)


def chen_product_backward(sig_a: Tensor, sig_b: Tensor, grad_out: Tensor, depth: int, d: int) -> Tuple[Tensor, Tensor]:
    """(dL/dsig_a, dL/dsig_b) from dL/d(chen_product)."""
    return _ops.chen_product_backward.default(sig_a, sig_b, grad_out, depth, d)


def logsig_backward(signature: Tensor, P_arr: Tensor, grad_logsig: Tensor, depth: int,
                    alternative_projection: bool, encoded_words: Tensor, level_sizes: List[int]) -> Tensor:
    """dL/dsignature from dL/dlogsig, using the cache returned by :func:`sig_to_logsig`."""
    return _ops.logsig_backward.default(signature, P_arr, grad_logsig, depth, alternative_projection,
                                        encoded_words, level_sizes)
