"""Operator layer: the reference's four operators, served by the B200 CUDA library.

Host-side mirror of ``src/pathsig/ops.py`` of the reference: thin wrappers around the dispatcher
entries, the same fake (meta) shape functions (``ops.py:59-84, 101-123, 152-179, 197-227``) and the
same autograd wiring (``ops.py:231-297``).  The operators themselves -- the four schemas of
``src/pathsig/bindings.cpp:9-63`` plus the projected log-signature and the Chen product, registered
for the CUDA key only -- live in the compiled library ``libpathsig_b200_torch.so``
(``csrc/torch_binding.cpp``), which validates like the reference launchers, allocates outputs with
torch's caching allocator and hands raw pointers plus the current stream to the C ABI
(``include/pathsig_b200.h``).  torch is used for memory, streams and dispatch only.

The operators are registered in the namespace ``pathsig_b200`` so that this package and a
build of the reference (namespace ``pathsig``) can live in one process, which is how the
parity tests compare them.  :func:`register_namespace` defines the same operators under
another namespace (``pathsig_b200.install_as_pathsig`` uses it for ``pathsig``), forwarding to
the compiled ones.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

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

# Kernel family used by the signature operators: _load.ALGO_AUTO / ALGO_GENERIC / ALGO_TILED / ALGO_CLOSURE.
# Tests flip it to compare the register-tiled kernels with the generic ones.  The compiled operator layer
# holds the value it acts on; this copy serves the shape queries made from Python.
_algo = _load.ALGO_AUTO
CLOSURE_ALGOS = (_load.ALGO_AUTO, _load.ALGO_CLOSURE)   # selections under which a word set can get generated kernels


def closure_kernels_available() -> bool:
    """Whether the run-time compiler the prefix-closure kernels need can be loaded on this machine."""
    return bool(_load.ensure_loaded().psig_closure_available())


def set_algorithm(name: str) -> None:
    """Select the signature kernel family: "auto", "generic", "tiled" or "closure"."""
    global _algo
    _algo = {"auto": _load.ALGO_AUTO, "generic": _load.ALGO_GENERIC, "tiled": _load.ALGO_TILED,
             "closure": _load.ALGO_CLOSURE}[name]
    _load.ensure_binding_loaded().psig_torch_set_algorithm(_algo)


# --------------------------------------------------------------------------------------
# helpers of the shape queries
# --------------------------------------------------------------------------------------

def _dtype_id(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return _load.PSIG_F32
    if t.dtype == torch.float64:
        return _load.PSIG_F64
    raise RuntimeError("path must be float32 or float64")


def _log_desc_for_shapes(signature: Tensor, depth: int, d: int, alt: bool, encoded_words: Tensor,
                         level_sizes: Sequence[int]) -> _load.LogDesc:
    """``PsigLogDesc`` for host-only shape queries (fake tensors): no device pointer is read."""
    depth, d = int(depth), int(d)
    if not (1 <= depth <= _load.MAX_DEPTH):
        raise RuntimeError("depth must be in [1,12]")
    if d < 1:
        raise RuntimeError("d must be >= 1")
    desc = _load.LogDesc()
    desc.dtype = _dtype_id(signature)
    desc.d, desc.depth = d, depth
    desc.algo = _algo
    desc.rows = 0
    desc.top_size = d ** depth
    if alt:
        if len(level_sizes) < depth + 1:
            raise RuntimeError("level_sizes must have entries up to depth")
        desc.top_size = int(level_sizes[depth])
        if desc.top_size != d ** depth:
            desc.top_words = 1 if encoded_words.numel() > 0 else None  # non-null marker, never read
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
    desc = _log_desc_for_shapes(signature, depth, d, alternative_projection, encoded_words, level_sizes)
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

_FAKES = {
    "compute_signature": _fake_compute_signature,
    "signature_backward": _fake_signature_backward,
    "sig_to_logsig": _fake_sig_to_logsig,
    "logsig_backward": _fake_logsig_backward,
    "logsig_projected": _fake_logsig_projected,
    "logsig_projected_backward": _fake_logsig_projected_backward,
    "chen_product": _fake_chen_product,
    "chen_product_backward": _fake_chen_product_backward,
}
_libraries = {}  # namespace -> torch.library.Library or True (kept alive for the life of the process)


def _forward_to_compiled(name):
    compiled = getattr(getattr(torch.ops, NAMESPACE), name).default

    def impl(*args):
        return compiled(*args)
    return impl


def register_namespace(ns: str) -> None:
    """Fake implementations and autograd formulas of the operators under ``torch.ops.<ns>``.

    For ``pathsig_b200`` the operators themselves (schemas and CUDA implementations) come from the
    compiled library ``libpathsig_b200_torch.so``; any other namespace (``pathsig``, for code written
    against the reference) is defined here and forwards to them.
    """
    if ns in _libraries:
        return
    lib = None
    if ns == NAMESPACE:
        _load.ensure_binding_loaded()
        for name, fake_impl in _FAKES.items():
            torch.library.register_fake(f"{ns}::{name}", fake_impl)
    else:
        lib = torch.library.Library(ns, "FRAGMENT")
        for name, schema in _SCHEMAS.items():
            lib.define(name + schema, tags=(torch.Tag.pt2_compliant_tag,))
            lib.impl(name, _forward_to_compiled(name), "CUDA")
            torch.library.register_fake(f"{ns}::{name}", _FAKES[name], lib=lib)

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
    _libraries[ns] = lib if lib is not None else True


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
