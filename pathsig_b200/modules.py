"""``Signature`` and ``LogSignature`` modules: the user-facing API.

Host-side mirror of the reference's ``src/pathsig/modules.py``: keyword-only ``depth``,
``projection`` and ``windows``; the same argument checks and exception types
(``modules.py:10-38``); the same buffer names and persistence, so a reference ``state_dict``
loads (``_windows``, ``_encoded_words``, ``_top_words``, ``_indices_from_sig``,
``modules.py:54-59, 84-110``); the same output shapes ``(B, D)`` / ``(B, W, D)``.

``LogSignature`` keeps the reference's composition (``modules.py:112-135``): signature in the
hybrid layout (dense degrees below ``depth``, projected top degree), tensor logarithm in word
coordinates, then the column selection of the projected case.  Where the row fits the shared-memory
log-signature kernels, logarithm and selection are one kernel (``ops.logsig_projected``): only the
requested columns are written, and the backward starts from the projected gradient; otherwise the
selection is a stock gather after ``sig_to_logsig`` as in the reference.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import nn

from . import ops as ops_module
from .ops import compute_signature, logsig_projected, logsig_projected_supported, sig_to_logsig
from .projections import _default_device

_MAX_DEPTH = 12


def _checked_depth(depth: int) -> int:
    if not (1 <= depth <= _MAX_DEPTH):
        raise ValueError("depth must satisfy 1 <= depth <= 12.")
    return depth


def _window_buffer(windows: Optional[torch.Tensor]) -> Tuple[bool, torch.Tensor]:
    """(use_windows, contiguous int32 (W, 2) buffer); an empty (0, 2) buffer when unused."""
    if windows is None:
        return False, torch.empty((0, 2), dtype=torch.int32, device=_default_device())
    if windows.device.type != "cuda":
        raise TypeError("windows must be a CUDA tensor.")
    if windows.dim() != 2 or windows.size(1) != 2:
        raise TypeError("windows must have shape [num_windows, 2].")
    if windows.dtype not in (torch.int32, torch.int64):
        raise TypeError("windows must have dtype int32 or int64.")
    return True, windows.contiguous().to(dtype=torch.int32)


def _projection_words(projection) -> Tuple[bool, Optional[torch.Tensor]]:
    if projection is None:
        return False, None
    words = projection.encoded_words
    if words.device.type != "cuda" or words.dtype != torch.int64 or words.dim() != 1:
        raise TypeError("projection.encoded_words must be a 1D CUDA int64 tensor.")
    return True, words.contiguous()


def _no_words() -> torch.Tensor:
    return torch.empty(0, dtype=torch.int64, device=_default_device())


def _host_codes(projection, words: torch.Tensor) -> List[int]:
    codes = getattr(projection, "_host_codes", None)
    return list(codes) if codes is not None else words.tolist()


def _check_codes(codes: List[int], level_sizes: List[int], d: int, depth: int) -> None:
    """Every stored code of an incomplete degree k must be a word of that degree: 0 <= code < d**k.
    The kernels index dense images of a degree by these codes, so a bad code (a hand-made projection,
    a state_dict from another configuration) would read or write out of bounds on the device."""
    used = 0
    for k in range(1, depth + 1):
        size, full = int(level_sizes[k]), d ** k
        if size == full:
            continue
        level = codes[used: used + size]
        if len(level) < size:
            raise ValueError(f"encoded_words holds {len(codes)} codes, fewer than level_sizes requires.")
        if level and (min(level) < 0 or max(level) >= full):
            raise ValueError(f"encoded_words has a code outside [0, {d}**{k}) at degree {k}.")
        used += size


_MAX_CLOSURE_WIDTH = 16384   # largest row the prefix-closure kernels are generated for
_CLOSURE_MIN_UNITS = 256     # ... and the work below which the library does not select them
_CLOSURE_MIN_WORK = 2.0e7
_MAX_CLOSURE_GROWTH = 4       # the closed row may be at most this many times as wide as the requested one


def _prefix_closure(codes: List[int], level_sizes: List[int], d: int, depth: int):
    """The requested words together with all their prefixes, in the row layout of the operators.

    Returns ``(closure_codes, closure_level_sizes, columns)``: the codes of the incomplete degrees of the
    closed set (ascending within a degree), its level sizes, and for every column of the requested row its
    column in the closed row; or ``None`` when the set is already closed, lists a word twice, would be
    wider than the kernels generated for word sets accept, or more than four times as wide as the request."""
    requested: List[Optional[List[int]]] = [None] * (depth + 1)   # None: complete degree
    used = 0
    for k in range(1, depth + 1):
        size = int(level_sizes[k])
        if size != d ** k:
            requested[k] = codes[used: used + size]
            used += size
            if len(set(requested[k])) != size:
                return None
    closed: List[Optional[set]] = [None if requested[k] is None else set(requested[k]) for k in range(depth + 1)]
    closed[0] = set()
    for k in range(depth, 1, -1):
        if closed[k - 1] is None:
            continue
        if closed[k] is None:
            closed[k - 1] = None      # every word of degree k is wanted: so is every word below it
            continue
        closed[k - 1].update(c // d for c in closed[k])
        if len(closed[k - 1]) == d ** (k - 1):
            closed[k - 1] = None
    sizes = [0] + [d ** k if closed[k] is None else len(closed[k]) for k in range(1, depth + 1)]
    requested_width = sum(int(v) for v in level_sizes[1: depth + 1])
    if sizes == [0] + [int(v) for v in level_sizes[1: depth + 1]] or sum(sizes) > _MAX_CLOSURE_WIDTH:
        return None
    if sum(sizes) > _MAX_CLOSURE_GROWTH * requested_width:
        return None   # the saved signature would cost much more memory than the one that was asked for
    closure_codes: List[int] = []
    columns: List[int] = []
    offset = 0
    for k in range(1, depth + 1):
        if closed[k] is None:
            position = None
        else:
            ordered = sorted(closed[k])
            closure_codes.extend(ordered)
            position = {c: i for i, c in enumerate(ordered)}
        wanted = range(d ** k) if requested[k] is None else requested[k]
        columns.extend(offset + (c if position is None else position[c]) for c in wanted)
        offset += sizes[k]
    return closure_codes, sizes, columns


class Signature(nn.Module):
    """Truncated signature of a batch of paths ``(B, L, d)`` -> ``(B, D)`` or ``(B, W, D)``.

    With a projection whose words have prefixes that are not requested themselves, large enough problems
    are evaluated on the prefix closure of the word set and the requested columns are selected from that
    row: the kernels generated for a word set compute every prefix anyway, and with all of them in the
    saved signature the backward pass does not have to rebuild them with a second forward sweep (the
    reference recomputes them inside its backward kernel, ``recompute_sig`` in
    ``src/pathsig/backward/sig_backward_kernels.cu:204-318``)."""

    def __init__(self, *, depth: int, projection=None, windows=None):
        super().__init__()
        self.depth = _checked_depth(depth)
        self.projection = projection
        self.alternative_projection, words = _projection_words(projection)
        self.use_windows, window_buffer = _window_buffer(windows)
        self.register_buffer("_windows", window_buffer, persistent=self.use_windows)
        self.register_buffer("_encoded_words", words if self.alternative_projection else _no_words(),
                             persistent=self.alternative_projection)
        self._level_sizes: List[int] = projection.level_sizes if self.alternative_projection else []
        self._closure_sizes: Optional[List[int]] = None
        if self.alternative_projection:
            codes = _host_codes(projection, words)
            _check_codes(codes, self._level_sizes, int(projection.path_dim), self.depth)
            self._refresh_closure(codes)
            self.register_load_state_dict_post_hook(_recheck_loaded_words)

    def _refresh_closure(self, codes: List[int]) -> None:
        """Derived from the word codes actually in the buffer (re-derived after load_state_dict)."""
        d = int(self.projection.path_dim)
        device = self._encoded_words.device
        plan = _prefix_closure(codes, self._level_sizes, d, self.depth) if d <= 64 else None
        if plan is not None and not ops_module.closure_kernels_available():
            plan = None
        self._closure_sizes = None if plan is None else plan[1]
        self.register_buffer("_closure_words", torch.tensor([] if plan is None else plan[0], dtype=torch.int64,
                                                            device=device), persistent=False)
        self.register_buffer("_closure_columns", torch.tensor([] if plan is None else plan[2], dtype=torch.int64,
                                                              device=device), persistent=False)

    def _closure_pays(self, path: torch.Tensor) -> bool:
        """The library's own rule for selecting the kernels generated for a word set, on the closed row."""
        if self._closure_sizes is None or path.dim() != 3 or ops_module._algo not in ops_module.CLOSURE_ALGOS:
            return False
        units = path.shape[0] * (self._windows.shape[0] if self.use_windows else 1)
        work = float(units) * float(path.shape[1] - 1) * float(sum(self._closure_sizes))
        return units >= _CLOSURE_MIN_UNITS and work >= _CLOSURE_MIN_WORK

    def forward(self, path: torch.Tensor) -> torch.Tensor:
        if self._closure_pays(path):
            closed = compute_signature(path, self.depth, True, self._closure_words, self._closure_sizes,
                                       self.use_windows, self._windows)
            return _SelectColumns.apply(closed, self._closure_columns)
        return compute_signature(path, self.depth, self.alternative_projection, self._encoded_words,
                                 self._level_sizes, self.use_windows, self._windows)


def _recheck_loaded_words(module, incompatible_keys) -> None:
    """After load_state_dict: the word codes now in the buffers must still be words of this projection."""
    codes = module._encoded_words.tolist()
    _check_codes(codes, module._level_sizes, int(module.projection.path_dim), module.depth)
    if isinstance(module, Signature):
        module._refresh_closure(codes)
    if isinstance(module, LogSignature):
        top = module._top_words.tolist()
        full = int(module.projection.path_dim) ** module.depth
        if top and (min(top) < 0 or max(top) >= full):
            raise ValueError("_top_words has a code outside the top degree.")
        module._refresh_columns()


class _SelectColumns(torch.autograd.Function):
    """``x.index_select(-1, index)`` for an index without repeats.  Autograd's own backward of
    ``index_select`` is an ``index_add_`` (float atomics, run-dependent last bits, 4x the time of the
    forward at the benchmark shape); without repeats a plain scatter into zeros is the same adjoint."""

    @staticmethod
    def forward(ctx, x, index):
        ctx.save_for_backward(index)
        ctx.width = x.shape[-1]
        return x.index_select(-1, index)

    @staticmethod
    def backward(ctx, grad):
        (index,) = ctx.saved_tensors
        full = grad.new_zeros(grad.shape[:-1] + (ctx.width,))
        full.index_copy_(-1, index, grad)
        return full, None


class LogSignature(nn.Module):
    """Truncated log-signature in word coordinates (optionally projected, optionally windowed)."""

    def __init__(self, *, depth: int, projection=None, windows=None):
        super().__init__()
        self.depth = _checked_depth(depth)
        self.projection = projection
        self.alternative_projection, words = _projection_words(projection)
        self.use_windows, window_buffer = _window_buffer(windows)
        self.register_buffer("_windows", window_buffer, persistent=self.use_windows)

        if not self.alternative_projection:
            for name in ("_encoded_words", "_top_words", "_indices_from_sig"):
                self.register_buffer(name, _no_words(), persistent=False)
            self._level_sizes: List[int] = []
            self._ext_level_sizes: List[int] = []
            return

        self.register_buffer("_encoded_words", words, persistent=True)
        self._level_sizes = projection.level_sizes
        d = self._path_dim = int(projection.path_dim)

        # The log needs every word below the top degree, so those degrees are computed dense;
        # only the top degree stays projected.  Its codes are the tail of encoded_words.
        explicit_below_top = sum(self._level_sizes[k] for k in range(1, self.depth)
                                 if self._level_sizes[k] != d ** k)
        self.register_buffer("_top_words", words[explicit_below_top:], persistent=True)
        self._ext_level_sizes = [0] + [d ** k for k in range(1, self.depth)] + [int(self._level_sizes[self.depth])]
        _check_codes(_host_codes(projection, words), self._level_sizes, d, self.depth)
        host_columns = projection.logsig_indices().tolist()
        columns = torch.tensor(host_columns, dtype=torch.int64, device=words.device)
        self.register_buffer("_indices_from_sig", columns, persistent=True)
        self._refresh_columns(host_columns)
        self.register_load_state_dict_post_hook(_recheck_loaded_words)

    def _refresh_columns(self, host_columns: Optional[List[int]] = None) -> None:
        """Facts derived from the column index actually in the buffer (re-derived after load_state_dict)."""
        if host_columns is None:
            host_columns = self._indices_from_sig.tolist()
        width = sum(self._ext_level_sizes)
        if host_columns and (min(host_columns) < 0 or max(host_columns) >= width):
            raise ValueError(f"_indices_from_sig has a column outside [0, {width}).")
        # a projection that lists a word twice selects a column twice: those gradients must add up
        self._columns_repeat = len(set(host_columns)) != len(host_columns)
        # The fused logarithm + selection writes "requested words below the top degree, then the whole top
        # degree": that is the layout logsig_indices() gives; an index replaced through load_state_dict
        # may not have it, and then the stock gather serves it.
        lower = sum(self._ext_level_sizes[: self.depth])
        top = int(self._ext_level_sizes[self.depth])
        n_low = len(host_columns) - top
        self._fusable = (n_low >= 0 and host_columns[n_low:] == list(range(lower, lower + top))
                         and all(c < lower for c in host_columns[:n_low]))
        device = self._indices_from_sig.device
        self.register_buffer("_lower_columns", torch.tensor(host_columns[:n_low] if self._fusable else [],
                                                            dtype=torch.int64, device=device), persistent=False)
        self._fused_ok = {}

    def forward(self, path: torch.Tensor) -> torch.Tensor:
        if self.alternative_projection:
            d = self._path_dim
            level_sizes = self._ext_level_sizes
        else:
            d = int(path.shape[-1])
            level_sizes = [0] + [d ** k for k in range(1, self.depth + 1)]
        sig = compute_signature(path, self.depth, self.alternative_projection, self._top_words, level_sizes,
                                self.use_windows, self._windows)
        if self.alternative_projection and self._fusable:
            key = (sig.dtype, ops_module._algo)  # the kernel family is a property of dtype, shape and selected algorithm
            fused = self._fused_ok.get(key)
            if fused is None:
                fused = self._fused_ok[key] = logsig_projected_supported(sig.dtype, self.depth, d, level_sizes)
            if fused:
                return logsig_projected(sig, self.depth, d, self._top_words, level_sizes, self._lower_columns)
        logsig, _ = sig_to_logsig(sig, self.depth, d, self.alternative_projection, self._top_words, level_sizes)
        if not self.alternative_projection:
            return logsig
        index = self._indices_from_sig.to(logsig.device)
        if self._columns_repeat:
            return logsig.index_select(dim=-1, index=index)
        return _SelectColumns.apply(logsig, index)
