"""Signature / log-signature projections: which word coordinates an operator returns.

Host-side mirror of the reference's ``src/pathsig/projections.py`` (same public names,
argument meaning, attribute names and error behaviour):

* ``Projection`` base: ``encoded_words``, ``level_sizes``, ``sig_size``, ``logsig_indices()``
  (``projections.py:8-50``) and the argument checks of ``_validate_inputs`` (``52-74``).
* ``WordsProjection`` (``76-130``), ``AnisotropicProjection`` (``132-223``),
  ``LyndonProjection`` (``225-272``) and the ``projections`` namespace (``274-298``).

Conventions shared with the kernels: a word ``(w_0, …, w_{n-1})`` over letters ``0..d-1`` is
stored as the base-``d`` integer ``sum_i w_i d^(n-1-i)`` (first letter most significant);
``level_sizes[k]`` is the number of words kept at degree ``k`` (entry 0 unused);
``encoded_words`` holds the codes of the degrees that are *not* complete, concatenated by
degree.  A complete degree is implicit and always in lexicographic (= code) order.

All work here is plain Python on small lists; the result is uploaded once.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple, Union

import torch

_MAX_DEPTH = 12
_WORD_BITS = 64
# Largest d for which d**n still fits int64 when n is a power of two (the only depths where
# the base-d overflow limit is tighter than the letter-packing limit).
_INT64_BASE_LIMIT = {2: 3037000499, 4: 55108, 8: 234}


def _default_device() -> torch.device:
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def _check_arguments(d: int, depth: int, full_levels: Iterable[int]) -> None:
    if d <= 1:
        raise ValueError(f"path_dim must be >= 2 (got {d}).")
    if not (1 <= depth <= _MAX_DEPTH):
        raise ValueError(f"depth must satisfy 1 <= depth <= {_MAX_DEPTH} (got {depth}).")
    full_levels = list(full_levels)
    if full_levels and (min(full_levels) < 1 or max(full_levels) > depth):
        raise ValueError("full_levels entries must satisfy 1 <= level <= depth.")

    n_eff = max(depth, 2)  # depth 1 is held to the length-2 limit
    bits_needed = (d - 1).bit_length()
    bits_available = _WORD_BITS // n_eff
    if bits_needed > bits_available:
        raise ValueError(f"Maximum path_dim for depth={depth} is {1 << bits_available}, but got path_dim={d}.")
    limit = _INT64_BASE_LIMIT.get(n_eff)
    if limit is not None and d > limit:
        raise ValueError(f"Maximum path_dim for depth={depth} is {limit}, but got path_dim={d}.")


def _encode(word: Iterable[int], d: int) -> Tuple[int, int]:
    code, n = 0, 0
    for letter in word:
        if not (0 <= letter < d):
            raise ValueError("Invalid letter encountered in a word, ensure all letters satisfy 0 <= letter < d.")
        code = code * d + int(letter)
        n += 1
    return code, n


def _strip_complete_levels(per_level: List[List[int]], d: int, forced_full: Iterable[int]) -> Tuple[List[int], List[int]]:
    """Per-degree code lists -> (codes of incomplete degrees, level_sizes)."""
    forced_full = set(forced_full)
    sizes = [0] * len(per_level)
    codes: List[int] = []
    for n in range(1, len(per_level)):
        full = d ** n
        if n in forced_full or len(per_level[n]) == full:
            sizes[n] = full
        else:
            sizes[n] = len(per_level[n])
            codes.extend(per_level[n])
    return codes, sizes


class Projection:
    """Base class for (log-)signature projections."""

    path_dim: int
    depth: int
    _codes: torch.Tensor
    _level_sizes: List[int]

    @property
    def encoded_words(self) -> torch.Tensor:
        """Base-d codes of the words of the incomplete degrees (1-D int64)."""
        return self._codes

    @property
    def level_sizes(self) -> List[int]:
        """Number of words kept per degree (index 0 unused)."""
        return self._level_sizes

    @property
    def sig_size(self) -> int:
        """Width of the projected signature."""
        return sum(self._level_sizes[1: self.depth + 1])

    def _finish(self, codes: List[int], sizes: List[int], device) -> None:
        self._level_sizes = sizes
        self._host_codes = list(codes)  # host copy: consumers validate and index without a device read
        self._codes = torch.tensor(codes, dtype=torch.int64, device=device or _default_device())

    def logsig_indices(self) -> torch.Tensor:
        """Columns to keep from the hybrid log-signature layout.

        The log-signature operator works on "dense degrees 1..depth-1, projected top degree";
        this returns, for every kept word, its column in that layout.
        """
        d = self.path_dim
        codes = self._host_codes if hasattr(self, "_host_codes") else self._codes.tolist()
        columns: List[int] = []
        dense_offset, used = 0, 0
        for n in range(1, self.depth):
            full = d ** n
            size = self._level_sizes[n]
            if size == full:
                columns.extend(range(dense_offset, dense_offset + full))
            else:
                columns.extend(dense_offset + c for c in codes[used: used + size])
                used += size
            dense_offset += full
        columns.extend(range(dense_offset, dense_offset + self._level_sizes[self.depth]))
        return torch.tensor(columns, dtype=torch.int64, device=self._codes.device)


class WordsProjection(Projection):
    """Projection onto an explicit list of words (non-decreasing length)."""

    def __init__(self, words: Iterable[Iterable[int]], depth: int, path_dim: int,
                 full_levels: Iterable[int] = (), *, device=None) -> None:
        self.path_dim = int(path_dim)
        self.depth = int(depth)
        self._full_levels = {int(n) for n in full_levels}
        _check_arguments(self.path_dim, self.depth, self._full_levels)

        per_level: List[List[int]] = [[] for _ in range(self.depth + 1)]
        longest = 0
        for word in words:
            code, n = _encode(word, self.path_dim)
            if n < longest:
                raise ValueError("Words must be non-decreasing in length.")
            if n > self.depth:
                break  # words beyond the truncation depth end the list
            longest = n
            per_level[n].append(code)
        for n in self._full_levels:
            if per_level[n]:
                raise ValueError(f"Degree {n} is marked as full, but explicit words were also provided for that level.")
        codes, sizes = _strip_complete_levels(per_level, self.path_dim, self._full_levels)
        self._finish(codes, sizes, device)


class AnisotropicProjection(Projection):
    """Keep the words whose summed letter weights stay within ``weight_threshold``."""

    def __init__(self, weights: Union[Sequence[float], torch.Tensor], weight_threshold: float, depth: int,
                 path_dim: int, full_levels: Iterable[int] = (), *, device=None) -> None:
        self.path_dim = int(path_dim)
        self.depth = int(depth)
        self._full_levels = {int(n) for n in full_levels}
        _check_arguments(self.path_dim, self.depth, self._full_levels)

        self.weight_threshold = float(weight_threshold)
        if self.weight_threshold <= 0.0:
            raise ValueError("weight_threshold must be > 0.")
        if isinstance(weights, torch.Tensor):
            weights = weights.detach().cpu().flatten().tolist()
        self.weights = [float(w) for w in weights]
        if len(self.weights) != self.path_dim:
            raise ValueError(f"weights must have length == path_dim ({self.path_dim}), got {len(self.weights)}.")
        if any(w < 0.0 for w in self.weights):
            raise ValueError("weights must be non-negative.")

        d, thr = self.path_dim, self.weight_threshold
        per_level: List[List[int]] = [[] for _ in range(self.depth + 1)]
        # Grow admissible words one letter at a time; the running weight is accumulated in the
        # same left-to-right order as the word is read.
        frontier = [(a, self.weights[a]) for a in range(d) if self.weights[a] <= thr]
        if not frontier:
            raise ValueError("At least one weight must be <= weight_threshold.")
        per_level[1] = [c for c, _ in frontier]
        for n in range(2, self.depth + 1):
            grown = []
            for code, wt in frontier:
                for a in range(d):
                    total = wt + self.weights[a]
                    if total <= thr:
                        grown.append((code * d + a, total))
            frontier = grown
            per_level[n] = [c for c, _ in frontier]
            if not frontier:
                break
        codes, sizes = _strip_complete_levels(per_level, d, self._full_levels)
        self._finish(codes, sizes, device)


def lyndon_words(d: int, n: int) -> List[int]:
    """Codes of the Lyndon words of length exactly ``n`` over ``d`` letters, in lexicographic order.

    Duval's generation: repeat the current word periodically up to length n, strip trailing
    maximal letters, increment the last letter; a generated word is Lyndon exactly when its
    length before the periodic extension equals n.
    """
    out: List[int] = []
    w = [-1]
    while w:
        w[-1] += 1
        period = len(w)
        if period == n:
            code = 0
            for a in w:
                code = code * d + a
            out.append(code)
        while len(w) < n:
            w.append(w[len(w) - period])
        while w and w[-1] == d - 1:
            w.pop()
    return out


class LyndonProjection(Projection):
    """Word coordinates at the Lyndon words (degree 1 complete)."""

    def __init__(self, depth: int, path_dim: int, full_levels: Iterable[int] = (), *, device=None) -> None:
        self.depth = int(depth)
        self.path_dim = int(path_dim)
        self._full_levels = {int(n) for n in full_levels}
        _check_arguments(self.path_dim, self.depth, self._full_levels)

        d = self.path_dim
        sizes = [0] * (self.depth + 1)
        sizes[1] = d
        codes: List[int] = []
        for n in range(2, self.depth + 1):
            if n in self._full_levels:
                sizes[n] = d ** n
            else:
                level = lyndon_words(d, n)
                sizes[n] = len(level)
                codes.extend(level)
        self._finish(codes, sizes, device)


class projections:
    """Namespace of projection constructors (``pathsig.projections.words`` etc.)."""

    @staticmethod
    def words(words: Iterable[Iterable[int]], depth: int, path_dim: int,
              full_levels: Iterable[int] = (), *, device=None) -> WordsProjection:
        return WordsProjection(words, depth, path_dim, full_levels, device=device)

    @staticmethod
    def anisotropic(weights: Union[Sequence[float], torch.Tensor], weight_threshold: float, depth: int,
                    path_dim: int, full_levels: Iterable[int] = (), *, device=None) -> AnisotropicProjection:
        return AnisotropicProjection(weights, weight_threshold, depth, path_dim, full_levels, device=device)

    @staticmethod
    def lyndon(depth: int, path_dim: int, full_levels: Iterable[int] = (), *, device=None) -> LyndonProjection:
        return LyndonProjection(depth, path_dim, full_levels, device=device)
