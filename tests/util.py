"""Shared helpers of the test-suite: seeded inputs, the parity metric, reference loading."""
from __future__ import annotations

import math
import os
import random
from typing import List, Optional, Sequence

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libpathsig_ops.so")

# Parity tolerances: relative to the largest coefficient of the same degree (signatures) or of
# the whole tensor (gradients).
TOL = {torch.float32: 1e-5, torch.float64: 1e-11}


def brownian_path(B: int, L: int, d: int, seed: int = 0, dtype=torch.float64, device="cpu") -> torch.Tensor:
    """cumsum of i.i.d. N(0, 1/L) increments, generated on the CPU in float64, then cast."""
    g = torch.Generator().manual_seed(seed)
    x = torch.cumsum(torch.randn(B, L, d, generator=g, dtype=torch.float64) / math.sqrt(L), dim=1)
    return x.to(dtype).to(device)


def normal_like(shape, seed: int, dtype=torch.float64, device="cpu") -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(tuple(shape), generator=g, dtype=torch.float64).to(dtype).to(device)


def level_widths(d: int, depth: int, level_sizes: Optional[Sequence[int]] = None) -> List[int]:
    if level_sizes:
        return [int(s) for s in level_sizes[1: depth + 1]]
    return [d ** k for k in range(1, depth + 1)]


def level_rel_errors(got: torch.Tensor, want: torch.Tensor, widths: Sequence[int]) -> List[float]:
    """max|got-want| / max|want| per degree (last dimension split by `widths`)."""
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    out, off = [], 0
    for w in widths:
        if w == 0:
            continue
        a, b = got[..., off: off + w], want[..., off: off + w]
        denom = b.abs().max().item()
        out.append((a - b).abs().max().item() / (denom if denom > 0 else 1.0))
        off += w
    assert off == got.shape[-1]
    return out


def rel_error(got: torch.Tensor, want: torch.Tensor) -> float:
    got = got.detach().double().cpu()
    want = want.detach().double().cpu()
    denom = want.abs().max().item()
    return (got - want).abs().max().item() / (denom if denom > 0 else 1.0)


def random_words(n_words: int, d: int, min_len: int, max_len: int, seed: int) -> List[tuple]:
    """`n_words` distinct words, lengths uniform in [min_len, max_len], letters uniform, sorted by length."""
    rng = random.Random(seed)
    seen = set()
    while len(seen) < n_words:
        n = rng.randint(min_len, max_len)
        seen.add(tuple(rng.randrange(d) for _ in range(n)))
    return sorted(seen, key=lambda w: (len(w), w))


def sliding_windows(L: int, length: int, stride: int, device="cpu") -> torch.Tensor:
    starts = range(0, L - length + 1, stride)
    return torch.tensor([[s, s + length] for s in starts], dtype=torch.int32, device=device)


_ref_ops = None


def reference_ops():
    """``torch.ops.pathsig`` of the reference's own CUDA build, or None when it was not built."""
    global _ref_ops
    if _ref_ops is None and os.path.isfile(REF_LIB):
        torch.ops.load_library(REF_LIB)
        _ref_ops = torch.ops.pathsig
    return _ref_ops
