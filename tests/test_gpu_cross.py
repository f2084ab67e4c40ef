"""Randomised cross-checks on the GPU between kernel families that compute the same thing by different
routes: register-tiled against generic signature kernels (every tiled shape, both dtypes, ragged windows,
lengths on both sides of the staging chunk), and the row-in-shared-memory against the streamed form of the
log-signature kernels.  The oracle pins each family separately on a few shapes; this file widens the
net cheaply, with seeded draws."""
from __future__ import annotations

import random

import pytest
import torch

from . import util
from .test_gpu_parity import TILED, TILED_PROJECTED_TOP

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _both(ps, fn):
    out = {}
    for algo in ("tiled", "generic"):
        ps.ops.set_algorithm(algo)
        try:
            out[algo] = fn()
        finally:
            ps.ops.set_algorithm("auto")
    return out["tiled"], out["generic"]


def _windows(rng, L, W):
    rows = []
    for _ in range(W):
        a = rng.randrange(0, L)
        b = rng.randrange(a, L + 1)
        rows.append([a, b])  # includes empty and one-point windows
    return torch.tensor(rows, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("seed", range(140))
def test_tiled_agrees_with_generic(ps, seed):
    rng = random.Random(1000 + seed)
    d, depth = TILED[seed % len(TILED)]
    dtype = torch.float64 if rng.random() < 0.5 else torch.float32
    width = sum(d ** k for k in range(1, depth + 1))
    B = rng.choice([1, 2, 5]) if width > 20000 else rng.choice([1, 3, 8, 33])
    L = rng.choice([2, 5, 63, 64, 65, 66, 130, 200]) if width <= 20000 else rng.choice([2, 9, 65, 70])
    use_windows = rng.random() < 0.4
    win = _windows(rng, L, rng.choice([1, 4, 9])) if use_windows else None
    x = util.brownian_path(B, L, d, seed=seed, dtype=dtype).to(DEV)
    mod = ps.Signature(depth=depth, windows=win)
    g = None

    def run():
        nonlocal g
        xg = x.clone().requires_grad_(True)
        out = mod(xg)
        if g is None:
            g = util.normal_like(out.shape, seed + 7, dtype).to(DEV)
        (out * g).sum().backward()
        return out.detach(), xg.grad

    (sig_t, grad_t), (sig_g, grad_g) = _both(ps, run)
    tol = 2e-5 if dtype == torch.float32 else 1e-11
    widths = util.level_widths(d, depth)
    assert max(util.level_rel_errors(sig_t, sig_g, widths)) < tol
    assert util.rel_error(grad_t, grad_g) < tol


@pytest.mark.parametrize("seed", range(52))
def test_tiled_projected_top_agrees_with_generic(ps, seed):
    rng = random.Random(2000 + seed)
    d, depth = TILED_PROJECTED_TOP[seed % len(TILED_PROJECTED_TOP)]
    dtype = torch.float64 if seed % 2 else torch.float32
    n_top = rng.randrange(1, min(d ** depth, 300))
    top = util.random_words(n_top, d, depth, depth, seed=seed)
    proj = ps.projections.words(top, depth, d, full_levels=tuple(range(1, depth)))
    L = rng.choice([3, 40, 90])
    x = util.brownian_path(rng.choice([1, 4]), L, d, seed=seed, dtype=dtype).to(DEV)
    win = _windows(rng, L, 3) if rng.random() < 0.5 else None
    mod = ps.Signature(depth=depth, projection=proj, windows=win)

    def run():
        xg = x.clone().requires_grad_(True)
        out = mod(xg)
        out.square().sum().backward()
        return out.detach(), xg.grad

    (sig_t, grad_t), (sig_g, grad_g) = _both(ps, run)
    tol = 2e-5 if dtype == torch.float32 else 1e-11
    assert util.rel_error(sig_t, sig_g) < tol
    assert util.rel_error(grad_t, grad_g) < tol


@pytest.mark.parametrize("seed", range(60))
def test_log_kernel_families_agree(ps, seed):
    rng = random.Random(3000 + seed)
    d = rng.choice([1, 2, 3, 4, 5, 7, 8])
    depth = rng.randrange(1, {1: 9, 2: 9, 3: 7, 4: 6, 5: 5, 7: 4, 8: 4}[d] + 1)
    dtype = torch.float64 if rng.random() < 0.5 else torch.float32
    lower = sum(d ** k for k in range(1, depth))
    dense_top = d ** depth
    projected = rng.random() < 0.5 and dense_top > 1
    empty_w = torch.empty(0, dtype=torch.int64, device=DEV)
    if projected:
        n_top = rng.randrange(1, min(dense_top, 200) + 1)
        codes = [rng.randrange(dense_top) for _ in range(n_top)]  # duplicates allowed
        words = torch.tensor(codes, dtype=torch.int64, device=DEV)
        ls = [0] + [d ** k for k in range(1, depth)] + [n_top]
        top = n_top
    else:
        words, ls, top = empty_w, [0] + [d ** k for k in range(1, depth + 1)], dense_top
    rows = rng.choice([1, 3, 17])
    sig = (util.normal_like((rows, lower + top), seed, dtype) * 0.3).to(DEV)
    g = util.normal_like((rows, lower + top), seed + 1, dtype).to(DEV)
    res = {}
    for algo in ("auto", "generic"):
        ps.ops.set_algorithm(algo)
        try:
            logsig, cache = ps.ops.sig_to_logsig(sig, depth, d, projected, words, ls)
            res[algo] = (logsig, ps.ops.logsig_backward(sig, cache, g, depth, projected, words, ls), cache.shape[-1])
        finally:
            ps.ops.set_algorithm("auto")
    assert res["auto"][2] == 0 and res["generic"][2] == (lower + top) * depth
    tol = 3e-5 if dtype == torch.float32 else 1e-11
    assert util.rel_error(res["auto"][0], res["generic"][0]) < tol
    assert util.rel_error(res["auto"][1], res["generic"][1]) < tol
