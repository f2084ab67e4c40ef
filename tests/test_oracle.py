"""Pins the CPU oracle (oracle/) against the mathematical definition and closed forms.

The oracle restates the reference's per-word recursions; these tests compare it with an
independent dense tensor-algebra evaluation (tests/tensor_algebra.py), with closed-form
identities and with finite differences.  No GPU needed.
"""
from __future__ import annotations

import itertools
import math

import numpy as np
import pytest
import torch

from pathsig_b200.projections import projections

from . import tensor_algebra as ta
from . import util


def _path(B, L, d, seed=0, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    return torch.cumsum(torch.randn(B, L, d, generator=g, dtype=torch.float64) / math.sqrt(L), dim=1).to(dtype)


@pytest.mark.parametrize("d,depth", [(2, 1), (2, 5), (3, 4), (5, 3), (8, 2)])
def test_forward_matches_definition(oracle, d, depth):
    x = _path(3, 9, d, seed=d * 10 + depth)
    got = oracle.sig_forward(x, depth)
    for b in range(x.shape[0]):
        want = ta.signature(x[b].numpy(), depth)
        np.testing.assert_allclose(got[b].numpy(), want, rtol=0, atol=1e-13 * max(1.0, np.abs(want).max()))


def test_straight_line_closed_form(oracle):
    # One increment v: S(w) = prod_i v[w_i] / |w|!
    d, depth = 3, 5
    v = torch.tensor([0.7, -1.3, 0.4], dtype=torch.float64)
    x = torch.stack([torch.zeros(d, dtype=torch.float64), v])[None]
    got = oracle.sig_forward(x, depth)[0].numpy()
    want = []
    for n in range(1, depth + 1):
        for w in itertools.product(range(d), repeat=n):
            want.append(np.prod([v[a].item() for a in w]) / math.factorial(n))
    np.testing.assert_allclose(got, np.array(want), rtol=1e-14, atol=1e-15)


def test_time_reparametrisation_invariance(oracle):
    # Inserting a point on a segment does not change the signature.
    d, depth = 3, 4
    x = _path(1, 6, d, seed=3)
    mid = 0.3 * x[:, 2] + 0.7 * x[:, 3]
    x2 = torch.cat([x[:, :3], mid[:, None], x[:, 3:]], dim=1)
    np.testing.assert_allclose(oracle.sig_forward(x, depth).numpy(), oracle.sig_forward(x2, depth).numpy(), atol=1e-14)


def test_float32_close_to_float64(oracle):
    x = _path(4, 200, 4, seed=7)
    s64 = oracle.sig_forward(x, 4)
    s32 = oracle.sig_forward(x.float(), 4)
    assert (s32.double() - s64).abs().max() / s64.abs().max() < 2e-6


@pytest.mark.parametrize("windows", [[[0, 7]], [[0, 4], [2, 9], [8, 10], [3, 3], [5, 6]]])
def test_windows_equal_slices(oracle, windows):
    d, depth = 3, 3
    x = _path(2, 10, d, seed=11)
    win = torch.tensor(windows, dtype=torch.int32)
    got = oracle.sig_forward(x, depth, windows=win)
    assert got.shape == (2, len(windows), 39)
    for i, (s, e) in enumerate(windows):
        if e - s < 2:
            assert torch.all(got[:, i] == 0)
        else:
            np.testing.assert_allclose(got[:, i].numpy(), oracle.sig_forward(x[:, s:e], depth).numpy(), atol=1e-15)


def _full_columns(proj):
    """Columns of the dense signature picked by a projection (same rule as the reference's
    tests/test_projections.py:13-37)."""
    d, cols, off, used = proj.path_dim, [], 0, 0
    codes = proj.encoded_words.tolist()
    for n in range(1, proj.depth + 1):
        size = proj.level_sizes[n]
        if size == d ** n:
            cols.extend(range(off, off + d ** n))
        elif size > 0:
            cols.extend(off + c for c in codes[used: used + size])
            used += size
        off += d ** n
    return torch.tensor(cols, dtype=torch.int64)


@pytest.mark.parametrize("make", [
    lambda: projections.lyndon(4, 3, device="cpu"),
    lambda: projections.words([(0,), (2,), (0, 1), (2, 2), (1, 0, 2), (2, 2, 2, 1)], 4, 3, device="cpu"),
    lambda: projections.words([(1, 0), (0, 1, 1)], 3, 2, full_levels=(1,), device="cpu"),
    lambda: projections.anisotropic([1.0, 2.0, 1.5], 4.0, 4, 3, device="cpu"),
])
def test_projected_forward_and_backward(oracle, make):
    proj = make()
    x = _path(2, 8, proj.path_dim, seed=5)
    cols = _full_columns(proj)
    full = oracle.sig_forward(x, proj.depth)
    got = oracle.sig_forward(x, proj.depth, proj.encoded_words, proj.level_sizes)
    assert got.shape[-1] == proj.sig_size
    np.testing.assert_allclose(got.numpy(), full[:, cols].numpy(), atol=1e-14)

    g = torch.randn(got.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    gfull = torch.zeros_like(full)
    gfull.index_add_(1, cols, g)
    want = oracle.sig_backward(x, full, gfull, proj.depth)
    have = oracle.sig_backward(x, got, g, proj.depth, proj.encoded_words, proj.level_sizes)
    np.testing.assert_allclose(have.numpy(), want.numpy(), atol=1e-12)


def _finite_difference(f, x, g, eps=1e-6):
    out = torch.zeros_like(x)
    flat = x.reshape(-1)
    for i in range(flat.numel()):
        xp, xm = flat.clone(), flat.clone()
        xp[i] += eps
        xm[i] -= eps
        out.reshape(-1)[i] = ((f(xp.reshape(x.shape)) - f(xm.reshape(x.shape))) * g).sum() / (2 * eps)
    return out


@pytest.mark.parametrize("d,depth", [(2, 4), (3, 3)])
def test_backward_matches_finite_differences(oracle, d, depth):
    x = _path(1, 5, d, seed=2)
    sig = oracle.sig_forward(x, depth)
    g = torch.randn(sig.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    got = oracle.sig_backward(x, sig, g, depth)
    want = _finite_difference(lambda p: oracle.sig_forward(p, depth), x, g)
    np.testing.assert_allclose(got.numpy(), want.numpy(), atol=2e-8)


def test_backward_sums_overlapping_windows(oracle):
    d, depth = 2, 3
    x = _path(2, 9, d, seed=4)
    win = torch.tensor([[0, 5], [2, 9], [4, 6]], dtype=torch.int32)
    sig = oracle.sig_forward(x, depth, windows=win)
    g = torch.randn(sig.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(6))
    got = oracle.sig_backward(x, sig, g, depth, windows=win)
    want = torch.zeros_like(x)
    for i, (s, e) in enumerate(win.tolist()):
        want[:, s:e] += oracle.sig_backward(x[:, s:e], sig[:, i], g[:, i], depth)
    np.testing.assert_allclose(got.numpy(), want.numpy(), atol=1e-13)


@pytest.mark.parametrize("d,depth", [(2, 5), (3, 4), (4, 3)])
def test_logsig_matches_definition(oracle, d, depth):
    x = _path(2, 7, d, seed=9)
    got = oracle.logsignature(x, depth)
    for b in range(2):
        want = ta.logsignature(x[b].numpy(), depth)
        np.testing.assert_allclose(got[b].numpy(), want, atol=1e-13)


def test_logsig_of_straight_line_is_the_increment(oracle):
    d, depth = 3, 4
    x = torch.tensor([[[0.0, 0.0, 0.0], [0.5, -0.2, 1.1]]], dtype=torch.float64)
    got = oracle.logsignature(x, depth)[0]
    np.testing.assert_allclose(got[:d].numpy(), x[0, 1].numpy(), atol=1e-15)
    assert got[d:].abs().max() < 1e-15


def test_lyndon_logsig_and_gradient(oracle):
    d, depth = 3, 4
    proj = projections.lyndon(depth, d, device="cpu")
    x = _path(1, 5, d, seed=12)
    explicit_below_top = sum(proj.level_sizes[k] for k in range(1, depth) if proj.level_sizes[k] != d ** k)
    top = proj.encoded_words[explicit_below_top:]
    ext = [0] + [d ** k for k in range(1, depth)] + [proj.level_sizes[depth]]
    idx = proj.logsig_indices()
    got = oracle.logsignature(x, depth, top_words=top, ext_level_sizes=ext, indices=idx)
    assert got.shape == (1, proj.sig_size)
    full = oracle.logsignature(x, depth)
    np.testing.assert_allclose(got.numpy(), full[:, _full_columns(proj)].numpy(), atol=1e-14)

    g = torch.randn(got.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(8))
    _, grad = oracle.logsignature(x, depth, top_words=top, ext_level_sizes=ext, indices=idx, grad_out=g)
    want = _finite_difference(
        lambda p: oracle.logsignature(p, depth, top_words=top, ext_level_sizes=ext, indices=idx), x, g)
    np.testing.assert_allclose(grad.numpy(), want.numpy(), atol=2e-8)


def test_shuffle_identity(oracle):
    # S(i) S(j) = S(ij) + S(ji)
    d = 3
    x = _path(1, 12, d, seed=21)
    s = oracle.sig_forward(x, 2)[0]
    for i in range(d):
        for j in range(d):
            assert abs(s[i] * s[j] - s[d + i * d + j] - s[d + j * d + i]) < 1e-14


@pytest.mark.parametrize("d,depth", [(2, 5), (3, 4), (5, 3)])
def test_chen_product_glues_signatures(oracle, d, depth):
    """S(x[:m+1]) (x) S(x[m:]) = S(x), and the gradient through the glued pieces equals the gradient
    through the whole path (both sides computed by the oracle)."""
    x = util.brownian_path(2, 14, d, seed=d + depth)
    m = 6
    whole = oracle.sig_forward(x, depth)
    sa, sb = oracle.sig_forward(x[:, : m + 1].contiguous(), depth), oracle.sig_forward(x[:, m:].contiguous(), depth)
    glued, grad_fn = oracle.chen_product(sa, sb, d, depth)
    assert util.rel_error(glued, whole) < 1e-13
    g = util.normal_like(whole.shape, 3)
    ga, gb = grad_fn(g)
    want = oracle.sig_backward(x, whole, g, depth)
    got = torch.zeros_like(x)
    got[:, : m + 1] += oracle.sig_backward(x[:, : m + 1].contiguous(), sa, ga, depth)
    got[:, m:] += oracle.sig_backward(x[:, m:].contiguous(), sb, gb, depth)
    assert util.rel_error(got, want) < 1e-12
