"""Logarithm + column selection as one kernel (``ops.logsig_projected``) against the two-stage composition
the reference uses (``sig_to_logsig`` followed by ``index_select``, src/pathsig/modules.py:112-135 of the
reference), and against the CPU oracle: values and input gradients, both dtypes, with windows, for Lyndon,
explicit-word and anisotropic projections, and for a column list with a repeated word."""
from __future__ import annotations

import pytest
import torch

from . import util
from .test_gpu_parity import _oracle_logsig

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _two_stage(ps, mod, x):
    """The same module evaluated the reference's way: signature, logarithm, stock gather."""
    d, ls = mod._path_dim, mod._ext_level_sizes
    sig = ps.ops.compute_signature(x, mod.depth, True, mod._top_words, ls, mod.use_windows, mod._windows)
    logsig, _ = ps.ops.sig_to_logsig(sig, mod.depth, d, True, mod._top_words, ls)
    return logsig.index_select(-1, mod._indices_from_sig)


def _projection(ps, kind):
    P = ps.projections
    if kind == "lyndon":
        return P.lyndon(5, 3, device=DEV)
    if kind == "lyndon46":
        return P.lyndon(6, 4, device=DEV)
    if kind == "words":
        return P.words(util.random_words(30, 4, 1, 4, seed=3), 4, 4, device=DEV)
    if kind == "top_full":
        return P.lyndon(3, 3, full_levels=(3,), device=DEV)   # dense top degree, listed lower degree
    return P.anisotropic([1.0, 2.0, 1.5, 3.0], 5.0, 5, 4, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("kind", ["lyndon", "lyndon46", "words", "anisotropic", "top_full"])
@pytest.mark.parametrize("windowed", [False, True])
def test_fused_selection_matches_two_stage_and_oracle(ps, oracle, dtype, kind, windowed):
    proj = _projection(ps, kind)
    x = util.brownian_path(5, 24, proj.path_dim, seed=17, dtype=dtype).to(DEV)
    win = util.sliding_windows(24, 10, 7, device=DEV) if windowed else None
    mod = ps.LogSignature(depth=proj.depth, projection=proj, windows=win)
    assert mod._fusable and ps.ops.logsig_projected_supported(dtype, proj.depth, proj.path_dim, mod._ext_level_sizes)
    xa = x.clone().requires_grad_(True)
    out = mod(xa)
    g = util.normal_like(out.shape, 9, dtype).to(DEV)
    (out * g).sum().backward()
    xb = x.clone().requires_grad_(True)
    ref = _two_stage(ps, mod, xb)
    (ref * g).sum().backward()
    assert out.shape == ref.shape
    tol = 1e-12 if dtype == torch.float64 else 2e-6
    assert util.rel_error(out, ref) < tol
    assert util.rel_error(xa.grad, xb.grad) < (1e-11 if dtype == torch.float64 else 2e-5)
    want, want_grad = _oracle_logsig(oracle, mod, x.double().cpu(), g.double().cpu(), None if win is None else win.cpu())
    assert util.rel_error(out, want) < (1e-11 if dtype == torch.float64 else 5e-5)
    assert util.rel_error(xa.grad, want_grad) < (1e-11 if dtype == torch.float64 else 5e-5)


def test_repeated_lower_column_adds_its_gradients(ps):
    """A column list that asks for a word below the top degree twice: both gradients reach the word."""
    proj = ps.projections.lyndon(4, 3, device=DEV)
    mod = ps.LogSignature(depth=4, projection=proj)
    x = util.brownian_path(3, 15, 3, seed=5, dtype=torch.float64).to(DEV)
    ls, tw = mod._ext_level_sizes, mod._top_words
    sig = ps.ops.compute_signature(x, 4, True, tw, ls, False, mod._windows).requires_grad_(True)
    cols = torch.tensor([0, 2, 2, 7, 20, 7], dtype=torch.int64, device=DEV)
    out = ps.ops.logsig_projected(sig, 4, 3, tw, ls, cols)
    g = torch.randn_like(out)
    (out * g).sum().backward()
    sig2 = sig.detach().clone().requires_grad_(True)
    full, _ = ps.ops.sig_to_logsig(sig2, 4, 3, True, tw, ls)
    lower = sum(ls[:4])
    index = torch.cat([cols, torch.arange(lower, lower + ls[4], device=DEV)])
    (full.index_select(-1, index) * g).sum().backward()
    torch.testing.assert_close(out, full.index_select(-1, index), atol=1e-13, rtol=1e-12)
    torch.testing.assert_close(sig.grad, sig2.grad, atol=1e-13, rtol=1e-12)


def test_projected_operator_registration_checks(ps):
    proj = ps.projections.lyndon(3, 3, device=DEV)
    mod = ps.LogSignature(depth=3, projection=proj)
    x = util.brownian_path(2, 9, 3, seed=2, dtype=torch.float64).to(DEV)
    sig = ps.ops.compute_signature(x, 3, True, mod._top_words, mod._ext_level_sizes, False, mod._windows)
    args = (sig.requires_grad_(True), 3, 3, mod._top_words, mod._ext_level_sizes, mod._lower_columns)
    torch.library.opcheck(torch.ops.pathsig_b200.logsig_projected.default, args)
    assert torch.autograd.gradcheck(lambda s: ps.ops.logsig_projected(s, *args[1:]), (sig,), atol=1e-8, rtol=1e-6)


def test_replaced_column_index_falls_back_to_the_gather(ps):
    """An index loaded through a state_dict that is not "lower words, then the whole top degree" cannot
    use the fused kernel; the module then evaluates the two-stage form."""
    proj = ps.projections.lyndon(3, 3, device=DEV)
    mod = ps.LogSignature(depth=3, projection=proj)
    state = {k: v.clone() for k, v in mod.state_dict().items()}
    state["_indices_from_sig"] = state["_indices_from_sig"].flip(0)
    mod.load_state_dict(state)
    assert mod._fusable is False
    x = util.brownian_path(2, 9, 3, seed=2, dtype=torch.float64).to(DEV)
    torch.testing.assert_close(mod(x), _two_stage(ps, mod, x))
