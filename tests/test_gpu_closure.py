"""The prefix-closure kernels (generated per word set) against the CPU oracle.

These kernels are picked automatically only for large projected workloads; here they are forced
(``set_algorithm("closure")``) on small seeded cases: explicit words, Lyndon words, the hybrid layout the
log-signature asks for, anisotropic projections, dense rows, ragged and overlapping windows, batches
that do not fill a warp of units, both dtypes.  The float64 cases pin the generated arithmetic to 1e-11.
"""
from __future__ import annotations

import pytest
import torch

from . import util
from .test_gpu_parity import _oracle_logsig, _run_sig

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.float64]


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", ["lyndon", "words", "words_full1", "anisotropic", "lyndon_full", "many_words"])
def test_projected_rows(ps, oracle, dtype, kind):
    P = ps.projections
    B, L = 37, 25
    if kind == "lyndon":
        proj, d = P.lyndon(5, 3), 3
    elif kind == "lyndon_full":
        proj, d = P.lyndon(4, 3, full_levels=(2,)), 3
    elif kind == "words":
        proj, d = P.words(util.random_words(40, 4, 1, 5, seed=3), 5, 4), 4
    elif kind == "words_full1":
        proj, d = P.words(util.random_words(60, 8, 2, 6, seed=4), 6, 8, full_levels=(1,)), 8
    elif kind == "many_words":   # several bins per block row and several block rows
        proj, d, B, L = P.words(util.random_words(300, 6, 2, 6, seed=6), 6, 6, full_levels=(1,)), 6, 70, 40
    else:
        proj, d = P.anisotropic([1.0, 2.0, 1.5, 3.0], 5.0, 5, 4), 4
    x = util.brownian_path(B, L, d, seed=13, dtype=dtype)
    _run_sig(ps, oracle, x, proj.depth, proj=proj, algo="closure")
    _run_sig(ps, oracle, x[:5], proj.depth, proj=proj, windows=util.sliding_windows(L, 10, 5), algo="closure")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,depth", [(2, 5), (3, 4), (4, 3), (8, 2), (5, 1)])
def test_dense_rows(ps, oracle, dtype, d, depth):
    x = util.brownian_path(33, 21, d, seed=d * depth, dtype=dtype)
    _run_sig(ps, oracle, x, depth, algo="closure")


@pytest.mark.parametrize("dtype", DTYPES)
def test_ragged_and_overlapping_windows(ps, oracle, dtype):
    x = util.brownian_path(3, 40, 3, seed=8, dtype=dtype)
    win = torch.tensor([[0, 40], [5, 7], [10, 30], [3, 3], [12, 13], [20, 40], [0, 21], [-4, 9], [30, 55]],
                       dtype=torch.int32)
    x_ref = x.clone()
    ps.ops.set_algorithm("closure")
    try:
        xg = x.to(DEV).requires_grad_(True)
        out = ps.Signature(depth=3, windows=win.to(DEV))(xg)
        g = util.normal_like(out.shape, 2, dtype)
        (out * g.to(DEV)).sum().backward()
    finally:
        ps.ops.set_algorithm("auto")
    # windows reaching outside the path are clamped to it
    clamped = win.clamp(min=0, max=40)
    want = oracle.sig_forward(x_ref.double(), 3, windows=clamped)
    want_grad = oracle.sig_backward(x_ref.double(), want, g.double(), 3, windows=clamped)
    assert max(util.level_rel_errors(out, want, util.level_widths(3, 3))) < util.TOL[dtype]
    assert util.rel_error(xg.grad, want_grad) < util.TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_log_signature_over_closure_kernels(ps, oracle, dtype):
    """The hybrid layout of LogSignature (dense below a listed top degree) served by the closure kernels."""
    d, depth = 3, 5
    x = util.brownian_path(34, 30, d, seed=21, dtype=dtype)
    mod = ps.LogSignature(depth=depth, projection=ps.projections.lyndon(depth, d, device=DEV))
    ps.ops.set_algorithm("closure")
    try:
        xg = x.to(DEV).requires_grad_(True)
        out = mod(xg)
        g = util.normal_like(out.shape, 4, dtype)
        (out * g.to(DEV)).sum().backward()
    finally:
        ps.ops.set_algorithm("auto")
    want, want_grad = _oracle_logsig(oracle, mod, x.double(), g.double(), None)
    tol = util.TOL[dtype] if dtype == torch.float64 else 5e-5
    assert util.rel_error(out, want) < tol
    assert util.rel_error(xg.grad, want_grad) < tol


def test_closure_and_lane_kernels_agree_on_a_large_projection(ps):
    """Automatic selection: a projected workload with enough work runs on the closure kernels; the result
    matches the generic kernels on the same tensors."""
    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    words = util.random_words(120, 8, 2, 6, seed=9)
    proj = ps.projections.words(words, 6, 8, full_levels=(1,), device=DEV)
    x = util.brownian_path(512, 400, 8, seed=3, dtype=torch.float32).to(DEV)
    mod = ps.Signature(depth=6, projection=proj)

    def run(algo):
        ps.ops.set_algorithm(algo)
        try:
            xa = x.clone().requires_grad_(True)
            out = mod(xa)
            out.backward(torch.ones_like(out))
            return out.detach(), xa.grad
        finally:
            ps.ops.set_algorithm("auto")

    out_c, grad_c = run("closure")
    out_g, grad_g = run("generic")
    out_a, grad_a = run("auto")
    widths = util.level_widths(8, 6, proj.level_sizes)
    assert max(util.level_rel_errors(out_c, out_g, widths)) < 1e-5
    assert util.rel_error(grad_c, grad_g) < 1e-5
    # "auto" took the closure kernels: forward results are bitwise those of the forced run
    assert torch.equal(out_a, out_c)
    assert lib.psig_kernel_launches() > 0


def test_repeated_word_falls_back(ps, oracle):
    """A word listed twice has no unique column; the closure plan is refused and "auto" still serves it."""
    proj = ps.projections.words([(0, 1), (0, 1), (1, 0, 1)], 3, 2, full_levels=(1,), device=DEV)
    x = util.brownian_path(40, 12, 2, seed=1, dtype=torch.float64)
    _run_sig(ps, oracle, x, 3, proj=proj, algo="auto")
    ps.ops.set_algorithm("closure")
    try:
        with pytest.raises(RuntimeError, match="no kernel"):
            ps.Signature(depth=3, projection=proj)(x.to(DEV))
    finally:
        ps.ops.set_algorithm("auto")


@pytest.mark.parametrize("d,depth", [(3, 4), (40, 2)])
def test_dense_shape_without_a_tiled_instance_takes_the_closure_kernels(ps, d, depth):
    """Dense rows of a shape the register-tiled table does not hold, with enough work: the automatic
    selection specialises closure kernels for the shape; the result matches the generic kernels."""
    x = util.brownian_path(2048, 128, d, seed=11, dtype=torch.float32).to(DEV)
    mod = ps.Signature(depth=depth)

    def run(algo):
        ps.ops.set_algorithm(algo)
        try:
            xa = x.clone().requires_grad_(True)
            out = mod(xa)
            out.backward(torch.ones_like(out))
            return out.detach(), xa.grad
        finally:
            ps.ops.set_algorithm("auto")

    out_a, grad_a = run("auto")
    out_c, grad_c = run("closure")
    out_g, grad_g = run("generic")
    assert torch.equal(out_a, out_c)
    assert max(util.level_rel_errors(out_c, out_g, util.level_widths(d, depth))) < 1e-5
    assert util.rel_error(grad_c, grad_g) < 1e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("windowed", [False, True])
def test_module_evaluates_large_projections_on_the_closed_word_set(ps, oracle, dtype, windowed):
    """``Signature`` with a projection whose words have prefixes that are not requested: a problem large
    enough for the generated kernels runs on the prefix closure of the word set (so that the backward
    pass finds every prefix in the saved signature) and selects the requested columns; values and
    input gradient match the oracle on the requested layout, and the plain operator call."""
    words = util.random_words(90, 5, 2, 5, seed=21)
    proj = ps.projections.words(words, 5, 5, full_levels=(1,), device=DEV)
    B, L = (128, 200) if windowed else (512, 300)
    win = util.sliding_windows(L, 60, 10, device=DEV) if windowed else None
    x = util.brownian_path(B, L, 5, seed=2, dtype=dtype).to(DEV)
    mod = ps.Signature(depth=5, projection=proj, windows=win)
    assert mod._closure_sizes is not None and sum(mod._closure_sizes) > sum(proj.level_sizes[1:])
    assert mod._closure_pays(x) and not mod._closure_pays(x[:4])
    xa = x.clone().requires_grad_(True)
    out = mod(xa)
    g = util.normal_like(out.shape, 4, dtype).to(DEV)
    out.backward(g)
    # the operator on the requested word set itself
    xb = x.clone().requires_grad_(True)
    plain = ps.ops.compute_signature(xb, 5, True, mod._encoded_words, mod._level_sizes, mod.use_windows, mod._windows)
    plain.backward(g)
    tol = util.TOL[dtype]
    assert out.shape == plain.shape
    assert util.rel_error(out, plain) < tol and util.rel_error(xa.grad, xb.grad) < tol
    rows = slice(0, 6)
    xs = x[rows].double().cpu()
    win_cpu = None if win is None else win.cpu()
    want = oracle.sig_forward(xs, 5, proj.encoded_words.cpu(), list(proj.level_sizes), win_cpu)
    assert util.rel_error(out[rows], want) < tol
    want_grad = oracle.sig_backward(xs, want, g[rows].double().cpu(), 5, proj.encoded_words.cpu(),
                                    list(proj.level_sizes), win_cpu)
    assert util.rel_error(xa.grad[rows], want_grad) < tol
    # a small problem takes the requested word set as it is
    small = mod(x[:4])
    assert util.rel_error(small, out[:4]) < tol
    # the closed set is re-derived from the codes a state_dict brings: a module built for another word set
    # with the same level sizes (one word replaced by an unused word of its length) takes over this one's
    longest = max(words, key=len)
    swapped = next(w for w in (longest[:-1] + (a,) for a in range(5)) if w not in set(words))
    other_proj = ps.projections.words([swapped if w == longest else w for w in words], 5, 5, full_levels=(1,), device=DEV)
    assert list(other_proj.level_sizes) == list(proj.level_sizes)
    other = ps.Signature(depth=5, projection=other_proj, windows=win)
    assert not torch.equal(other._encoded_words, mod._encoded_words)
    other.load_state_dict(mod.state_dict())
    assert torch.equal(other._closure_words, mod._closure_words) and torch.equal(other._closure_columns, mod._closure_columns)
    assert util.rel_error(other(x), out) < tol


def test_closed_word_set_path_traces_under_torch_compile(ps):
    """The module's choice between the requested and the closed word set is shape arithmetic in Python and
    its column selection a custom autograd function: both trace without graph breaks, and the compiled
    function gives the eager values and gradient."""
    proj = ps.projections.words(util.random_words(90, 5, 2, 5, seed=21), 5, 5, full_levels=(1,), device=DEV)
    mod = ps.Signature(depth=5, projection=proj)
    x1 = util.brownian_path(512, 300, 5, seed=2, dtype=torch.float32).to(DEV).requires_grad_(True)
    x2 = x1.detach().clone().requires_grad_(True)
    assert mod._closure_pays(x1)

    def fn(x):
        return mod(x).square().sum()

    compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
    y1, y2 = fn(x1), compiled(x2)
    y1.backward()
    y2.backward()
    assert torch.allclose(y1, y2, rtol=1e-5)
    assert util.rel_error(x2.grad, x1.grad) < util.TOL[torch.float32]
