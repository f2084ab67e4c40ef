"""GPU parity: the CUDA library (through the operator layer / C ABI) against the CPU oracle.

Every case runs the same seeded inputs through ``pathsig_b200`` on the GPU and through
``oracle/`` on the CPU.  Tolerances (tests/util.py): 1e-5 (float32) and 1e-11 (float64) of
the largest coefficient of the same degree, and of the largest entry for input gradients.
"""
from __future__ import annotations

import pytest
import torch

from . import util

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _check_levels(got, want, widths, dtype, what=""):
    errs = util.level_rel_errors(got, want, widths)
    assert max(errs) < util.TOL[dtype], f"{what}: per-degree relative errors {errs}"


def _run_sig(ps, oracle, x, depth, proj=None, windows=None, seed=1, algo="auto"):
    """Forward + backward on GPU and oracle; returns nothing, asserts parity."""
    dtype = x.dtype
    ps.ops.set_algorithm(algo)
    try:
        xg = x.to(DEV).requires_grad_(True)
        mod = ps.Signature(depth=depth, projection=proj, windows=None if windows is None else windows.to(DEV))
        out = mod(xg)
        g = util.normal_like(out.shape, seed, dtype)
        (out * g.to(DEV)).sum().backward()
    finally:
        ps.ops.set_algorithm("auto")
    ew = None if proj is None else proj.encoded_words.cpu()
    ls = None if proj is None else proj.level_sizes
    x64 = x.double()
    want = oracle.sig_forward(x64, depth, ew, ls, windows)
    want_grad = oracle.sig_backward(x64, want, g.double(), depth, ew, ls, windows)
    widths = util.level_widths(x.shape[-1], depth, ls)
    assert out.shape == want.shape
    _check_levels(out, want, widths, dtype, "signature")
    err = util.rel_error(xg.grad, want_grad)
    assert err < util.TOL[dtype], f"path gradient relative error {err}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth", [(2, 1), (2, 6), (3, 4), (4, 5), (5, 3), (8, 4), (16, 3), (40, 2), (3, 9)])
def test_dense_signature(ps, oracle, dtype, d, depth):
    x = util.brownian_path(3, 33, d, seed=d + depth, dtype=dtype)
    _run_sig(ps, oracle, x, depth, algo="generic")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_depth_twelve(ps, oracle, dtype):
    x = util.brownian_path(2, 12, 2, seed=5, dtype=dtype)
    _run_sig(ps, oracle, x, 12, algo="generic")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("L", [2, 3, 65, 200])
def test_path_lengths(ps, oracle, dtype, L):
    x = util.brownian_path(5, L, 3, seed=L, dtype=dtype)
    _run_sig(ps, oracle, x, 4, algo="generic")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_windows_ragged(ps, oracle, dtype):
    x = util.brownian_path(3, 40, 3, seed=8, dtype=dtype)
    win = torch.tensor([[0, 40], [5, 7], [10, 30], [3, 3], [12, 13], [20, 40], [0, 21]], dtype=torch.int32)
    _run_sig(ps, oracle, x, 3, windows=win, algo="generic")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_windows_sliding(ps, oracle, dtype):
    x = util.brownian_path(4, 96, 4, seed=9, dtype=dtype)
    _run_sig(ps, oracle, x, 3, windows=util.sliding_windows(96, 32, 8), algo="generic")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("kind", ["lyndon", "words", "words_full1", "anisotropic", "lyndon_full"])
def test_projections(ps, oracle, dtype, kind):
    P = ps.projections
    if kind == "lyndon":
        proj, d = P.lyndon(5, 3), 3
    elif kind == "lyndon_full":
        proj, d = P.lyndon(4, 3, full_levels=(2,)), 3
    elif kind == "words":
        proj, d = P.words(util.random_words(40, 4, 1, 5, seed=3), 5, 4), 4
    elif kind == "words_full1":
        proj, d = P.words(util.random_words(60, 8, 2, 6, seed=4), 6, 8, full_levels=(1,)), 8
    else:
        proj, d = P.anisotropic([1.0, 2.0, 1.5, 3.0], 5.0, 5, 4), 4
    x = util.brownian_path(3, 25, d, seed=13, dtype=dtype)
    _run_sig(ps, oracle, x, proj.depth, proj=proj)
    win = util.sliding_windows(25, 10, 5)
    _run_sig(ps, oracle, x, proj.depth, proj=proj, windows=win)


def _oracle_logsig(oracle, mod, x64, g64, windows):
    if mod.alternative_projection:
        return oracle.logsignature(x64, mod.depth, top_words=mod._top_words.cpu(),
                                   ext_level_sizes=mod._ext_level_sizes, indices=mod._indices_from_sig.cpu(),
                                   windows=windows, grad_out=g64)
    return oracle.logsignature(x64, mod.depth, windows=windows, grad_out=g64)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth,projected", [(2, 5, False), (3, 4, False), (3, 5, True), (4, 6, True), (5, 2, True)])
@pytest.mark.parametrize("windowed", [False, True])
@pytest.mark.parametrize("algo", ["auto", "generic"])  # row in shared memory / streamed through global scratch
def test_logsignature(ps, oracle, dtype, d, depth, projected, windowed, algo):
    x = util.brownian_path(3, 21, d, seed=17 + d, dtype=dtype)
    win = util.sliding_windows(21, 9, 4) if windowed else None
    proj = ps.projections.lyndon(depth, d) if projected else None
    mod = ps.LogSignature(depth=depth, projection=proj, windows=None if win is None else win.to(DEV))
    xg = x.to(DEV).requires_grad_(True)
    ps.ops.set_algorithm(algo)
    try:
        out = mod(xg)
        g = util.normal_like(out.shape, 23, dtype)
        (out * g.to(DEV)).sum().backward()
    finally:
        ps.ops.set_algorithm("auto")
    want, want_grad = _oracle_logsig(oracle, mod, x.double(), g.double(), win)
    assert out.shape == want.shape
    assert util.rel_error(out, want) < util.TOL[dtype]
    assert util.rel_error(xg.grad, want_grad) < util.TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("projected", [False, True])
def test_logsignature_of_rows_beyond_shared_memory(ps, oracle, dtype, projected):
    """d = 6 at depth 6: the 9 330 scalars of the degrees below the top do not fit the shared-memory form
    five times over, so the same Horner kernels run on global scratch (the operator's cache forward, its
    workspace backward).  Values and input gradient against the oracle, dense and Lyndon top degree."""
    from pathsig_b200 import _load
    d, depth = 6, 6
    x = util.brownian_path(2, 9, d, seed=29, dtype=dtype)
    proj = ps.projections.lyndon(depth, d) if projected else None
    mod = ps.LogSignature(depth=depth, projection=proj)
    ls = mod._ext_level_sizes if projected else [0] + [d ** k for k in range(1, depth + 1)]
    assert not ps.ops.logsig_projected_supported(dtype, depth, d, ls)      # the row does not fit shared memory
    xg = x.to(DEV).requires_grad_(True)
    out = mod(xg)
    g = util.normal_like(out.shape, 31, dtype)
    (out * g.to(DEV)).sum().backward()
    want, want_grad = _oracle_logsig(oracle, mod, x.double(), g.double(), None)
    assert out.shape == want.shape
    assert util.rel_error(out, want) < util.TOL[dtype]
    assert util.rel_error(xg.grad, want_grad) < util.TOL[dtype]


def test_zero_batch_and_errors(ps):
    sig = ps.Signature(depth=3)
    assert sig(torch.zeros(0, 5, 2, device=DEV)).shape == (0, 14)
    with pytest.raises(RuntimeError):
        sig(torch.zeros(2, 1, 2, device=DEV))          # fewer than 2 points
    with pytest.raises(RuntimeError):
        sig(torch.zeros(2, 5, 2, device=DEV, dtype=torch.float16))
    with pytest.raises(RuntimeError):
        sig(torch.zeros(2, 5, 2))                      # CPU tensor: there is no CPU implementation
    with pytest.raises(ValueError):
        ps.Signature(depth=13)
    with pytest.raises(TypeError):
        ps.Signature(depth=2, windows=torch.zeros(3, 2, dtype=torch.int32))  # CPU windows


def test_empty_and_out_of_range_windows(ps, oracle):
    x = util.brownian_path(2, 12, 3, seed=1, dtype=torch.float64)
    none = torch.empty((0, 2), dtype=torch.int32, device=DEV)
    xg = x.to(DEV).requires_grad_(True)
    out = ps.Signature(depth=2, windows=none)(xg)
    assert out.shape == (2, 0, 12)
    out.sum().backward()
    assert torch.all(xg.grad == 0)
    # a window reaching past the end is clamped to the points that exist
    win = torch.tensor([[8, 20], [-3, 5]], dtype=torch.int32, device=DEV)
    got = ps.Signature(depth=2, windows=win)(x.to(DEV))
    assert util.rel_error(got[:, 0], oracle.sig_forward(x[:, 8:12], 2)) < 1e-12
    assert util.rel_error(got[:, 1], oracle.sig_forward(x[:, 0:5], 2)) < 1e-12
    x32 = util.brownian_path(2, 40, 8, seed=2, dtype=torch.float32)
    win = torch.tensor([[30, 99]], dtype=torch.int32, device=DEV)
    got = ps.Signature(depth=4, windows=win)(x32.to(DEV))  # tiled kernels
    want = oracle.sig_forward(x32[:, 30:40].double(), 4)
    assert max(util.level_rel_errors(got[:, 0], want, util.level_widths(8, 4))) < 1e-5


def test_non_contiguous_input_and_inference_mode(ps, oracle):
    x = util.brownian_path(4, 20, 6, seed=2, dtype=torch.float64)
    xt = x.to(DEV).transpose(0, 1).contiguous().transpose(0, 1)  # non-contiguous view, same values
    assert not xt.is_contiguous()
    with torch.inference_mode():
        out = ps.Signature(depth=3)(xt)
    assert util.rel_error(out, oracle.sig_forward(x, 3)) < 1e-12


def test_reference_build_agrees(ps, oracle):
    """Same tensors through the reference's own CUDA operators (when its library was built)."""
    ref = util.reference_ops()
    if ref is None:
        pytest.skip("oracle/_ref/libpathsig_ops.so not built")
    empty_w = torch.empty(0, dtype=torch.int64, device=DEV)
    empty_win = torch.empty((0, 2), dtype=torch.int32, device=DEV)
    for dtype in (torch.float32, torch.float64):
        x = util.brownian_path(4, 50, 4, seed=31, dtype=dtype).to(DEV)
        ours = ps.ops.compute_signature(x, 4, False, empty_w, [], False, empty_win)
        theirs = ref.compute_signature(x, 4, False, empty_w, [], False, empty_win)
        _check_levels(ours, theirs, util.level_widths(4, 4), dtype, "vs reference forward")
        g = util.normal_like(ours.shape, 5, dtype).to(DEV)
        ours_g = ps.ops.signature_backward(x, ours, g, 4, False, empty_w, [], False, empty_win)
        theirs_g = ref.signature_backward(x, theirs, g, 4, False, empty_w, [], False, empty_win)
        assert util.rel_error(ours_g, theirs_g) < util.TOL[dtype]
        ls = [0, 4, 16, 64, 256]
        ours_l, ours_c = ps.ops.sig_to_logsig(ours, 4, 4, False, empty_w, ls)
        theirs_l, theirs_c = ref.sig_to_logsig(theirs, 4, 4, False, empty_w, ls)
        assert util.rel_error(ours_l, theirs_l) < util.TOL[dtype]
        ours_gs = ps.ops.logsig_backward(ours, ours_c, g, 4, False, empty_w, ls)
        theirs_gs = ref.logsig_backward(theirs, theirs_c, g, 4, False, empty_w, ls)
        assert util.rel_error(ours_gs, theirs_gs) < util.TOL[dtype]


# ---- register-tiled kernels (dense, or dense below a projected top degree) ----

TILED = [(8, 4), (16, 4), (16, 3), (4, 6),
         (3, 5), (3, 6), (3, 7), (4, 4), (4, 5), (4, 7), (5, 4), (5, 5), (5, 6), (6, 4), (6, 5),
         (8, 3), (8, 5), (8, 6), (10, 3), (10, 4), (12, 3), (16, 2), (32, 2), (32, 3),
         (2, 8), (2, 10), (5, 3), (6, 3), (6, 6), (7, 3), (7, 4), (9, 3), (9, 4), (12, 4), (20, 3)]
# shapes whose unit is one thread block and whose top degree fits the shared-memory staging
TILED_PROJECTED_TOP = [(4, 6), (8, 4), (16, 3), (3, 5), (3, 6), (3, 7), (4, 4), (4, 5), (5, 4), (5, 5), (6, 4),
                       (6, 5), (8, 3), (10, 3), (12, 3), (16, 2), (32, 2),
                       (2, 8), (2, 10), (5, 3), (6, 3), (7, 3), (7, 4), (9, 3), (9, 4), (20, 3)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth", TILED)
@pytest.mark.parametrize("L", [2, 3, 34, 101])
def test_tiled_signature(ps, oracle, d, depth, L, dtype):
    x = util.brownian_path(3, L, d, seed=L + d, dtype=dtype)
    _run_sig(ps, oracle, x, depth, algo="tiled")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth", TILED)
def test_tiled_windows(ps, oracle, d, depth, dtype):
    x = util.brownian_path(2, 70, d, seed=d, dtype=dtype)
    win = torch.tensor([[0, 70], [5, 7], [10, 50], [3, 3], [12, 13], [20, 70], [0, 41], [33, 66]], dtype=torch.int32)
    _run_sig(ps, oracle, x, depth, windows=win, algo="tiled")


def test_tiled_unsupported_shape_is_an_error(ps):
    ps.ops.set_algorithm("tiled")
    try:
        with pytest.raises(RuntimeError):
            ps.Signature(depth=5)(torch.zeros(1, 4, 11, device=DEV))
    finally:
        ps.ops.set_algorithm("auto")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth", TILED_PROJECTED_TOP)
@pytest.mark.parametrize("windowed", [False, True])
def test_tiled_projected_top_degree(ps, oracle, d, depth, windowed, dtype):
    """Dense degrees below a projected top degree (the LogSignature layout) on the tiled kernels."""
    top = util.random_words(37, d, depth, depth, seed=d)
    proj = ps.projections.words(top, depth, d, full_levels=tuple(range(1, depth)))
    assert proj.level_sizes[depth] == 37
    x = util.brownian_path(3, 45, d, seed=3 * d, dtype=dtype)
    win = util.sliding_windows(45, 20, 9) if windowed else None
    _run_sig(ps, oracle, x, depth, proj=proj, windows=win, algo="tiled")
    _run_sig(ps, oracle, x, depth, proj=proj, windows=win, algo="generic")


def test_lyndon_logsignature_float32_on_tiled_kernels(ps, oracle):
    d, depth = 4, 6
    x = util.brownian_path(4, 60, d, seed=99, dtype=torch.float32)
    mod = ps.LogSignature(depth=depth, projection=ps.projections.lyndon(depth, d))
    ps.ops.set_algorithm("tiled")
    try:
        xg = x.to(DEV).requires_grad_(True)
        out = mod(xg)
        g = util.normal_like(out.shape, 7, torch.float32)
        (out * g.to(DEV)).sum().backward()
    finally:
        ps.ops.set_algorithm("auto")
    want, want_grad = _oracle_logsig(oracle, mod, x.double(), g.double(), None)
    assert util.rel_error(out, want) < util.TOL[torch.float32]
    assert util.rel_error(xg.grad, want_grad) < util.TOL[torch.float32]


# ---- batches of 32+ units: the generic "one lane per unit" kernels ----

@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth", [(2, 5), (3, 4), (5, 3), (6, 2), (2, 12)])
def test_many_units_dense(ps, oracle, dtype, d, depth):
    x = util.brownian_path(45, 23, d, seed=d * depth, dtype=dtype)
    _run_sig(ps, oracle, x, depth, algo="generic")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_many_units_ragged_windows_and_projection(ps, oracle, dtype):
    x = util.brownian_path(9, 50, 4, seed=77, dtype=dtype)
    win = torch.tensor([[0, 50], [5, 7], [10, 30], [3, 3], [12, 13], [20, 50], [0, 21], [44, 50]], dtype=torch.int32)
    _run_sig(ps, oracle, x, 4, windows=win, algo="generic")                       # 72 units of unequal length
    proj = ps.projections.words(util.random_words(70, 4, 1, 5, seed=8), 5, 4)
    _run_sig(ps, oracle, x, 5, proj=proj, windows=win)
    _run_sig(ps, oracle, util.brownian_path(64, 31, 4, seed=3, dtype=dtype), 5, proj=ps.projections.lyndon(5, 4))
