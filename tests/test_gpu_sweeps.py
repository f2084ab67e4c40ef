"""Shape sweeps in the style of the reference's own tests (tests/test_sig.py:115-151 and
tests/test_logsig.py:118-154 sweep batch, length, depth at d=3 and d at depth 3, on inputs
X = 200*rand - 100), here against the CPU oracle instead of keras_sig / pysiglib.
Sizes are trimmed so that the float64 oracle stays in seconds."""
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


def _uniform_path(B, T, d, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (200 * torch.rand(B, T, d, generator=g, dtype=torch.float64) - 100).to(dtype)


def _check(ps, oracle, x, depth, logsig=False):
    dtype = x.dtype
    tol = util.TOL[dtype]
    mod = ps.LogSignature(depth=depth, projection=ps.projections.lyndon(depth, x.shape[-1])) if logsig \
        else ps.Signature(depth=depth)
    xg = x.to(DEV).requires_grad_(True)
    out = mod(xg)
    g = util.normal_like(out.shape, 5, dtype)
    (out * g.to(DEV)).sum().backward()
    x64 = x.double()
    if logsig:
        want, want_grad = oracle.logsignature(x64, depth, top_words=mod._top_words.cpu(),
                                              ext_level_sizes=mod._ext_level_sizes,
                                              indices=mod._indices_from_sig.cpu(), grad_out=g.double())
        # whole-tensor metric as in the reference's log-signature tests; float32 carries the
        # cancellation of the logarithm on these large-amplitude inputs
        assert util.rel_error(out, want) < (1e-4 if dtype == torch.float32 else tol)
        assert util.rel_error(xg.grad, want_grad) < (1e-3 if dtype == torch.float32 else 1e-10)
    else:
        want = oracle.sig_forward(x64, depth)
        want_grad = oracle.sig_backward(x64, want, g.double(), depth)
        errs = util.level_rel_errors(out, want, util.level_widths(x.shape[-1], depth))
        assert max(errs) < tol, errs
        # gradients on X ~ U(-100, 100): the reference's own bounds are 1e-4 (float32) and 1e-12
        assert util.rel_error(xg.grad, want_grad) < (1e-4 if dtype == torch.float32 else 1e-11)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("B", [1, 2, 33, 128, 512])
def test_batch_sweep(ps, oracle, dtype, B):
    _check(ps, oracle, _uniform_path(B, 20, 3, dtype, seed=B), 4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("T", [2, 10, 100, 1000])
def test_length_sweep(ps, oracle, dtype, T):
    _check(ps, oracle, _uniform_path(2, T, 3, dtype, seed=T), 4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("depth", [1, 2, 3, 5, 7, 9, 10, 12])
def test_depth_sweep(ps, oracle, dtype, depth):
    _check(ps, oracle, _uniform_path(2, 12, 3, dtype, seed=depth), depth)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d", [2, 4, 7, 10, 16, 40, 100])
def test_channel_sweep(ps, oracle, dtype, d):
    _check(ps, oracle, _uniform_path(2, 10, d, dtype, seed=d), 3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth,B,T", [(2, 6, 40, 30), (3, 5, 3, 200), (5, 3, 64, 15), (4, 4, 1, 50)])
def test_lyndon_logsignature_sweep(ps, oracle, dtype, d, depth, B, T):
    _check(ps, oracle, _uniform_path(B, T, d, dtype, seed=d * depth) * 0.01, depth, logsig=True)
