"""The shape sweeps of the reference's own test-suite, run against the reference's CUDA build.

The reference checks itself against keras_sig / pysiglib (absent here) over batch sizes, sequence
lengths, truncation levels at d = 3 and channel counts at depth 3, on inputs X = 200*rand - 100, with
three metrics: whole-tensor forward error max|a-b| / max(1, max|b|), gradient dot-product error against
random directions, and gradient error at three time steps (tests/test_sig.py:73-151 and
tests/test_logsig.py:75-154 of the reference).  Here the same sweeps, inputs, metrics and tolerances are
applied to this library in both dtypes, with the reference's operators (compiled unchanged,
``oracle/_ref``) evaluated in float64 on the same inputs in the place of the third-party oracle.
The dot-product metric divides by a sum in which the gradient's few large entries cancel, so at some
shapes it magnifies float32 rounding past the reference's bound for ANY float32 implementation; the
reference's own float32 result is therefore put through the same metric, and a bound is
max(the reference's tolerance, twice what the reference itself reaches).
Skipped when that build is absent.
"""
from __future__ import annotations

import pytest
import torch

from . import util

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float64, torch.float32]
BATCHES = [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]
LENGTHS = [10, 20, 50, 100, 200, 500, 1000]
DEPTHS = [2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12]
CHANNELS = [2, 3, 4, 5, 7, 10, 12, 15, 18, 20, 22, 26, 30, 35, 40, 45, 50, 75, 100]


@pytest.fixture(scope="module")
def ref():
    ops = util.reference_ops()
    if ops is None:
        pytest.skip("reference build (oracle/_ref/libpathsig_ops.so) not present")
    return ops


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _sig_tolerances(dtype, depth):
    # the reference's own bounds (tests/test_sig.py:25-34 of the reference), except the float64 forward
    # bound: two float64 implementations that sum in different orders differ by a few ulps of the
    # largest coefficient, so 1e-13 / 1e-12 stand in for its 1e-14 / 1e-13
    if dtype == torch.float64:
        return (1e-13 if depth < 10 else 1e-12), (1e-12 if depth < 10 else 1e-11)
    return (1e-6 if depth < 10 else 1e-5), (1e-4 if depth < 10 else 1e-3)


def _log_tolerances(dtype, depth):
    if dtype == torch.float64:
        return (1e-12 if depth < 10 else 1e-11), (1e-10 if depth < 10 else 1e-9)
    return (1e-5 if depth < 10 else 1e-4), (1e-3 if depth < 10 else 1e-2)


def _inputs(B, T, d, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (200 * torch.rand((B, T, d), generator=g, dtype=torch.float64) - 100).to(dtype).to(DEV)


def _metrics(out, grad, ref_out, ref_grad, T):
    res = {}
    res["fwd"] = (out.double() - ref_out.double()).abs().max().item() / max(1.0, ref_out.double().abs().max().item())
    g = torch.Generator().manual_seed(7)
    dots = []
    for _ in range(5):
        H = torch.randn(grad.shape, generator=g, dtype=torch.float64).to(DEV)
        a, b = (grad.double() * H).sum().item(), (ref_grad.double() * H).sum().item()
        dots.append(abs(a - b) / max(1.0, abs(b)))
    res["grad_dot"] = max(dots)
    steps = [0, T // 2, T - 1] if T > 2 else [0]
    res["grad_timestep"] = max(
        (grad[:, t].double() - ref_grad[:, t].double()).abs().max().item() /
        max(1.0, ref_grad[:, t].double().abs().max().item()) for t in steps)
    return res


def _compare_signature(ps, ref, B, T, d, depth, dtype):
    x = _inputs(B, T, d, dtype)
    xa = x.clone().requires_grad_(True)
    out = ps.Signature(depth=depth)(xa)
    G = util.normal_like(out.shape, 3, dtype).to(DEV)
    (out * G).sum().backward()
    nowords = torch.empty(0, dtype=torch.int64, device=DEV)
    nowin = torch.empty((0, 2), dtype=torch.int32, device=DEV)
    x64, G64 = x.double(), G.double()
    ref_out = ref.compute_signature(x64, depth, False, nowords, [], False, nowin)
    ref_grad = ref.signature_backward(x64, ref_out, G64, depth, False, nowords, [], False, nowin)
    own_out = ref.compute_signature(x, depth, False, nowords, [], False, nowin)
    own_grad = ref.signature_backward(x, own_out, G, depth, False, nowords, [], False, nowin)
    return _metrics(out.detach(), xa.grad, ref_out, ref_grad, T), _metrics(own_out, own_grad, ref_out, ref_grad, T)


def _compare_logsignature(ps, ref, B, T, d, depth, dtype):
    x = _inputs(B, T, d, dtype)
    mod = ps.LogSignature(depth=depth, projection=ps.projections.lyndon(depth=depth, path_dim=d))
    xa = x.clone().requires_grad_(True)
    out = mod(xa)
    G = util.normal_like(out.shape, 3, dtype).to(DEV)
    (out * G).sum().backward()
    ls, tw, idx = list(mod._ext_level_sizes), mod._top_words, mod._indices_from_sig
    nowin = torch.empty((0, 2), dtype=torch.int32, device=DEV)
    x64 = x.double()
    sig = ref.compute_signature(x64, depth, True, tw, ls, False, nowin)
    logsig, cache = ref.sig_to_logsig(sig, depth, d, True, tw, ls)
    g_full = torch.zeros_like(logsig).index_add_(-1, idx, G.double())
    g_sig = ref.logsig_backward(sig, cache, g_full, depth, True, tw, ls)
    ref_grad = ref.signature_backward(x64, sig, g_sig, depth, True, tw, ls, False, nowin)
    sig32 = ref.compute_signature(x, depth, True, tw, ls, False, nowin)
    logsig32, cache32 = ref.sig_to_logsig(sig32, depth, d, True, tw, ls)
    g_full32 = torch.zeros_like(logsig32).index_add_(-1, idx, G)
    own_grad = ref.signature_backward(x, sig32, ref.logsig_backward(sig32, cache32, g_full32, depth, True, tw, ls),
                                      depth, True, tw, ls, False, nowin)
    want = logsig.index_select(-1, idx)
    return (_metrics(out.detach(), xa.grad, want, ref_grad, T),
            _metrics(logsig32.index_select(-1, idx), own_grad, want, ref_grad, T))


def _assert(both, tol_fwd, tol_rel):
    res, reference_itself = both
    assert res["fwd"] < max(tol_fwd, 2 * reference_itself["fwd"]), both
    assert res["grad_dot"] < max(tol_rel, 2 * reference_itself["grad_dot"]), both
    assert res["grad_timestep"] < max(tol_rel, 2 * reference_itself["grad_timestep"]), both


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B", BATCHES)
def test_signature_batch_sizes(ps, ref, dtype, B):
    _assert(_compare_signature(ps, ref, B, 50, 3, 4, dtype), *_sig_tolerances(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", LENGTHS)
def test_signature_sequence_lengths(ps, ref, dtype, T):
    _assert(_compare_signature(ps, ref, 4, T, 3, 4, dtype), *_sig_tolerances(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("depth", DEPTHS)
def test_signature_truncation_levels(ps, ref, dtype, depth):
    _assert(_compare_signature(ps, ref, 4, 50, 3, depth, dtype), *_sig_tolerances(dtype, depth))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", CHANNELS)
def test_signature_path_dimensions(ps, ref, dtype, d):
    _assert(_compare_signature(ps, ref, 2, 10, d, 3, dtype), *_sig_tolerances(dtype, 3))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("B", BATCHES)
def test_logsignature_batch_sizes(ps, ref, dtype, B):
    _assert(_compare_logsignature(ps, ref, B, 50, 3, 4, dtype), *_log_tolerances(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", LENGTHS)
def test_logsignature_sequence_lengths(ps, ref, dtype, T):
    _assert(_compare_logsignature(ps, ref, 4, T, 3, 4, dtype), *_log_tolerances(dtype, 4))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("depth", DEPTHS)
def test_logsignature_truncation_levels(ps, ref, dtype, depth):
    _assert(_compare_logsignature(ps, ref, 4, 50, 3, depth, dtype), *_log_tolerances(dtype, depth))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", CHANNELS)
def test_logsignature_path_dimensions(ps, ref, dtype, d):
    _assert(_compare_logsignature(ps, ref, 2, 10, d, 3, dtype), *_log_tolerances(dtype, 3))
