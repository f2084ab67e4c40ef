"""The five benchmark configurations at full size against the reference's own CUDA operators.

The reference build (``oracle/_ref/libpathsig_ops.so``, compiled unchanged by ``oracle/build_ref.py``)
and this library run on the same seeded tensors, full batches (config 5: one GPU's 512-path shard at
its full length and width).  Both metrics are asserted: whole tensor ``max|a-b| / max(1, max|b|)``
(the reference's own, ``tests/test_sig.py:88-91`` of the reference) and per degree
``max|a-b| / max|b|``; the input gradient over the whole ``(B, L, d)`` tensor.

Tolerance 1e-5 in float32 for the signature configurations.  The float32 log-signature of config 4
is the exception the numbers force: the reference's own result is 2e-5 .. 4e-5 away from the float64
value at degree 6 (cancellation in the logarithm) and its gradient differs by 8e-6 from one run of the
reference to the next (float atomics), so no implementation can sit within 1e-5 of it.  There the test
is three-way against a float64 evaluation: this library must be within 1e-5 of the float64 value or
at least as close to it as the reference is, per degree and for the gradient.
Skipped when the reference build is absent.
"""
from __future__ import annotations

import pytest
import torch

import bench

from . import util

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-5


@pytest.fixture(scope="module")
def ref():
    ops = util.reference_ops()
    if ops is None:
        pytest.skip("reference build (oracle/_ref/libpathsig_ops.so) not present")
    return ops


def _ours(wl, dtype=torch.float32):
    x = wl.x.to(dtype).detach().clone().requires_grad_(True)
    out = wl.mod(x)
    out.backward(wl.G.to(dtype))
    return out.detach(), x.grad.detach()


def _reference(ref, wl):
    m = wl.mod
    if wl.spec["kind"] == "loglyndon":
        ls, tw, idx = list(m._ext_level_sizes), m._top_words, m._indices_from_sig
        sargs = (m.depth, m.alternative_projection, tw, ls, m.use_windows, m._windows)
        sig = ref.compute_signature(wl.x, *sargs)
        logsig, cache = ref.sig_to_logsig(sig, m.depth, wl.d, m.alternative_projection, tw, ls)
        g_full = torch.zeros_like(logsig).index_add_(-1, idx, wl.G)
        g_sig = ref.logsig_backward(sig, cache, g_full, m.depth, m.alternative_projection, tw, ls)
        return logsig.index_select(-1, idx), ref.signature_backward(wl.x, sig, g_sig, *sargs)
    args = (m.depth, m.alternative_projection, m._encoded_words, list(m._level_sizes), m.use_windows, m._windows)
    sig = ref.compute_signature(wl.x, *args)
    return sig, ref.signature_backward(wl.x, sig, wl.G, *args)


def _whole(a, b):
    return ((a.double() - b.double()).abs().max() / b.double().abs().max().clamp(min=1.0)).item()


@pytest.mark.parametrize("name,B", [("cfg1", None), ("cfg2", None), ("cfg3", None), ("cfg5", 512)])
def test_full_batch_matches_reference_build(ref, name, B):
    wl = bench.Workload(name, B=B).build(DEV)
    out, grad = _ours(wl)
    ref_out, ref_grad = _reference(ref, wl)
    assert out.shape == ref_out.shape and grad.shape == ref_grad.shape
    per_degree = util.level_rel_errors(out, ref_out, wl.degree_widths())
    assert max(per_degree) < TOL, per_degree
    assert _whole(out, ref_out) < TOL
    assert util.rel_error(grad, ref_grad) < TOL


def test_config4_log_signature_three_way(ref):
    wl = bench.Workload("cfg4").build(DEV)
    widths = wl.degree_widths()
    out, grad = _ours(wl)
    ref_out, ref_grad = _reference(ref, wl)
    true_out, true_grad = _ours(wl, torch.float64)   # the same kernels in float64 (pinned to 1e-11 elsewhere)
    ours_err = util.level_rel_errors(out, true_out, widths)
    ref_err = util.level_rel_errors(ref_out, true_out, widths)
    for k, (a, b) in enumerate(zip(ours_err, ref_err), start=1):
        assert a < max(TOL, b), f"degree {k}: ours {a:.2e}, reference {b:.2e} (both against float64)"
    assert max(ours_err[:4]) < TOL                     # degrees 1-4 carry no cancellation to speak of
    g_ours, g_ref = util.rel_error(grad, true_grad), util.rel_error(ref_grad, true_grad)
    assert g_ours < max(TOL, g_ref), f"gradient: ours {g_ours:.2e}, reference {g_ref:.2e} (both against float64)"
    # and the two float32 results agree as far as their own errors allow
    assert max(util.level_rel_errors(out, ref_out, widths)) < 1e-4
    assert util.rel_error(grad, ref_grad) < 1e-4
