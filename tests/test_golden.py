"""Golden vectors recorded from the reference's own CUDA operators on a B200
(tests/golden/golden_reference.pt, written by tests/golden/make_golden.py).

CPU part: pins the oracle against them (float64 cases to 1e-12, float32 cases to the float32
tolerance, since the recorded float32 outputs carry float32 rounding).
GPU part: the CUDA library against the same vectors.
"""
from __future__ import annotations

import os

import pytest
import torch

from . import util

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden_reference.pt")
_data = torch.load(GOLDEN)
CASES = _data["cases"]
SIG_CASES = sorted(k for k, v in CASES.items() if v["kind"] == "sig")
LOG_CASES = sorted(k for k, v in CASES.items() if v["kind"] == "log")


def _tol(case, f64=1e-12):
    return f64 if case["path"].dtype == torch.float64 else 1e-5


def _widths(case):
    return util.level_widths(case["path"].shape[-1], case["depth"], case["level_sizes"] or None)


def test_golden_file_is_from_the_reference():
    assert "reference CUDA operators" in _data["meta"]["source"]
    assert len(SIG_CASES) >= 8 and len(LOG_CASES) >= 3


@pytest.mark.parametrize("name", SIG_CASES)
def test_oracle_signature_matches_reference(oracle, name):
    c = CASES[name]
    x = c["path"].double()
    ls = c["level_sizes"] or None
    sig = oracle.sig_forward(x, c["depth"], c["words"], ls, c["windows"])
    assert max(util.level_rel_errors(sig, c["sig"], _widths(c))) < _tol(c)
    grad = oracle.sig_backward(x, sig, c["grad_sig"].double(), c["depth"], c["words"], ls, c["windows"])
    assert util.rel_error(grad, c["grad_path"]) < _tol(c, 1e-11)


@pytest.mark.parametrize("name", LOG_CASES)
def test_oracle_logsignature_matches_reference(oracle, name):
    c = CASES[name]
    x = c["path"].double()
    d, depth = x.shape[-1], c["depth"]
    tw = c["top_words"] if c["alt"] else None
    ls = c["level_sizes"] if c["alt"] else None
    sig = oracle.sig_forward(x, depth, tw, ls)
    assert max(util.level_rel_errors(sig, c["sig"], _widths(c))) < _tol(c)
    logsig, P = oracle.sig_to_logsig(sig, depth, d, tw, ls)
    assert util.rel_error(logsig, c["logsig"]) < _tol(c)
    gsig = oracle.logsig_backward(sig, P, c["grad_logsig"].double(), depth, d, tw, ls)
    assert util.rel_error(gsig, c["grad_sig"]) < _tol(c, 1e-11)
    gpath = oracle.sig_backward(x, sig, gsig, depth, tw, ls)
    assert util.rel_error(gpath, c["grad_path"]) < _tol(c, 1e-11)


@pytest.mark.gpu
@pytest.mark.parametrize("algo", ["auto", "generic"])
@pytest.mark.parametrize("name", SIG_CASES)
def test_cuda_signature_matches_reference(name, algo):
    import pathsig_b200 as ps
    c = CASES[name]
    dev = "cuda"
    x = c["path"].to(dev)
    alt = bool(c["level_sizes"])
    use_w = c["windows"] is not None
    win = c["windows"].to(dev) if use_w else torch.empty((0, 2), dtype=torch.int32, device=dev)
    ew = c["words"].to(dev)
    tol = util.TOL[x.dtype]
    ps.ops.set_algorithm(algo)
    try:
        sig = ps.ops.compute_signature(x, c["depth"], alt, ew, c["level_sizes"], use_w, win)
        grad = ps.ops.signature_backward(x, sig, c["grad_sig"].to(dev), c["depth"], alt, ew, c["level_sizes"],
                                         use_w, win)
    finally:
        ps.ops.set_algorithm("auto")
    assert max(util.level_rel_errors(sig, c["sig"], _widths(c))) < tol
    assert util.rel_error(grad, c["grad_path"]) < tol


@pytest.mark.gpu
@pytest.mark.parametrize("name", LOG_CASES)
def test_cuda_logsignature_matches_reference(name):
    import pathsig_b200 as ps
    c = CASES[name]
    dev = "cuda"
    x = c["path"].to(dev)
    d, depth, alt = x.shape[-1], c["depth"], c["alt"]
    tw = c["top_words"].to(dev)
    ls = c["level_sizes"]
    tol = util.TOL[x.dtype]
    no_win = torch.empty((0, 2), dtype=torch.int32, device=dev)
    sig = ps.ops.compute_signature(x, depth, alt, tw, ls if alt else [], False, no_win)
    logsig, cache = ps.ops.sig_to_logsig(sig, depth, d, alt, tw, ls)
    assert util.rel_error(logsig, c["logsig"]) < tol
    gsig = ps.ops.logsig_backward(sig, cache, c["grad_logsig"].to(dev), depth, alt, tw, ls)
    assert util.rel_error(gsig, c["grad_sig"]) < tol
    gpath = ps.ops.signature_backward(x, sig, gsig, depth, alt, tw, ls if alt else [], False, no_win)
    assert util.rel_error(gpath, c["grad_path"]) < tol
