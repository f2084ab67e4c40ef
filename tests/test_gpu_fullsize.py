"""The five benchmark configurations at their full sizes, checked through properties that do
not need a full-size oracle run:

* degree 1 equals the total increment, and the shuffle identity S(i)S(j) = S(ij) + S(ji);
* translation invariance: the signature ignores a constant shift of the path, so the gradient
  with respect to the path sums to zero over time, per path and channel;
* a random subset of rows / windows against the CPU oracle (float64 on the float32 inputs);
* Chen's identity on a long path: S(x[0:L]) = S(x[0:m]) (x) S(x[m-1:L]) at degree 2;
* the register-tiled and the generic kernels agree on a subset.
Inputs are the seeded synthetic Brownian paths of bench.py.
"""
from __future__ import annotations

import pytest
import torch

import bench

from . import util

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-5
# Input gradients against the float64 oracle.  Measured over full batches: 4e-7 .. 1.5e-6 of the
# largest entry (worst single path 4e-6) for the four signature configurations, below the
# reference's own float32 error on the same inputs (5e-7 .. 2.7e-6).
GRAD_TOL = 1e-5
# The float32 log-signature of config 4 loses digits to the cancellation inside the logarithm: this
# library is 2.6e-5 from the float64 value at degree 6 and 1.2e-5 in the gradient, the reference
# 3.8e-5 and 1.8e-5 (tests/test_gpu_reference_fullsize.py asserts the three-way comparison).
LOG_F32_TOL = 5e-5


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _fwd_bwd(wl):
    x = wl.x.detach().clone().requires_grad_(True)
    out = wl.mod(x)
    out.backward(wl.G)
    return out.detach(), x.grad.detach()


def _check_level_one_and_shuffle(out, x, d, windows=None):
    if windows is None:
        total = (x[:, -1] - x[:, 0]).double()
        s = out.double()
    else:
        w0, w1 = windows[3].tolist()
        total = (x[:, w1 - 1] - x[:, w0]).double()
        s = out[:, 3].double()
    scale = total.abs().max().item()
    assert (s[:, :d] - total).abs().max().item() < TOL * scale
    lvl2 = s[:, d: d + d * d].reshape(-1, d, d)
    prod = s[:, :d, None] * s[:, None, :d]
    assert (lvl2 + lvl2.transpose(1, 2) - prod).abs().max().item() < 4 * TOL * max(1.0, prod.abs().max().item())


def _check_translation_invariance(grad):
    g = grad.double()
    assert g.sum(dim=1).abs().max().item() < 2e-5 * g.abs().sum(dim=1).max().item()


def test_config1_full_against_oracle(ps, oracle):
    wl = bench.Workload("cfg1").build(DEV)
    out, grad = _fwd_bwd(wl)
    x64 = wl.x.double().cpu()
    want = oracle.sig_forward(x64, 4)
    assert max(util.level_rel_errors(out, want, util.level_widths(8, 4))) < TOL
    want_grad = oracle.sig_backward(x64, want, wl.G.double().cpu(), 4)
    assert util.rel_error(grad, want_grad) < GRAD_TOL
    _check_translation_invariance(grad)


def test_config2_full(ps, oracle):
    wl = bench.Workload("cfg2").build(DEV)
    assert wl.x.shape == (256, 1024, 8) and wl.windows.shape == (61, 2)
    out, grad = _fwd_bwd(wl)
    assert out.shape == (256, 61, 4680)
    _check_level_one_and_shuffle(out, wl.x, 8, wl.windows)
    _check_translation_invariance(grad)
    # subset of paths, all windows, against the oracle (forward and backward)
    rows = [0, 97, 255]
    x64 = wl.x[rows].double().cpu()
    want = oracle.sig_forward(x64, 4, windows=wl.windows)
    assert max(util.level_rel_errors(out[rows], want, util.level_widths(8, 4))) < TOL
    want_grad = oracle.sig_backward(x64, want, wl.G[rows].double().cpu(), 4, windows=wl.windows)
    assert util.rel_error(grad[rows], want_grad) < GRAD_TOL
    # the generic kernels on a slice of the batch
    ps.ops.set_algorithm("generic")
    try:
        small = bench.Workload("cfg2", B=4).build(DEV)
        out_g, grad_g = _fwd_bwd(small)
    finally:
        ps.ops.set_algorithm("auto")
    out_t, grad_t = _fwd_bwd(small)
    assert max(util.level_rel_errors(out_t, out_g, util.level_widths(8, 4))) < TOL
    assert util.rel_error(grad_t, grad_g) < GRAD_TOL


def test_config3_full(ps, oracle):
    wl = bench.Workload("cfg3").build(DEV)
    out, grad = _fwd_bwd(wl)
    proj = wl.mod.projection
    assert out.shape == (512, proj.sig_size) and proj.sig_size == 208
    total = (wl.x[:, -1] - wl.x[:, 0]).double()
    assert (out[:, :8].double() - total).abs().max().item() < TOL * total.abs().max().item()
    _check_translation_invariance(grad)
    rows = [0, 300, 511]
    x64 = wl.x[rows].double().cpu()
    want = oracle.sig_forward(x64, 6, proj.encoded_words.cpu(), proj.level_sizes)
    assert max(util.level_rel_errors(out[rows], want, util.level_widths(8, 6, proj.level_sizes))) < TOL
    want_grad = oracle.sig_backward(x64, want, wl.G[rows].double().cpu(), 6, proj.encoded_words.cpu(), proj.level_sizes)
    assert util.rel_error(grad[rows], want_grad) < GRAD_TOL


def test_config4_full(ps, oracle):
    wl = bench.Workload("cfg4").build(DEV)
    out, grad = _fwd_bwd(wl)
    mod = wl.mod
    assert out.shape == (1024, 964)
    total = (wl.x[:, -1] - wl.x[:, 0]).double()
    assert (out[:, :4].double() - total).abs().max().item() < TOL * total.abs().max().item()  # log S at degree 1
    _check_translation_invariance(grad)
    rows = [0, 511, 1023]
    want, want_grad = oracle.logsignature(wl.x[rows].double().cpu(), 6, top_words=mod._top_words.cpu(),
                                          ext_level_sizes=mod._ext_level_sizes, indices=mod._indices_from_sig.cpu(),
                                          grad_out=wl.G[rows].double().cpu())
    widths = util.level_widths(4, 6, mod.projection.level_sizes)
    per_degree = util.level_rel_errors(out[rows], want, widths)
    assert max(per_degree[:4]) < TOL and max(per_degree) < LOG_F32_TOL, per_degree
    assert util.rel_error(grad[rows], want_grad) < LOG_F32_TOL


def test_config5_shard(ps, oracle):
    """One GPU's share (512 paths) of the 4 096-path batch at its full length and width."""
    wl = bench.Workload("cfg5", B=512).build(DEV)
    out, grad = _fwd_bwd(wl)
    assert out.shape == (512, 69904)
    _check_level_one_and_shuffle(out, wl.x, 16)
    _check_translation_invariance(grad)
    # Chen at degree 2 for a split in the middle: S2(x) = S2(a) + S2(b) + S1(a) (x) S1(b)
    m = 1000
    sig = ps.Signature(depth=4)
    a = sig(wl.x[:8, :m].contiguous()).double()
    b = sig(wl.x[:8, m - 1:].contiguous()).double()
    s2 = out[:8, 16:272].double().reshape(8, 16, 16)
    chen = a[:, 16:272].reshape(8, 16, 16) + b[:, 16:272].reshape(8, 16, 16) + a[:, :16, None] * b[:, None, :16]
    assert (s2 - chen).abs().max().item() < TOL * s2.abs().max().item()
    # eight paths spread over the shard against the oracle, forward and backward
    rows = [0, 1, 77, 200, 301, 400, 510, 511]
    x64 = wl.x[rows].double().cpu()
    want = oracle.sig_forward(x64, 4)
    assert max(util.level_rel_errors(out[rows], want, util.level_widths(16, 4))) < TOL
    want_grad = oracle.sig_backward(x64, want, wl.G[rows].double().cpu(), 4)
    assert util.rel_error(grad[rows], want_grad) < GRAD_TOL
