"""Chen product of truncated signatures on the GPU (an operator the reference does not have):
checked against the definition-level tensor algebra, against Chen's identity on signatures
computed by this package, and through float64 gradcheck / gradgradcheck."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from . import tensor_algebra as ta
from . import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _levels(flat, d, depth):
    out, off = [np.ones(())], 0
    for k in range(1, depth + 1):
        out.append(flat[off: off + d ** k].reshape((d,) * k))
        off += d ** k
    return out


@pytest.mark.parametrize("d,depth", [(1, 5), (2, 6), (3, 4), (5, 3), (8, 4), (4, 1), (16, 3)])
@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-13), (torch.float32, 2e-6)])
def test_matches_tensor_algebra(ps, d, depth, dtype, tol):
    D = sum(d ** k for k in range(1, depth + 1))
    a = util.normal_like((3, D), 1) * 0.5
    b = util.normal_like((3, D), 2) * 0.5
    got = ps.chen_product(a.to(dtype).to(DEV), b.to(dtype).to(DEV), path_dim=d, depth=depth).double().cpu()
    for r in range(3):
        want = ta.flatten(ta.mul(_levels(a[r].numpy(), d, depth), _levels(b[r].numpy(), d, depth), depth))
        assert util.rel_error(got[r], torch.from_numpy(want)) < tol


@pytest.mark.parametrize("d,depth,L,m", [(8, 4, 40, 17), (3, 6, 25, 1), (16, 3, 30, 28), (2, 8, 20, 10)])
def test_chen_identity(ps, d, depth, L, m):
    x = util.brownian_path(4, L, d, seed=5).to(DEV)
    sig = ps.Signature(depth=depth)
    whole = sig(x)
    glued = ps.chen_product(sig(x[:, : m + 1].contiguous()), sig(x[:, m:].contiguous()), path_dim=d, depth=depth)
    widths = util.level_widths(d, depth)
    assert max(util.level_rel_errors(glued, whole, widths)) < 1e-11


def test_windows_from_pieces(ps):
    """A (B, W, D) batch of window signatures glued from two halves of each window."""
    d, depth = 4, 5
    x = util.brownian_path(3, 65, d, seed=9, dtype=torch.float32).to(DEV)
    lo = torch.tensor([[0, 17], [16, 33], [32, 49]], dtype=torch.int32, device=DEV)
    hi = torch.tensor([[16, 33], [32, 49], [48, 65]], dtype=torch.int32, device=DEV)
    both = torch.tensor([[0, 33], [16, 49], [32, 65]], dtype=torch.int32, device=DEV)
    a = ps.Signature(depth=depth, windows=lo)(x)
    b = ps.Signature(depth=depth, windows=hi)(x)
    want = ps.Signature(depth=depth, windows=both)(x)
    got = ps.chen_product(a, b, path_dim=d, depth=depth)
    assert got.shape == want.shape
    assert max(util.level_rel_errors(got, want, util.level_widths(d, depth))) < 1e-5


@pytest.mark.parametrize("d,depth", [(2, 4), (3, 3), (6, 4)])
def test_gradients(ps, d, depth):
    D = sum(d ** k for k in range(1, depth + 1))
    a = (util.normal_like((2, D), 3) * 0.5).to(DEV).requires_grad_(True)
    b = (util.normal_like((2, D), 4) * 0.5).to(DEV).requires_grad_(True)
    fn = lambda p, q: ps.chen_product(p, q, path_dim=d, depth=depth)
    assert torch.autograd.gradcheck(fn, (a, b), eps=1e-6, atol=1e-8, rtol=1e-6, nondet_tol=0.0)
    if D <= 64:
        assert torch.autograd.gradgradcheck(fn, (a, b), eps=1e-6, atol=1e-8, rtol=1e-6)


def test_gradient_through_glued_signature(ps):
    """dL/dx through two half signatures and the product equals dL/dx through the whole signature."""
    d, depth, L, m = 8, 4, 33, 16
    x0 = util.brownian_path(2, L, d, seed=11).to(DEV)
    G = util.normal_like((2, sum(d ** k for k in range(1, depth + 1))), 12).to(DEV)
    sig = ps.Signature(depth=depth)
    x1 = x0.clone().requires_grad_(True)
    (sig(x1) * G).sum().backward()
    x2 = x0.clone().requires_grad_(True)
    glued = ps.chen_product(sig(x2[:, : m + 1].contiguous()), sig(x2[:, m:].contiguous()), path_dim=d, depth=depth)
    (glued * G).sum().backward()
    assert util.rel_error(x2.grad, x1.grad) < 1e-11


def test_backward_is_reproducible(ps):
    d, depth = 8, 4
    D = sum(d ** k for k in range(1, depth + 1))
    a = util.normal_like((16, D), 1, dtype=torch.float32).to(DEV)
    b = util.normal_like((16, D), 2, dtype=torch.float32).to(DEV)
    g = util.normal_like((16, D), 3, dtype=torch.float32).to(DEV)
    first = ps.ops.chen_product_backward(a, b, g, depth, d)
    again = ps.ops.chen_product_backward(a, b, g, depth, d)
    assert torch.equal(first[0], again[0]) and torch.equal(first[1], again[1])


def test_argument_checks_and_opcheck(ps):
    d, depth = 3, 3
    D = 3 + 9 + 27
    a = torch.randn(2, D, device=DEV, dtype=torch.float64, requires_grad=True)
    b = torch.randn(2, D, device=DEV, dtype=torch.float64, requires_grad=True)
    with pytest.raises(RuntimeError):
        ps.chen_product(a[:, :-1], b[:, :-1], path_dim=d, depth=depth)
    with pytest.raises(RuntimeError):
        ps.chen_product(a, b.float(), path_dim=d, depth=depth)
    with pytest.raises(ValueError):
        ps.chen_product(a, b, path_dim=d, depth=13)
    assert ps.chen_product(a[:0], b[:0], path_dim=d, depth=depth).shape == (0, D)
    torch.library.opcheck(torch.ops.pathsig_b200.chen_product.default, (a, b, depth, d))
    g = torch.randn(2, D, device=DEV, dtype=torch.float64)
    torch.library.opcheck(torch.ops.pathsig_b200.chen_product_backward.default,
                          (a.detach(), b.detach(), g, depth, d), test_utils=("test_schema", "test_faketensor"))


@pytest.mark.parametrize("d,depth", [(2, 7), (4, 4), (8, 4), (6, 3)])
@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-13), (torch.float32, 2e-6)])
def test_matches_oracle_forward_and_backward(ps, oracle, d, depth, dtype, tol):
    D = sum(d ** k for k in range(1, depth + 1))
    a = util.normal_like((2, 3, D), 5) * 0.4
    b = util.normal_like((2, 3, D), 6) * 0.4
    g = util.normal_like((2, 3, D), 7)
    want, grad_fn = oracle.chen_product(a.to(dtype).double(), b.to(dtype).double(), d, depth)
    want_ga, want_gb = grad_fn(g.to(dtype).double())
    got = ps.ops.chen_product(a.to(dtype).to(DEV), b.to(dtype).to(DEV), depth, d)
    got_ga, got_gb = ps.ops.chen_product_backward(a.to(dtype).to(DEV), b.to(dtype).to(DEV), g.to(dtype).to(DEV), depth, d)
    assert util.rel_error(got, want) < tol
    assert util.rel_error(got_ga, want_ga) < tol and util.rel_error(got_gb, want_gb) < tol
