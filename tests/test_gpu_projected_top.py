"""Projected top degree on the register-tiled kernels: threads that own no listed word skip the top
target degree when the caller provides a host copy of the word list (``PsigSigDesc.words_host``).

The skip must not change a single bit of the requested words, and the input gradient only by the order
in which the threads' shares are summed: the same call is made through the C ABI with and without the host
copy (without it nothing is skipped), for word lists that leave whole warps without a listed word, lists
that do not, and a list with a word listed twice.  Values and gradients are also checked against the CPU
oracle.
The row layout is the one ``LogSignature`` asks for (src/pathsig/modules.py:96-111 of the reference):
every degree below the top dense, the top degree an explicit word list.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from . import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _desc(_load, x, depth, codes_dev, codes_host, windows):
    desc = _load.SigDesc()
    desc.dtype = _load.PSIG_F32 if x.dtype == torch.float32 else _load.PSIG_F64
    desc.B, desc.L, desc.d = x.shape
    desc.depth = depth
    desc.projected = 1
    d = x.shape[2]
    for k in range(1, depth):
        desc.level_sizes[k] = d ** k
    desc.level_sizes[depth] = codes_dev.numel()
    desc.words = codes_dev.data_ptr()
    desc.words_host = codes_host.data_ptr() if codes_host is not None else None
    desc.algo = _load.ALGO_TILED
    if windows is not None:
        desc.W = windows.shape[0]
        desc.windows = windows.data_ptr()
    return desc


def _run(_load, lib, x, depth, codes, host, windows):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    codes_dev = codes.to(DEV)
    desc = _desc(_load, x, depth, codes_dev, codes if host else None, windows)
    width = lib.psig_sig_size(ctypes.byref(desc))
    d = x.shape[2]
    assert width == sum(d ** k for k in range(1, depth)) + codes.numel()
    shape = (x.shape[0], windows.shape[0], width) if windows is not None else (x.shape[0], width)
    sig = torch.full(shape, float("nan"), dtype=x.dtype, device=DEV)
    assert lib.psig_sig_forward(ctypes.byref(desc), _ptr(x), _ptr(sig), stream) == 0
    g = util.normal_like(shape, 23, x.dtype).to(DEV)
    ws_bytes = lib.psig_sig_backward_workspace(ctypes.byref(desc))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=DEV)
    gx = torch.full_like(x, float("nan"))
    assert lib.psig_sig_backward(ctypes.byref(desc), _ptr(x), _ptr(sig), _ptr(g), _ptr(gx), _ptr(ws), ws_bytes,
                                 stream) == 0
    torch.cuda.synchronize()
    return sig, gx, g


def _codes(kind, d, depth):
    top = d ** depth
    if kind == "one_prefix":      # every listed word starts with the first letter twice: most threads own none
        return torch.arange(0, top // (d * d), 3, dtype=torch.int64)
    if kind == "last_prefixes":   # owners are the last threads of the unit
        return torch.arange(top - top // d, top, 5, dtype=torch.int64)
    if kind == "lyndon":
        import pathsig_b200 as ps
        proj = ps.projections.lyndon(depth, d, device="cpu")
        sizes = proj.level_sizes
        return proj.encoded_words[-sizes[depth]:].clone()
    if kind == "repeated":        # a word listed twice has two columns; both receive gradient
        return torch.tensor([5, 5, 7, top - 1, 0, 5], dtype=torch.int64)
    if kind == "everywhere":      # every thread owns a word: nothing to skip
        return torch.arange(0, top, 2, dtype=torch.int64)
    raise AssertionError(kind)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("d,depth", [(4, 6), (3, 5), (8, 4), (5, 4)])
@pytest.mark.parametrize("kind", ["one_prefix", "last_prefixes", "lyndon", "repeated", "everywhere"])
@pytest.mark.parametrize("windowed", [False, True])
def test_skipping_unlisted_prefixes_changes_no_bit(oracle, dtype, d, depth, kind, windowed):
    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    codes = _codes(kind, d, depth)
    x = util.brownian_path(5, 19, d, seed=41, dtype=dtype).to(DEV)
    windows = torch.tensor([[0, 19], [2, 9], [7, 8], [11, 19]], dtype=torch.int32, device=DEV) if windowed else None
    sig_a, gx_a, g = _run(_load, lib, x, depth, codes, True, windows)
    sig_b, gx_b, _ = _run(_load, lib, x, depth, codes, False, windows)
    assert torch.equal(sig_a, sig_b)
    # the block sums the threads' shares of dL/d(dx) in slot order, which the reordering changes
    assert util.rel_error(gx_a, gx_b) < util.TOL[dtype]
    # against the oracle in float64, same row layout
    ls = [0] + [d ** k for k in range(1, depth)] + [codes.numel()]
    xd = x.double().cpu()
    win_cpu = None if windows is None else windows.cpu()
    want = oracle.sig_forward(xd, depth, codes, ls, win_cpu)
    assert util.rel_error(sig_a, want) < util.TOL[dtype]
    want_gx = oracle.sig_backward(xd, want, g.double().cpu(), depth, codes, ls, win_cpu)
    assert util.rel_error(gx_a, want_gx) < util.TOL[dtype]
