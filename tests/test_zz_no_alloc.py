"""psig_sig_backward_static: the signature backward for callers that cannot allocate.

Some hosts of this library have no way to give the backward kernel its scratch accumulator: the
card's memory belongs to a pre-sized arena, or the call sits in a hook that is not allowed to
allocate.  For them the library carries a fixed 8 MiB array and exposes one entry point that uses
it.  This test drives that entry point straight through the C ABI (ctypes, raw device pointers),
twice in a row on the same inputs, and compares both results with the regular entry point fed
with caller-provided scratch.  It also checks that a problem beyond the fixed array is refused
with an error instead of being run.

The file name sorts last on purpose: if this addition ever fails, `pytest -x` has already run
everything else.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from . import util

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _desc(_load, x, depth, windows=None):
    desc = _load.SigDesc()
    desc.dtype = _load.PSIG_F32 if x.dtype == torch.float32 else _load.PSIG_F64
    desc.B, desc.L, desc.d = x.shape
    desc.depth = depth
    desc.algo = _load.ALGO_GENERIC
    if windows is not None:
        desc.W = windows.shape[0]
        desc.windows = windows.data_ptr()
    return desc


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("windowed", [False, True])
def test_static_scratch_entry_point_matches_regular_one(dtype, windowed):
    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    d, depth = 3, 4
    x = util.brownian_path(5, 40, d, seed=77, dtype=dtype).to(DEV)
    win = torch.tensor([[0, 40], [3, 17], [10, 12], [25, 40]], dtype=torch.int32, device=DEV) if windowed else None
    desc = _desc(_load, x, depth, win)
    D = lib.psig_sig_size(ctypes.byref(desc))
    assert D == 120
    shape = (5, 4, D) if windowed else (5, D)
    sig = torch.empty(shape, dtype=dtype, device=DEV)
    assert lib.psig_sig_forward(ctypes.byref(desc), _ptr(x), _ptr(sig), stream) == 0
    g = util.normal_like(shape, 5, dtype).to(DEV)

    # regular entry point, scratch supplied by the caller
    ws_bytes = lib.psig_sig_backward_workspace(ctypes.byref(desc))
    assert ws_bytes > 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    want = torch.empty_like(x)
    assert lib.psig_sig_backward(ctypes.byref(desc), _ptr(x), _ptr(sig), _ptr(g), _ptr(want), _ptr(ws), ws_bytes,
                                 stream) == 0

    # the entry point under test: no scratch argument, called twice back to back
    assert ws_bytes <= lib.psig_sig_backward_static_limit()
    first = torch.full_like(x, float("nan"))
    second = torch.full_like(x, float("nan"))
    assert lib.psig_sig_backward_static(ctypes.byref(desc), _ptr(x), _ptr(sig), _ptr(g), _ptr(first), stream) == 0
    assert lib.psig_sig_backward_static(ctypes.byref(desc), _ptr(x), _ptr(sig), _ptr(g), _ptr(second), stream) == 0
    torch.cuda.synchronize()
    tol = util.TOL[dtype]
    assert util.rel_error(first, want) < tol
    assert util.rel_error(second, want) < tol

    # The reason the entry point exists: a call takes no device memory.  After the warm calls above
    # (the first one may load the kernels' module) the free memory of the device and the bytes held
    # by torch's allocator are the same before and after one more call.
    third = torch.full_like(x, float("nan"))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    held_before = torch.cuda.memory_allocated()
    assert lib.psig_sig_backward_static(ctypes.byref(desc), _ptr(x), _ptr(sig), _ptr(g), _ptr(third), stream) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after >= free_before  # nothing was taken from the device
    assert torch.cuda.memory_allocated() == held_before
    assert util.rel_error(third, want) < tol


def test_static_scratch_entry_point_refuses_oversized_problems():
    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    limit = lib.psig_sig_backward_static_limit()
    assert limit == 8 << 20
    # 4 * 64 * 4095 * 8 bytes = 8 MiB minus 2 KiB fits; one more path does not
    x = torch.zeros(65, 4096, 8, dtype=torch.float32, device=DEV)
    desc = _desc(_load, x, 2)
    assert 4 * 65 * 4095 * 8 > limit
    out = torch.zeros_like(x)
    sig = torch.zeros(65, 72, dtype=torch.float32, device=DEV)
    rc = lib.psig_sig_backward_static(ctypes.byref(desc), _ptr(x), _ptr(sig), _ptr(sig), _ptr(out), None)
    assert rc == -8  # PSIG_ERR_TOO_LARGE
    assert b"exceeds" in lib.psig_status_string(rc)
