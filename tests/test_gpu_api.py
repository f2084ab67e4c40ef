"""API-level behaviour on the GPU: the self-consistency properties the reference's own test-suite
checks (tests/test_windows.py and tests/test_projections.py of the reference), restated for this
package: windowed == per-slice, projected == columns of the full result, gradients of overlapping
windows add up, float64 gradcheck, shapes, buffers and operator registration checks."""
from __future__ import annotations

import itertools

import pytest
import torch

from . import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ps():
    import pathsig_b200
    return pathsig_b200


def _path(B, L, d, seed=42, dtype=torch.float64):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, L, d, generator=g, dtype=torch.float64).to(dtype).to(DEV)


def _full_columns(proj):
    d, cols, off, used = proj.path_dim, [], 0, 0
    codes = proj.encoded_words.tolist()
    for n in range(1, proj.depth + 1):
        size = proj.level_sizes[n]
        if size == d ** n:
            cols.extend(range(off, off + d ** n))
        elif size > 0:
            cols.extend(off + c for c in codes[used: used + size])
            used += size
        off += d ** n
    return torch.tensor(cols, dtype=torch.int64, device=DEV)


@pytest.mark.parametrize("kind", ["sig", "logsig"])
@pytest.mark.parametrize("depth,d", [(2, 2), (3, 3), (4, 4), (4, 2)])
def test_windowed_equals_per_slice(ps, kind, depth, d):
    x = _path(3, 50, d)
    win = util.sliding_windows(50, 15, 5, device=DEV)
    cls = ps.Signature if kind == "sig" else ps.LogSignature
    windowed = cls(depth=depth, windows=win)(x)
    plain = cls(depth=depth)
    assert windowed.shape[:2] == (3, win.shape[0])
    for w, (s, e) in enumerate(win.tolist()):
        torch.testing.assert_close(windowed[:, w], plain(x[:, s:e]), atol=1e-10, rtol=1e-10)


def test_window_edge_patterns(ps):
    x = _path(2, 30, 3)
    sig = ps.Signature(depth=3)
    for win in ([[0, 30]], [[0, 2], [28, 30]], [[0, 10], [10, 20], [20, 30]], [[5, 25], [0, 30], [7, 9]]):
        w = torch.tensor(win, dtype=torch.int64, device=DEV)  # int64 windows are accepted
        out = ps.Signature(depth=3, windows=w)(x)
        for i, (s, e) in enumerate(win):
            torch.testing.assert_close(out[:, i], sig(x[:, s:e]), atol=1e-10, rtol=1e-10)


def test_overlapping_window_gradients_add_up(ps):
    x = _path(2, 24, 3)
    win = torch.tensor([[0, 12], [6, 18], [10, 24], [3, 5]], dtype=torch.int32, device=DEV)
    xa = x.clone().requires_grad_(True)
    out = ps.Signature(depth=3, windows=win)(xa)
    g = torch.randn_like(out)
    (out * g).sum().backward()
    expect = torch.zeros_like(x)
    for i, (s, e) in enumerate(win.tolist()):
        xi = x[:, s:e].clone().requires_grad_(True)
        (ps.Signature(depth=3)(xi) * g[:, i]).sum().backward()
        expect[:, s:e] += xi.grad
    torch.testing.assert_close(xa.grad, expect, atol=1e-10, rtol=1e-10)


@pytest.mark.parametrize("make", [
    lambda P: P.lyndon(4, 3),
    lambda P: P.lyndon(3, 4, full_levels=(2,)),
    lambda P: P.words([(0,), (2,), (1, 1), (0, 2), (2, 1, 0), (1, 0, 0, 2)], 4, 3),
    lambda P: P.words([(0, 1), (1, 1, 0)], 3, 2, full_levels=(1,)),
    lambda P: P.anisotropic([1.0, 2.0, 1.5], 4.5, 4, 3),
    lambda P: P.anisotropic([1.0, 1.0], 3.0, 3, 2, full_levels=(1, 2)),
])
def test_projected_equals_columns_of_full(ps, make):
    proj = make(ps.projections)
    x = _path(3, 17, proj.path_dim)
    cols = _full_columns(proj)
    xa = x.clone().requires_grad_(True)
    out = ps.Signature(depth=proj.depth, projection=proj)(xa)
    assert out.shape == (3, proj.sig_size)
    xb = x.clone().requires_grad_(True)
    full = ps.Signature(depth=proj.depth)(xb)
    torch.testing.assert_close(out, full[:, cols], atol=1e-11, rtol=1e-11)
    g = torch.randn_like(out)
    (out * g).sum().backward()
    (full[:, cols] * g).sum().backward()
    torch.testing.assert_close(xa.grad, xb.grad, atol=1e-10, rtol=1e-10)


def test_lyndon_logsignature_equals_columns_of_full_log(ps):
    for d, depth in [(2, 5), (3, 4), (4, 3)]:
        proj = ps.projections.lyndon(depth, d)
        x = _path(2, 14, d)
        out = ps.LogSignature(depth=depth, projection=proj)(x)
        full = ps.LogSignature(depth=depth)(x)
        torch.testing.assert_close(out, full[:, _full_columns(proj)], atol=1e-11, rtol=1e-11)


def test_projection_ignores_extra_channels(ps):
    """Words over the first d0 letters of a wider path give the signature of the narrower path."""
    d0, extra, depth = 2, 2, 3
    x = _path(2, 12, d0 + extra)
    words = [w for n in range(1, depth + 1) for w in itertools.product(range(d0), repeat=n)]
    proj = ps.projections.words(words, depth, d0 + extra)
    out = ps.Signature(depth=depth, projection=proj)(x)
    narrow = ps.Signature(depth=depth)(x[:, :, :d0].contiguous())
    torch.testing.assert_close(out, narrow, atol=1e-11, rtol=1e-11)


@pytest.mark.parametrize("case", ["sig", "sig_windows", "sig_lyndon", "logsig", "logsig_lyndon_windows"])
def test_gradcheck_float64(ps, case):
    d, depth = 2, 3
    x = (_path(2, 6, d, seed=3) * 0.5).requires_grad_(True)
    win = torch.tensor([[0, 4], [2, 6]], dtype=torch.int32, device=DEV)
    mod = {
        "sig": lambda: ps.Signature(depth=depth),
        "sig_windows": lambda: ps.Signature(depth=depth, windows=win),
        "sig_lyndon": lambda: ps.Signature(depth=depth, projection=ps.projections.lyndon(depth, d)),
        "logsig": lambda: ps.LogSignature(depth=depth),
        "logsig_lyndon_windows": lambda: ps.LogSignature(depth=depth, projection=ps.projections.lyndon(depth, d),
                                                         windows=win),
    }[case]()
    assert torch.autograd.gradcheck(mod, (x,), eps=1e-6, atol=1e-6, rtol=1e-5, nondet_tol=1e-9)


def test_shapes_dtypes_and_state_dict(ps):
    x32 = _path(4, 9, 3, dtype=torch.float32)
    assert ps.Signature(depth=3)(x32).dtype == torch.float32
    assert ps.Signature(depth=3)(x32).shape == (4, 39)
    assert ps.LogSignature(depth=3)(x32).shape == (4, 39)
    proj = ps.projections.lyndon(3, 3)
    assert ps.LogSignature(depth=3, projection=proj)(x32).shape == (4, proj.sig_size)
    win = util.sliding_windows(9, 4, 2, device=DEV)
    m = ps.LogSignature(depth=3, projection=proj, windows=win)
    assert m(x32).shape == (4, win.shape[0], proj.sig_size)
    sd = m.state_dict()
    assert set(sd) == {"_windows", "_encoded_words", "_top_words", "_indices_from_sig"}
    m2 = ps.LogSignature(depth=3, projection=ps.projections.lyndon(3, 3), windows=win.clone())
    m2.load_state_dict(sd)
    torch.testing.assert_close(m2(x32), m(x32))
    assert ps.Signature(depth=2)(x32.double()).dtype == torch.float64


def test_operator_registration_checks(ps):
    """torch.library.opcheck: schema, fake implementation and autograd registration of each operator."""
    x = _path(2, 7, 2).requires_grad_(True)
    no_words = torch.empty(0, dtype=torch.int64, device=DEV)
    no_win = torch.empty((0, 2), dtype=torch.int32, device=DEV)
    ops = torch.ops.pathsig_b200
    tests = ("test_schema", "test_faketensor", "test_autograd_registration")
    torch.library.opcheck(ops.compute_signature.default, (x, 3, False, no_words, [], False, no_win), test_utils=tests)
    sig = ops.compute_signature(x, 3, False, no_words, [], False, no_win).detach().requires_grad_(True)
    torch.library.opcheck(ops.sig_to_logsig.default, (sig, 3, 2, False, no_words, [0, 2, 4, 8]), test_utils=tests)
    g = torch.randn_like(sig)
    torch.library.opcheck(ops.signature_backward.default, (x.detach(), sig.detach(), g, 3, False, no_words, [],
                                                            False, no_win), test_utils=("test_schema", "test_faketensor"))
    _, cache = ops.sig_to_logsig(sig.detach(), 3, 2, False, no_words, [0, 2, 4, 8])
    torch.library.opcheck(ops.logsig_backward.default, (sig.detach(), cache, g, 3, False, no_words, [0, 2, 4, 8]),
                          test_utils=("test_schema", "test_faketensor"))


def test_cuda_graph_capture_and_replay(ps):
    """Forward and backward enqueue work on the current stream only (no allocation inside the
    library, no synchronisation), so a whole step can be captured once and replayed."""
    x = _path(8, 40, 8, dtype=torch.float32).requires_grad_(True)
    win = util.sliding_windows(40, 16, 8, device=DEV)
    mod = ps.Signature(depth=4, windows=win)
    w = torch.randn(8, win.shape[0], 4680, device=DEV)

    def step():
        out = mod(x)
        (grad,) = torch.autograd.grad((out * w).sum(), x)
        return out, grad

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm up off the default stream, as graph capture requires
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g, grad_g = step()
    want_out, want_grad = step()
    with torch.no_grad():
        x.mul_(0.5)                      # new input values in the captured buffer
    graph.replay()
    torch.cuda.synchronize()
    ref_out, ref_grad = step()
    torch.testing.assert_close(out_g, ref_out, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(grad_g, ref_grad, rtol=1e-4, atol=1e-5)
    assert not torch.allclose(ref_out, want_out)


def test_traced_by_torch_compile(ps):
    """The operators trace under torch.compile (fake implementations + registered autograd): a compiled
    function gives the eager result, forward and backward, without graph breaks."""
    win = torch.tensor([[0, 12], [5, 20]], dtype=torch.int32, device=DEV)
    sig = ps.Signature(depth=3, windows=win)
    logsig = ps.LogSignature(depth=4, projection=ps.projections.lyndon(4, 3))

    def fn(x):
        a = sig(x)
        b = logsig(x)
        c = ps.chen_product(a[:, 0], a[:, 1], path_dim=3, depth=3)
        return a.square().sum() + b.sum() + c.sum()

    compiled = torch.compile(fn, backend="aot_eager", fullgraph=True)
    x1 = _path(3, 20, 3).requires_grad_(True)
    x2 = x1.detach().clone().requires_grad_(True)
    y1, y2 = fn(x1), compiled(x2)
    y1.backward()
    y2.backward()
    assert torch.allclose(y1, y2, rtol=1e-12, atol=0)
    assert torch.allclose(x1.grad, x2.grad, rtol=1e-10, atol=1e-12)


def test_concurrent_host_threads_and_streams(ps):
    """The operators are re-entrant: four host threads, each on its own stream and its own shape, get the
    results a single thread gets (the reference's launchers are re-entrant too, guarded per device)."""
    import threading

    shapes = [(8, 4, False), (3, 5, False), (5, 3, True), (4, 6, True)]  # (d, depth, log-signature)
    inputs = [_path(6, 40 + 3 * i, d, seed=i) for i, (d, _, _) in enumerate(shapes)]

    def work(i, stream, out):
        d, depth, log = shapes[i]
        mod = ps.LogSignature(depth=depth) if log else ps.Signature(depth=depth)
        with torch.cuda.stream(stream):
            for _ in range(5):
                x = inputs[i].clone().requires_grad_(True)
                y = mod(x)
                y.square().sum().backward()
            out[i] = (y.detach(), x.grad)
            stream.synchronize()

    serial, threaded = {}, {}
    for i in range(len(shapes)):
        work(i, torch.cuda.current_stream(), serial)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream() for _ in shapes]
    threads = [threading.Thread(target=work, args=(i, streams[i], threaded)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    for i in range(len(shapes)):
        assert util.rel_error(threaded[i][0], serial[i][0]) < 1e-12
        assert util.rel_error(threaded[i][1], serial[i][1]) < 1e-11


@pytest.mark.parametrize("d,depth,B,L,dtype,log", [
    (3, 3, 70000, 4, torch.float32, False),   # lane kernels, more unit groups than one grid dimension holds
    (8, 4, 70000, 3, torch.float32, False),   # tiled kernels, 70 000 blocks
    (2, 2, 200000, 2, torch.float64, False),
    (4, 3, 70000, 5, torch.float32, True),    # log-signature rows beyond 65 535
])
def test_batches_beyond_grid_limits(ps, d, depth, B, L, dtype, log):
    """The reference maps batch and windows to grid.y / grid.z and so stops at 65 535 of each
    (src/pathsig/forward/sig_launch.cu:47); here sampled rows of a larger batch equal the same rows
    computed on their own."""
    x = _path(B, L, d, seed=B % 97, dtype=dtype)
    mod = (ps.LogSignature if log else ps.Signature)(depth=depth)
    xg = x.clone().requires_grad_(True)
    out = mod(xg)
    out.square().sum().backward()
    rows = torch.tensor([0, 1, B // 2, 65535, 65536, B - 1], device=DEV)
    xs = x[rows].clone().requires_grad_(True)
    sub = mod(xs)
    sub.square().sum().backward()
    tol = 2e-5 if dtype == torch.float32 else 1e-11
    assert torch.isfinite(out).all() and torch.isfinite(xg.grad).all()
    assert util.rel_error(out[rows], sub) < tol
    assert util.rel_error(xg.grad[rows], xs.grad) < tol


def test_bad_word_codes_and_foreign_devices_raise_on_the_host(ps):
    """Codes outside their degree and operands on another device are refused before any launch."""
    proj = ps.projections.words([(0, 1), (2, 2), (1, 0, 2)], 3, 3, full_levels=(1,), device=DEV)
    proj._host_codes[1] = 9          # not a word of degree 2 over 3 letters
    proj._codes[1] = 9
    with pytest.raises(ValueError, match="outside"):
        ps.Signature(depth=3, projection=proj)
    with pytest.raises(ValueError, match="outside"):
        ps.LogSignature(depth=3, projection=proj)
    good = ps.projections.words([(0, 1), (2, 2), (1, 0, 2)], 3, 3, full_levels=(1,), device=DEV)
    mod = ps.Signature(depth=3, projection=good)
    bad_state = {k: v.clone() for k, v in mod.state_dict().items()}
    bad_state["_encoded_words"][2] = 27
    with pytest.raises(ValueError, match="outside"):
        mod.load_state_dict(bad_state)
    # a CPU tensor among CUDA operands: refused by the operator itself
    x = _path(2, 8, 3)
    with pytest.raises(RuntimeError, match="same device|must be CUDA"):
        ps.ops.compute_signature(x, 3, True, good.encoded_words.cpu(), good.level_sizes, False,
                                 torch.empty((0, 2), dtype=torch.int32, device=DEV))
    if torch.cuda.device_count() > 1:
        other = good.encoded_words.to("cuda:1")
        with pytest.raises(RuntimeError, match="same device"):
            ps.ops.compute_signature(x, 3, True, other, good.level_sizes, False,
                                     torch.empty((0, 2), dtype=torch.int32, device=DEV))


def test_loaded_column_index_with_repeats_keeps_every_gradient(ps):
    """A state_dict may replace the column index by one that selects a column twice; the gradients of
    both selections must add up (the scatter used for repeat-free indices would drop one)."""
    proj = ps.projections.lyndon(3, 3, device=DEV)
    mod = ps.LogSignature(depth=3, projection=proj)
    assert mod._columns_repeat is False
    state = {k: v.clone() for k, v in mod.state_dict().items()}
    state["_indices_from_sig"][1] = state["_indices_from_sig"][0]
    mod.load_state_dict(state)
    assert mod._columns_repeat is True
    x = _path(2, 12, 3).requires_grad_(True)
    out = mod(x)
    g = torch.randn_like(out)
    (out * g).sum().backward()
    full = ps.LogSignature(depth=3)
    x2 = x.detach().clone().requires_grad_(True)
    sel = full(x2)
    # columns of the hybrid layout == columns of the dense log-signature below the top degree
    idx = state["_indices_from_sig"]
    dense_cols = _full_columns(proj)
    hybrid_to_dense = torch.cat([torch.arange(3 + 9, device=DEV), dense_cols[3 + 3:]])  # degrees 1, 2 dense; top listed
    (sel.index_select(-1, hybrid_to_dense[idx]) * g).sum().backward()
    torch.testing.assert_close(x.grad, x2.grad, atol=1e-10, rtol=1e-10)


def test_bounded_wait_of_the_bulk_staging_runs_out_harmlessly(ps, oracle):
    """The tiled forward stages long un-windowed paths with bulk copies and waits for each chunk a bounded
    number of polls.  With the bound lowered to zero polls the wait runs out at once, the blocks fall back
    to plain loads of the same bytes and count the event; results are unchanged.  The bound is restored
    afterwards."""
    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    x = util.brownian_path(6, 300, 8, seed=4, dtype=torch.float32)     # 299 steps: five chunks of 64
    want = oracle.sig_forward(x.double(), 4)
    sig = ps.Signature(depth=4)
    torch.cuda.synchronize()
    assert lib.psig_bulk_copy_timeouts() >= 0                          # read and clear
    out_default = sig(x.to(DEV))
    torch.cuda.synchronize()
    assert lib.psig_bulk_copy_timeouts() == 0                          # copies land in time normally
    try:
        assert lib.psig_set_bulk_wait_polls(0) == 0
        out_short = sig(x.to(DEV))
        torch.cuda.synchronize()
        missed = lib.psig_bulk_copy_timeouts()
    finally:
        assert lib.psig_set_bulk_wait_polls(-1) == 0
    assert missed > 0
    widths = util.level_widths(8, 4)
    assert max(util.level_rel_errors(out_short, want, widths)) < 1e-5
    assert torch.equal(out_short, out_default)                          # same bytes, same arithmetic


@pytest.mark.parametrize("algo", ["tiled", "generic", "closure"])
def test_run_to_run_reproducibility(ps, algo):
    """What is promised about bits: the forward pass of every kernel family gives the same bytes on every run,
    and so does the tiled backward when one block holds the unit and no windows overlap (its sums run in a fixed
    order and it stores instead of adding).  The paths that add with float atomics (overlapping windows, the
    generic and closure backward) are only checked to agree within the float32 tolerance."""
    d, depth = (3, 4) if algo == "closure" else (8, 4)   # a small word tree keeps the run-time compilation short
    x = util.brownian_path(64, 200, d, seed=5, dtype=torch.float32).to(DEV)
    win = util.sliding_windows(200, 64, 16, device=DEV)
    ps.ops.set_algorithm(algo)
    try:
        for windows in (None, win):
            mod = ps.Signature(depth=depth, windows=windows)
            outs, grads = [], []
            for _ in range(3):
                xr = x.clone().requires_grad_(True)
                out = mod(xr)
                g = util.normal_like(out.shape, 3, torch.float32).to(DEV)
                (out * g).sum().backward()
                outs.append(out.detach().clone())
                grads.append(xr.grad.clone())
            assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
            if algo == "tiled" and windows is None:
                assert torch.equal(grads[0], grads[1]) and torch.equal(grads[0], grads[2])
            else:
                assert util.rel_error(grads[1], grads[0]) < util.TOL[torch.float32]
                assert util.rel_error(grads[2], grads[0]) < util.TOL[torch.float32]
        # the logarithm (row in shared memory) is reproducible forward
        log = ps.LogSignature(depth=depth)
        a, b = log(x), log(x)
        assert torch.equal(a, b)
    finally:
        ps.ops.set_algorithm("auto")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_deterministic_mode_gives_a_bit_reproducible_backward_at_16_channels(ps, dtype):
    """At d = 16, depth 4 a path spans 16 blocks of the reverse sweep, which by default add their shares of
    the path gradient with float atomics (run-dependent last bits).  Under
    ``torch.use_deterministic_algorithms(True)`` every block stores into its own slab of the workspace and
    the slabs are summed in a fixed order: same bits on every run, same values as the default path within
    the tolerance; the library reports which of the two it will run."""
    import ctypes

    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    x = util.brownian_path(6, 50, 16, seed=3, dtype=dtype).to(DEV)
    mod = ps.Signature(depth=4)

    def grads(n):
        out = []
        for _ in range(n):
            xr = x.clone().requires_grad_(True)
            y = mod(xr)
            g = util.normal_like(y.shape, 7, dtype).to(DEV)
            y.backward(g)
            out.append(xr.grad.clone())
        return out

    default = grads(1)[0]
    was = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        fixed = grads(4)
    finally:
        torch.use_deterministic_algorithms(was)
    assert all(torch.equal(fixed[0], g) for g in fixed[1:])
    assert util.rel_error(fixed[0], default) < util.TOL[dtype]
    desc = _load.SigDesc()
    desc.dtype = _load.PSIG_F32 if dtype == torch.float32 else _load.PSIG_F64
    desc.B, desc.L, desc.d, desc.depth = 6, 50, 16, 4
    assert lib.psig_sig_backward_reproducible(ctypes.byref(desc)) == 0
    assert lib.psig_sig_backward_workspace(ctypes.byref(desc)) == 0
    desc.flags = _load.FLAG_DETERMINISTIC
    assert lib.psig_sig_backward_reproducible(ctypes.byref(desc)) == 1
    blocks_per_path = 16 if dtype == torch.float32 else 32   # the float64 instance owns half as many first letters per thread
    assert lib.psig_sig_backward_workspace(ctypes.byref(desc)) == x.element_size() * 6 * blocks_per_path * 50 * 16
    desc.d, desc.flags = 8, 0                      # one block per unit: reproducible without the flag
    assert lib.psig_sig_backward_reproducible(ctypes.byref(desc)) == 1
