"""CPU tests of the host side: projections, module argument handling, fake (meta) operators,
and that the C-ABI library exports every symbol include/pathsig_b200.h declares."""
from __future__ import annotations

import ctypes
import itertools
import os
import re

import pytest
import torch

import pathsig_b200 as ps
from pathsig_b200 import _load
from pathsig_b200.projections import lyndon_words, projections

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- C ABI ----

def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "pathsig_b200.h")).read()
    declared = set(re.findall(r"\b(psig_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = ctypes.CDLL(_load.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(_load.EXPORTS), "ctypes table and header disagree"


def test_status_strings_and_sizes_without_a_gpu():
    lib = _load.ensure_loaded()
    assert lib.psig_abi_version() == _load.ABI_VERSION
    assert lib.psig_status_string(0) == b"ok"
    assert b"depth" in lib.psig_status_string(-3)
    desc = _load.SigDesc()
    desc.dtype, desc.d, desc.depth, desc.B, desc.L = 0, 8, 4, 2, 10
    assert lib.psig_sig_size(ctypes.byref(desc)) == 4680
    desc.depth = 13
    assert lib.psig_sig_size(ctypes.byref(desc)) == -3
    desc.depth, desc.L = 4, 1
    assert lib.psig_sig_size(ctypes.byref(desc)) == -4
    desc.L, desc.projected = 10, 1
    for k, s in enumerate([0, 8, 3, 0, 5]):
        desc.level_sizes[k] = s
    desc.words = 1 << 20  # any non-null address; nothing is dereferenced by the size query
    assert lib.psig_sig_size(ctypes.byref(desc)) == 16
    ldesc = _load.LogDesc()
    ldesc.dtype, ldesc.d, ldesc.depth, ldesc.rows, ldesc.top_size = 1, 4, 6, 3, 670
    ldesc.top_words = 1 << 20
    assert lib.psig_logsig_size(ctypes.byref(ldesc)) == 1364 + 670
    # rows small enough for the shared-memory form need no scratch; larger rows are streamed through global
    # scratch: four buffers of the degrees below the top plus every T_k (degrees 1..depth-k)
    assert lib.psig_logsig_backward_workspace(ctypes.byref(ldesc)) == 0
    assert lib.psig_logsig_cache_size(ctypes.byref(ldesc)) == 0
    ldesc.d, ldesc.depth, ldesc.top_size, ldesc.top_words = 16, 5, 16 ** 5, None
    width = 16 + 16 ** 2 + 16 ** 3 + 16 ** 4 + 16 ** 5
    lower = width - 16 ** 5
    every_t = sum(sum(16 ** n for n in range(1, 5 - k + 1)) for k in range(1, 5))
    assert lib.psig_logsig_size(ctypes.byref(ldesc)) == width
    assert lib.psig_logsig_cache_size(ctypes.byref(ldesc)) == width * 5
    assert lib.psig_logsig_backward_workspace(ctypes.byref(ldesc)) == 8 * 3 * (4 * lower + every_t)


# ---- projections ----

def _is_lyndon(w):
    return all(w < w[i:] + w[:i] for i in range(1, len(w)))


@pytest.mark.parametrize("d,n", [(2, 1), (2, 6), (3, 4), (4, 6), (5, 3)])
def test_lyndon_words_against_brute_force(d, n):
    want = [w for w in itertools.product(range(d), repeat=n) if _is_lyndon(w)]
    codes = lyndon_words(d, n)
    got = []
    for c in codes:
        w = []
        for _ in range(n):
            w.append(c % d)
            c //= d
        got.append(tuple(reversed(w)))
    assert got == want


def test_lyndon_projection_sizes_and_indices():
    p = projections.lyndon(6, 4, device="cpu")
    assert p.level_sizes == [0, 4, 6, 20, 60, 204, 670]
    assert p.sig_size == 964
    assert p.encoded_words.shape == (960,) and p.encoded_words.dtype == torch.int64
    idx = p.logsig_indices()
    assert idx.shape == (964,)
    assert idx[:4].tolist() == [0, 1, 2, 3]
    assert idx[-670:].tolist() == list(range(1364, 1364 + 670))
    q = projections.lyndon(3, 2, full_levels=(2,), device="cpu")
    assert q.level_sizes == [0, 2, 4, 2]


def test_words_projection_rules():
    p = projections.words([(0,), (1,), (0, 1), (1, 0), (1, 1, 0)], 3, 2, device="cpu")
    assert p.level_sizes == [0, 2, 2, 1]          # degree 1 is complete -> implicit
    assert p.encoded_words.tolist() == [1, 2, 6]
    # a degree given in full is re-ordered to code order and loses its explicit codes
    p = projections.words([(1, 1), (0, 0), (1, 0), (0, 1)], 2, 2, device="cpu")
    assert p.level_sizes == [0, 0, 4] and p.encoded_words.numel() == 0
    # words beyond the depth end the list
    p = projections.words([(0,), (0, 1), (0, 1, 1), (1,)], 2, 2, device="cpu")
    assert p.level_sizes == [0, 1, 1]
    with pytest.raises(ValueError):
        projections.words([(0, 1), (1,)], 2, 2, device="cpu")          # decreasing length
    with pytest.raises(ValueError):
        projections.words([(0, 2)], 2, 2, device="cpu")                 # letter out of range
    with pytest.raises(ValueError):
        projections.words([(0,)], 2, 2, full_levels=(1,), device="cpu")  # explicit words at a full degree
    with pytest.raises(ValueError):
        projections.words([], 2, 1, device="cpu")                        # path_dim < 2
    with pytest.raises(ValueError):
        projections.words([], 13, 2, device="cpu")
    with pytest.raises(ValueError):
        projections.words([], 12, 64, device="cpu")                      # letters do not fit 64/12 bits
    with pytest.raises(ValueError):
        projections.words([], 2, 2, full_levels=(3,), device="cpu")


def test_anisotropic_projection():
    p = projections.anisotropic([1.0, 2.0], 3.0, 3, 2, device="cpu")
    # weight(w) = sum of letter weights <= 3: degree1 {0,1}; degree2 {00,01,10}; degree3 {000}
    assert p.level_sizes == [0, 2, 3, 1]
    assert p.encoded_words.tolist() == [0, 1, 2, 0]
    p = projections.anisotropic(torch.tensor([1.0, 5.0]), 2.0, 3, 2, full_levels=(3,), device="cpu")
    assert p.level_sizes == [0, 1, 1, 8]
    assert p.encoded_words.tolist() == [0, 0]
    with pytest.raises(ValueError):
        projections.anisotropic([5.0, 5.0], 1.0, 2, 2, device="cpu")
    with pytest.raises(ValueError):
        projections.anisotropic([1.0], 1.0, 2, 2, device="cpu")
    with pytest.raises(ValueError):
        projections.anisotropic([1.0, -1.0], 1.0, 2, 2, device="cpu")
    with pytest.raises(ValueError):
        projections.anisotropic([1.0, 1.0], 0.0, 2, 2, device="cpu")


# ---- modules and operators (no GPU: meta device and error paths) ----

def test_module_argument_checks_and_buffers():
    with pytest.raises(ValueError):
        ps.Signature(depth=0)
    with pytest.raises(ValueError):
        ps.LogSignature(depth=13)
    with pytest.raises(TypeError):
        ps.Signature(depth=2, windows=torch.zeros(2, 2, dtype=torch.int32))   # not a CUDA tensor
    with pytest.raises(TypeError):
        ps.Signature(depth=2, projection=projections.lyndon(2, 2, device="cpu"))
    m = ps.Signature(depth=3)
    assert set(dict(m.named_buffers())) == {"_windows", "_encoded_words"}
    assert m.state_dict() == {}                                               # unused buffers are not persistent
    lm = ps.LogSignature(depth=3)
    assert set(dict(lm.named_buffers())) == {"_windows", "_encoded_words", "_top_words", "_indices_from_sig"}


def test_fake_operators_give_reference_shapes():
    x = torch.empty(32, 128, 8, device="meta")
    ew = torch.empty(0, dtype=torch.int64, device="meta")
    win = torch.empty((63, 2), dtype=torch.int32, device="meta")
    nowin = torch.empty((0, 2), dtype=torch.int32, device="meta")
    sig = ps.ops.compute_signature(x, 4, False, ew, [], False, nowin)
    assert sig.shape == (32, 4680)
    assert ps.ops.compute_signature(x, 4, False, ew, [], True, win).shape == (32, 63, 4680)
    words = torch.empty(200, dtype=torch.int64, device="meta")
    assert ps.ops.compute_signature(x, 3, True, words, [0, 8, 100, 100], False, nowin).shape == (32, 208)
    logsig, cache = ps.ops.sig_to_logsig(sig, 4, 8, False, ew, [0, 8, 64, 512, 4096])
    # the cache is empty when the row-in-shared-memory kernels serve the shape, the reference's table of
    # powers (S * depth per row) otherwise
    assert logsig.shape == (32, 4680) and cache.shape == (32, 0)
    big = torch.empty(2, 16 + 16 ** 2 + 16 ** 3 + 16 ** 4 + 16 ** 5, device="meta")
    _, big_cache = ps.ops.sig_to_logsig(big, 5, 16, False, ew, [0] + [16 ** k for k in range(1, 6)])
    assert big_cache.shape == (2, 5 * big.shape[1])
    assert ps.ops.signature_backward(x, sig, sig, 4, False, ew, [], False, nowin).shape == x.shape
    assert ps.ops.logsig_backward(sig, cache, sig, 4, False, ew, [0, 8, 64, 512, 4096]).shape == sig.shape
    with pytest.raises(RuntimeError):
        ps.ops.compute_signature(torch.empty(2, 1, 3, device="meta"), 2, False, ew, [], False, nowin)
    # Chen product and its adjoint keep the shape of their operands
    a = torch.empty(5, 7, 4680, device="meta")
    assert ps.ops.chen_product(a, a, 4, 8).shape == a.shape
    ga, gb = ps.ops.chen_product_backward(a, a, a, 4, 8)
    assert ga.shape == a.shape and gb.shape == a.shape


def test_cpu_tensors_are_refused():
    with pytest.raises(NotImplementedError):
        ps.ops.compute_signature(torch.zeros(2, 4, 3), 2, False, torch.empty(0, dtype=torch.int64), [], False,
                                 torch.empty((0, 2), dtype=torch.int32))


def test_install_as_pathsig_aliases_the_package():
    ps.install_as_pathsig()
    import pathsig
    assert pathsig.Signature is ps.Signature and pathsig.projections is ps.projections
    assert torch.ops.pathsig.compute_signature is not None


def test_operators_are_registered_by_the_compiled_library():
    """The eight operators come from libpathsig_b200_torch.so (TORCH_LIBRARY + TORCH_LIBRARY_IMPL for the
    CUDA key, like the reference's bindings.cpp and launchers); Python adds the fake implementations and
    the autograd formulas.  There is no CPU kernel: CPU tensors are refused by the dispatcher."""
    from pathsig_b200 import _load, ops
    binding = _load.ensure_binding_loaded()
    assert binding.psig_torch_get_algorithm() == _load.ALGO_AUTO
    for name, schema in ops._SCHEMAS.items():
        op = getattr(torch.ops.pathsig_b200, name).default
        assert str(op._schema) == f"pathsig_b200::{name}{schema}"
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"pathsig_b200::{name}", "CUDA")
        assert not torch._C._dispatch_has_kernel_for_dispatch_key(f"pathsig_b200::{name}", "CPU")
        assert torch.Tag.pt2_compliant_tag in op.tags
    ops.set_algorithm("generic")
    try:
        assert binding.psig_torch_get_algorithm() == _load.ALGO_GENERIC
    finally:
        ops.set_algorithm("auto")
    with pytest.raises(NotImplementedError):
        ops.chen_product(torch.zeros(2, 6), torch.zeros(2, 6), 2, 2)


def test_word_codes_are_range_checked_on_the_host():
    from pathsig_b200 import modules
    # d = 3, depth 3: degree 1 complete, two words at degree 2, one at degree 3
    modules._check_codes([0, 8, 26], [0, 3, 2, 1], 3, 3)
    with pytest.raises(ValueError, match=r"outside \[0, 3\*\*2\)"):
        modules._check_codes([0, 9, 26], [0, 3, 2, 1], 3, 3)
    with pytest.raises(ValueError, match=r"outside \[0, 3\*\*3\)"):
        modules._check_codes([0, 8, 27], [0, 3, 2, 1], 3, 3)
    with pytest.raises(ValueError, match="fewer than level_sizes requires"):
        modules._check_codes([0, 8], [0, 3, 2, 1], 3, 3)
    # the projections keep a host copy of their codes, so module construction reads nothing back
    proj = ps.projections.words([(0, 1), (2, 2), (1, 0, 2)], 3, 3, full_levels=(1,), device="cpu")
    assert proj._host_codes == proj.encoded_words.tolist() == [1, 8, 11]


def _closure_desc(codes, level_sizes, d, depth):
    from pathsig_b200 import _load
    desc = _load.SigDesc()
    desc.dtype, desc.d, desc.depth, desc.B, desc.L, desc.projected = _load.PSIG_F32, d, depth, 64, 16, 1
    for k in range(1, depth + 1):
        desc.level_sizes[k] = level_sizes[k]
    host = torch.tensor(codes, dtype=torch.int64)
    desc.words_host = host.data_ptr()
    desc.words = host.data_ptr()  # only offsets of it are formed on the host
    return desc, host


def test_closure_generator_counts_and_compiles_for_sm100a():
    """The code generator of the prefix-closure kernels: its closure of the config-3 word set has the
    algorithmic FMA count the benchmark credits, and the generated CUDA compiles for sm_100a with NVRTC
    (no device needed)."""
    import ctypes

    import bench
    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    wl = bench.Workload("cfg3")
    proj = ps.projections.words([w for w in wl.words if len(w) > 1], 6, 8, full_levels=(1,), device="cpu")
    desc, keep = _closure_desc(proj.encoded_words.tolist(), proj.level_sizes, 8, 6)
    stats = (ctypes.c_int64 * 5)()
    n = lib.psig_closure_source(ctypes.byref(desc), 16, None, 0, stats)
    assert n > 0
    nodes, algorithmic, executed, bins, per_lane = list(stats)
    assert algorithmic == wl.fma_fwd            # one FMA per (closure node, target degree) pair
    assert algorithmic <= executed <= 2 * algorithmic
    assert 1 <= bins <= 16 and per_lane <= 64 and nodes >= 208
    # a small word set, compiled
    small = ps.projections.words([(0, 1), (2, 2), (1, 0, 2), (1, 0, 0)], 3, 3, full_levels=(1,), device="cpu")
    desc, keep = _closure_desc(small.encoded_words.tolist(), small.level_sizes, 3, 3)
    n = lib.psig_closure_source(ctypes.byref(desc), 2, None, 0, stats)
    buf = ctypes.create_string_buffer(n + 1)
    assert lib.psig_closure_source(ctypes.byref(desc), 2, buf, n + 1, stats) == n
    assert b"closure_forward" in buf.value and b"closure_backward" in buf.value
    log = ctypes.create_string_buffer(1 << 14)
    rc = lib.psig_closure_compile(buf.value, b"sm_100a", log, 1 << 14)
    assert rc == 0, log.value.decode()
    # a word listed twice has no unique column: the plan is refused
    desc, keep = _closure_desc([1, 1], [0, 3, 2, 0], 3, 3)
    assert lib.psig_closure_source(ctypes.byref(desc), 2, None, 0, stats) < 0


def test_compiled_closure_kernels_are_kept_on_disk(tmp_path, monkeypatch):
    """A cubin compiled once is read back by the next compilation of the same source and options
    (another process, typically) from the cache directory."""
    import ctypes

    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    monkeypatch.setenv("PATHSIG_B200_CACHE_DIR", str(tmp_path / "kernels"))
    small = ps.projections.words([(0, 1), (1, 1, 0)], 3, 2, full_levels=(1,), device="cpu")
    desc, keep = _closure_desc(small.encoded_words.tolist(), small.level_sizes, 2, 3)
    stats = (ctypes.c_int64 * 5)()
    n = lib.psig_closure_source(ctypes.byref(desc), 1, None, 0, stats)
    buf = ctypes.create_string_buffer(n + 1)
    lib.psig_closure_source(ctypes.byref(desc), 1, buf, n + 1, stats)
    log = ctypes.create_string_buffer(1 << 14)
    assert lib.psig_closure_compile(buf.value, b"sm_100a", log, 1 << 14) == 0
    assert b"read from" not in log.value
    assert len(list((tmp_path / "kernels").glob("closure_*.cubin"))) == 2     # forward and backward pass
    assert lib.psig_closure_compile(buf.value, b"sm_100a", log, 1 << 14) == 0
    assert log.value.count(b"read from") == 2


def test_top_plan_orders_owners_of_listed_words_first():
    """Projected top degree on the tiled kernels: the launcher's order of a unit's work items puts the
    threads that own a listed word first and lets whole warps of the others skip the top degree.  For the
    Lyndon words of length 6 over 4 letters, 29 of the 64 prefixes of length 3 start a Lyndon word (a
    Lyndon word's first letter is its smallest), so one of the two warps skips."""
    import ctypes

    from pathsig_b200 import _load
    lib = _load.ensure_loaded()
    proj = ps.projections.lyndon(6, 4, device="cpu")
    sizes = list(proj.level_sizes)
    top = proj.encoded_words[-sizes[6]:].tolist()
    ext = [0] + [4 ** k for k in range(1, 6)] + [len(top)]
    desc, keep = _closure_desc(top, ext, 4, 6)
    items = (ctypes.c_ubyte * 256)()
    active = ctypes.c_int(0)
    for backward in (0, 1):
        nt = lib.psig_tiled_top_plan(ctypes.byref(desc), backward, items, ctypes.byref(active))
        assert nt == 64 and active.value == 32
        order = list(items)[:64]
        assert sorted(order) == list(range(64))                        # a permutation of the unit's items
        owners = sorted({code // 64 for code in top})                   # prefixes of length 3 with a listed word
        assert len(owners) == 29 and order[:29] == owners               # owners first, in their own order
        assert all(min(u // 16, (u // 4) % 4, u % 4) == u // 16 for u in owners)
    # without a host copy of the list nothing is reordered and nothing is skipped
    desc.words_host = None
    assert lib.psig_tiled_top_plan(ctypes.byref(desc), 0, items, ctypes.byref(active)) == 64
    assert active.value >= 64 and list(items)[:64] == list(range(64))
    # every prefix owns a word: nothing to skip either
    dense_top = list(range(0, 4 ** 6, 7))
    desc, keep = _closure_desc(dense_top, [0] + [4 ** k for k in range(1, 6)] + [len(dense_top)], 4, 6)
    assert lib.psig_tiled_top_plan(ctypes.byref(desc), 1, items, ctypes.byref(active)) == 64
    assert active.value >= 64
    # a shape whose unit spans several blocks has no projected-top path on the tiled kernels
    desc, keep = _closure_desc([1, 2, 3], [0, 16, 256, 4096, 3], 16, 4)
    assert lib.psig_tiled_top_plan(ctypes.byref(desc), 0, items, ctypes.byref(active)) < 0


def test_prefix_closure_of_a_word_set():
    """The closed word set ``Signature`` evaluates large projections on: every prefix of a requested word,
    complete degrees below a complete degree, columns of the requested row inside the closed row."""
    from pathsig_b200.modules import _prefix_closure
    # d = 3: degree 1 complete, (0,1) at degree 2, (1,0,0) and (1,0,2) at degree 3
    closed = _prefix_closure([1, 9, 11], [0, 3, 1, 2], 3, 3)
    assert closed == ([1, 3, 9, 11], [0, 3, 2, 2], [0, 1, 2, 3, 5, 6])
    assert _prefix_closure([1, 3, 9, 11], [0, 3, 2, 2], 3, 3) is None          # already closed
    assert _prefix_closure([9, 9], [0, 3, 9, 2], 3, 3) is None                  # a word listed twice
    # a complete degree above an incomplete one makes everything below complete
    codes, sizes, cols = _prefix_closure([1], [0, 1, 9], 3, 2)
    assert sizes == [0, 3, 9] and codes == [] and cols == [1] + list(range(3, 12))
    # no degree-1 word requested at all: its prefixes appear, the requested columns move behind them
    codes, sizes, cols = _prefix_closure([5, 7], [0, 0, 2], 3, 2)
    assert sizes == [0, 2, 2] and codes == [1, 2, 5, 7] and cols == [2, 3]
    # the benchmark's word list: 482 words in the closed set, as the kernel generator counts
    import bench
    wl = bench.Workload("cfg3")
    proj = ps.projections.words([w for w in wl.words if len(w) > 1], 6, 8, full_levels=(1,), device="cpu")
    codes, sizes, cols = _prefix_closure(proj.encoded_words.tolist(), list(proj.level_sizes), 8, 6)
    assert sum(sizes) == 482 and len(cols) == 208 and len(set(cols)) == 208 and cols == sorted(cols)
