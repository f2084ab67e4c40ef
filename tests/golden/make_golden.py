"""Records golden vectors from the reference's own CUDA operators.

Run on a machine with a CUDA GPU after ``python oracle/build_ref.py`` has produced
``oracle/_ref/libpathsig_ops.so`` (the reference's unchanged sources compiled with nvcc):

    python tests/golden/make_golden.py

which rewrites ``tests/golden/golden_reference.pt``.  Each case stores its inputs, the
operator arguments and the reference's outputs, so the consumers (tests/test_golden.py) need
neither the reference nor a GPU.  Only ``torch.ops.pathsig.*`` of the reference library is
called here; projections are described by explicit code lists.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests import util  # noqa: E402


def lyndon_codes(d, n):
    from pathsig_b200.projections import lyndon_words
    return lyndon_words(d, n)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "golden", "golden_reference.pt"))
    args = ap.parse_args()
    ref = util.reference_ops()
    if ref is None:
        raise SystemExit("oracle/_ref/libpathsig_ops.so is missing: run python oracle/build_ref.py first")
    dev = "cuda"
    no_words = torch.empty(0, dtype=torch.int64, device=dev)
    no_win = torch.empty((0, 2), dtype=torch.int32, device=dev)
    cases = {}

    def sig_case(name, x, depth, words=None, level_sizes=None, windows=None, seed=0):
        alt = level_sizes is not None
        ew = no_words if words is None else torch.tensor(words, dtype=torch.int64, device=dev)
        ls = list(level_sizes) if alt else []
        use_w = windows is not None
        win = no_win if windows is None else windows.to(dev)
        xg = x.to(dev)
        sig = ref.compute_signature(xg, depth, alt, ew, ls, use_w, win)
        g = util.normal_like(sig.shape, seed + 100, x.dtype).to(dev)
        grad = ref.signature_backward(xg, sig, g, depth, alt, ew, ls, use_w, win)
        cases[name] = dict(kind="sig", path=x.cpu(), depth=depth, words=ew.cpu(), level_sizes=ls,
                           windows=None if windows is None else windows.cpu(), sig=sig.cpu(), grad_sig=g.cpu(),
                           grad_path=grad.cpu())

    def log_case(name, x, depth, top_words=None, top_size=None, seed=0):
        d = x.shape[-1]
        alt = top_words is not None
        ew = no_words if not alt else torch.tensor(top_words, dtype=torch.int64, device=dev)
        ls = [0] + [d ** k for k in range(1, depth)] + [top_size if alt else d ** depth]
        xg = x.to(dev)
        sig = ref.compute_signature(xg, depth, alt, ew, ls if alt else [], False, no_win)
        logsig, cache = ref.sig_to_logsig(sig, depth, d, alt, ew, ls)
        g = util.normal_like(logsig.shape, seed + 200, x.dtype).to(dev)
        grad_sig = ref.logsig_backward(sig, cache, g, depth, alt, ew, ls)
        grad_path = ref.signature_backward(xg, sig, grad_sig, depth, alt, ew, ls if alt else [], False, no_win)
        cases[name] = dict(kind="log", path=x.cpu(), depth=depth, top_words=ew.cpu(), level_sizes=ls, alt=alt,
                           sig=sig.cpu(), logsig=logsig.cpu(), grad_logsig=g.cpu(), grad_sig=grad_sig.cpu(),
                           grad_path=grad_path.cpu())

    f32, f64 = torch.float32, torch.float64
    sig_case("dense_d3_n4_f64", util.brownian_path(2, 12, 3, 1, f64), 4)
    sig_case("dense_d8_n4_f64", util.brownian_path(2, 16, 8, 2, f64), 4)
    sig_case("dense_d8_n4_f32", util.brownian_path(2, 16, 8, 2, f32), 4)
    sig_case("dense_d2_n8_f64", util.brownian_path(1, 9, 2, 3, f64), 8)
    sig_case("dense_d16_n3_f32", util.brownian_path(1, 20, 16, 4, f32), 3)
    sig_case("windows_d3_n3_f64", util.brownian_path(2, 20, 3, 5, f64), 3,
             windows=torch.tensor([[0, 20], [3, 9], [8, 10], [5, 18]], dtype=torch.int32))
    # words projection: degree 1 complete, explicit words at degrees 2..4 (d = 3)
    words = [(0, 1), (2, 2), (1, 0), (0, 1, 2), (2, 0, 0), (1, 1, 1, 0), (0, 2, 1, 2)]
    codes = [sum(a * 3 ** (len(w) - 1 - i) for i, a in enumerate(w)) for w in words]
    sig_case("words_d3_n4_f64", util.brownian_path(2, 10, 3, 6, f64), 4, words=codes, level_sizes=[0, 3, 3, 2, 2])
    # Lyndon projection of the signature (d = 3, depth 4)
    lyn = [lyndon_codes(3, n) for n in range(2, 5)]
    sig_case("lyndon_d3_n4_f64", util.brownian_path(2, 10, 3, 7, f64), 4, words=sum(lyn, []),
             level_sizes=[0, 3] + [len(c) for c in lyn])
    log_case("log_dense_d3_n4_f64", util.brownian_path(2, 10, 3, 8, f64), 4)
    log_case("log_lyndon_d3_n4_f64", util.brownian_path(2, 10, 3, 9, f64), 4, top_words=lyn[-1], top_size=len(lyn[-1]))
    log_case("log_lyndon_d4_n5_f32", util.brownian_path(2, 14, 4, 10, f32), 5, top_words=lyndon_codes(4, 5),
             top_size=len(lyndon_codes(4, 5)))

    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    meta = dict(torch=str(torch.__version__), device=torch.cuda.get_device_name(0),
                source="reference CUDA operators (torch.ops.pathsig) compiled unchanged by oracle/build_ref.py")
    torch.save(dict(meta=meta, cases=cases), args.out)
    print("wrote", args.out, "with", len(cases), "cases")


if __name__ == "__main__":
    main()
