"""Compile the reference's own CUDA operators, unchanged, into ``oracle/_ref/libpathsig_ops.so``.

TEST INFRASTRUCTURE ONLY.  The reference has no CPU implementation, so its CUDA build is the
strongest parity pin there is: the GPU tests load this library next to ours (its operators
live in ``torch.ops.pathsig``, ours in ``torch.ops.pathsig_b200``) and compare outputs on the
same tensors, and ``tests/golden/make_golden.py`` records its outputs as fixtures.

The sources are compiled where they lie (the checkout named by the ``root`` argument or by
``$PATHSIG_REFERENCE_ROOT``) with plain nvcc commands; the reference's own CMake build is not run and
no source file enters the repository.  Outputs go to ``oracle/_ref/`` only, which git ignores.  When no
reference tree is given or found (for example on a GPU box) the function leaves an existing library
alone and reports whether one is there.

The same step stages the two acceptance files of the reference's test-suite that need nothing but the
public ``pathsig`` API (``tests/test_windows.py``, ``tests/test_projections.py``), byte for byte, under
``oracle/_ref/reference_tests/`` with their SHA-256 in ``PROVENANCE.txt``, so that the GPU tests can run
them unmodified against this package (``tests/test_gpu_reference_suites.py``).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libpathsig_ops.so")
SOURCES = [
    "src/pathsig/bindings.cpp",
    "src/pathsig/forward/sig_launch.cu",
    "src/pathsig/forward/sig_kernels.cu",
    "src/pathsig/backward/sig_backward_launch.cu",
    "src/pathsig/backward/sig_backward_kernels.cu",
]


TESTS_DIR = os.path.join(OUT_DIR, "reference_tests")
ACCEPTANCE_TESTS = ["tests/test_windows.py", "tests/test_projections.py"]


def reference_root(root: Optional[str] = None) -> Optional[str]:
    """The reference checkout to build from: the argument, else ``$PATHSIG_REFERENCE_ROOT``, else none."""
    return root or os.environ.get("PATHSIG_REFERENCE_ROOT") or None


def stage_acceptance_tests(root: str) -> None:
    """Copy the reference's API-only test files, unmodified, next to the built library."""
    files = [os.path.join(root, t) for t in ACCEPTANCE_TESTS]
    if not all(os.path.isfile(f) for f in files):
        return
    os.makedirs(TESTS_DIR, exist_ok=True)
    lines = ["Unmodified copies of files of the reference's test-suite (tobiasny12/pathsig v0.1.7), staged by",
             "oracle/build_ref.py for tests/test_gpu_reference_suites.py.  sha256  path-in-the-reference", ""]
    for rel, src in zip(ACCEPTANCE_TESTS, files):
        shutil.copyfile(src, os.path.join(TESTS_DIR, os.path.basename(rel)))
        with open(src, "rb") as fh:
            lines.append(f"{hashlib.sha256(fh.read()).hexdigest()}  {rel}")
    with open(os.path.join(TESTS_DIR, "PROVENANCE.txt"), "w") as fh:
        fh.write("\n".join(lines) + "\n")


def build(force: bool = False, verbose: bool = False, root: Optional[str] = None) -> bool:
    """Returns True when ``oracle/_ref/libpathsig_ops.so`` exists afterwards."""
    root = reference_root(root)
    if root is None:
        return os.path.isfile(LIB)
    srcs = [os.path.join(root, s) for s in SOURCES]
    if not all(os.path.isfile(s) for s in srcs):
        return os.path.isfile(LIB)
    stage_acceptance_tests(root)
    if os.path.isfile(LIB) and not force:
        newest = max(os.path.getmtime(s) for s in srcs)
        if os.path.getmtime(LIB) >= newest:
            return True

    import torch
    from torch.utils import cpp_extension

    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    includes = [os.path.join(root, "src", "pathsig")] + cpp_extension.include_paths("cuda")
    flags = [
        "-gencode", "arch=compute_100,code=sm_100", "-ccbin", "/usr/bin/g++", "-std=c++17", "-O3", "-DNDEBUG",
        "-rdc=true", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch.compiled_with_cxx11_abi())}",
    ]
    for inc in includes:
        flags += ["-isystem" if "torch" in inc else "-I", inc]

    def compile_one(src: str) -> str:
        obj = os.path.join(OUT_DIR, os.path.basename(src).rsplit(".", 1)[0] + ".o")
        cmd = [nvcc] + flags + ["-x", "cu", "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"reference build failed for {src}:\n{res.stderr[-4000:]}")
        if verbose:
            print("compiled", src, file=sys.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as pool:
        objs = list(pool.map(compile_one, srcs))

    lib_dirs = cpp_extension.library_paths("cuda")
    link = [nvcc, "-gencode", "arch=compute_100,code=sm_100", "-ccbin", "/usr/bin/g++", "-shared", "-o", LIB] + objs
    for ld in lib_dirs:
        link += ["-L", ld, "-Xlinker", f"-rpath={ld}"]
    link += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"reference link failed:\n{res.stderr[-4000:]}")
    for o in objs:
        os.remove(o)
    return True


if __name__ == "__main__":
    positional = [a for a in sys.argv[1:] if not a.startswith("--")]
    ok = build(force="--force" in sys.argv, verbose=True, root=positional[0] if positional else None)
    print("reference library:", LIB if ok else "unavailable")
