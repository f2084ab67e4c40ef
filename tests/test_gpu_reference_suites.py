"""The reference's own acceptance files, unmodified, against this package.

``tests/test_windows.py`` and ``tests/test_projections.py`` of the reference use nothing but the public
``pathsig`` API (modules, projections, autograd, ``gradcheck``).  ``oracle/build_ref.py`` stages byte-for-
byte copies under ``oracle/_ref/reference_tests/`` (git-ignored; the SHA-256 of each file is recorded
beside them).  Each file runs under pytest in a child process in which ``pathsig`` is this package
(``pathsig_b200.install_as_pathsig()``); the child must collect the expected number of tests and pass all
of them.  Skipped when the staged files are absent.
"""
from __future__ import annotations

import hashlib
import os
import re
import subprocess
import sys

import pytest

from . import util

pytestmark = pytest.mark.gpu
STAGED = os.path.join(util.ROOT, "oracle", "_ref", "reference_tests")


def _recorded_digest(name: str) -> str:
    with open(os.path.join(STAGED, "PROVENANCE.txt")) as fh:
        for line in fh:
            parts = line.split()
            if len(parts) == 2 and parts[1].endswith("/" + name):
                return parts[0]
    raise AssertionError(f"no digest recorded for {name}")


@pytest.mark.parametrize("name,at_least", [("test_windows.py", 91), ("test_projections.py", 161)])
def test_reference_suite_passes_unmodified(name, at_least):
    path = os.path.join(STAGED, name)
    if not os.path.isfile(path):
        pytest.skip("reference test files not staged (oracle/build_ref.py has not seen a reference checkout)")
    with open(path, "rb") as fh:
        assert hashlib.sha256(fh.read()).hexdigest() == _recorded_digest(name), "staged file was modified"
    env = dict(os.environ, PYTHONPATH=util.ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    res = subprocess.run(
        [sys.executable, "-m", "pytest", "-q", "-p", "tests.pathsig_alias_plugin", "-p", "no:cacheprovider", path],
        cwd=util.ROOT, env=env, capture_output=True, text=True, timeout=1500)
    tail = res.stdout[-3000:] + res.stderr[-2000:]
    assert res.returncode == 0, tail
    m = re.search(r"(\d+) passed", res.stdout)
    assert m and int(m.group(1)) >= at_least, tail
    assert "failed" not in res.stdout.splitlines()[-1] and "error" not in res.stdout.splitlines()[-1], tail
