"""pathsig_b200 — truncated path signatures and log-signatures on NVIDIA B200 (sm_100a).

Same public surface as the reference package (``src/pathsig/__init__.py:1-8``):
``Signature``, ``LogSignature`` and the ``projections`` namespace.  Importing the package
loads the CUDA library and the compiled operator registration; it fails loudly when either has
not been built.  :func:`install_as_pathsig` additionally exposes the package under the name
``pathsig`` for code written against the reference.
"""
from ._load import ensure_loaded as _ensure_loaded

_ensure_loaded()

from . import ops  # noqa: E402  (registers torch.ops.pathsig_b200.*)
from .modules import LogSignature, Signature  # noqa: E402
from .projections import projections  # noqa: E402

__all__ = ["Signature", "LogSignature", "projections", "chen_product", "install_as_pathsig"]
__version__ = "0.1.0"


def chen_product(sig_a, sig_b, *, path_dim: int, depth: int):
    """Signature of two paths run one after the other, from their signatures (Chen's identity).

    ``sig_a`` and ``sig_b`` are dense signatures ``(..., D)`` as :class:`Signature` returns them
    without a projection (``D = path_dim + ... + path_dim**depth``); the result has the same shape and
    is differentiable wrt both.  ``chen_product(S(x[:, :m+1]), S(x[:, m:]))`` equals ``S(x)``.  The
    reference package has no counterpart; signatures of adjoining or growing pieces of a path can be
    combined with it instead of being recomputed from the points.
    """
    if not isinstance(path_dim, int) or path_dim < 1:
        raise ValueError("path_dim must be a positive integer")
    if not isinstance(depth, int) or not (1 <= depth <= 12):
        raise ValueError("depth must be an integer in [1, 12]")
    return ops.chen_product(sig_a, sig_b, depth, path_dim)


def install_as_pathsig(register_ops: bool = True) -> None:
    """Make ``import pathsig`` resolve to this package.

    With ``register_ops`` the four operators are also defined under ``torch.ops.pathsig``; that
    part is skipped when a build of the reference already owns the namespace in this process.
    """
    import sys

    module = sys.modules[__name__]
    sys.modules.setdefault("pathsig", module)
    for sub in ("ops", "modules", "projections", "_load"):
        sys.modules.setdefault("pathsig." + sub, sys.modules[__name__ + "." + sub])
    if register_ops:
        import torch

        try:
            already = torch._C._dispatch_has_kernel("pathsig::compute_signature")
        except Exception:
            already = False
        if not already:
            ops.register_namespace("pathsig")
