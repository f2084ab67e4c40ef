"""Loads ``libpathsig_b200.so`` (the CUDA library behind the C ABI of ``include/pathsig_b200.h``) and
``libpathsig_b200_torch.so`` (the operator registration with the PyTorch dispatcher on top of it).

Counterpart of the reference's loader (``src/pathsig/_load.py:12-45``): one lock-guarded load
per process, a clear error when a native library is missing.  There is no CPU or PyTorch
fallback: without the libraries every operator raises.
"""
from __future__ import annotations

import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libpathsig_b200.so"
LIB_PATH = os.path.join(_HERE, LIB_NAME)
BINDING_NAME = "libpathsig_b200_torch.so"
BINDING_PATH = os.path.join(_HERE, BINDING_NAME)
MAX_DEPTH = 12
ABI_VERSION = 2

PSIG_F32, PSIG_F64 = 0, 1
ALGO_AUTO, ALGO_GENERIC, ALGO_TILED, ALGO_CLOSURE = 0, 1, 2, 3
FLAG_DETERMINISTIC = 1   # PSIG_FLAG_DETERMINISTIC of include/pathsig_b200.h

_lock = threading.Lock()
_lib = None
_binding = None


class SigDesc(ctypes.Structure):
    """``PsigSigDesc`` of include/pathsig_b200.h."""
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("d", ctypes.c_int32),
        ("depth", ctypes.c_int32),
        ("projected", ctypes.c_int32),
        ("B", ctypes.c_int64),
        ("L", ctypes.c_int64),
        ("W", ctypes.c_int64),
        ("windows", ctypes.c_void_p),
        ("words", ctypes.c_void_p),
        ("level_sizes", ctypes.c_int64 * (MAX_DEPTH + 1)),
        ("algo", ctypes.c_int32),
        ("flags", ctypes.c_int32),
        ("words_host", ctypes.c_void_p),
    ]


class LogDesc(ctypes.Structure):
    """``PsigLogDesc`` of include/pathsig_b200.h."""
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("d", ctypes.c_int32),
        ("depth", ctypes.c_int32),
        ("algo", ctypes.c_int32),
        ("rows", ctypes.c_int64),
        ("top_size", ctypes.c_int64),
        ("top_words", ctypes.c_void_p),
        ("lower_columns", ctypes.c_void_p),
        ("n_lower_columns", ctypes.c_int64),
    ]


class ChenDesc(ctypes.Structure):
    """``PsigChenDesc`` of include/pathsig_b200.h."""
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("d", ctypes.c_int32),
        ("depth", ctypes.c_int32),
        ("reserved", ctypes.c_int32),
        ("rows", ctypes.c_int64),
    ]


# name -> (restype, argtypes); every symbol include/pathsig_b200.h declares.
_vp, _i64, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
_SigP, _LogP, _ChenP = ctypes.POINTER(SigDesc), ctypes.POINTER(LogDesc), ctypes.POINTER(ChenDesc)
EXPORTS = {
    "psig_abi_version": (_int, []),
    "psig_status_string": (ctypes.c_char_p, [_int]),
    "psig_sig_size": (_i64, [_SigP]),
    "psig_logsig_size": (_i64, [_LogP]),
    "psig_logsig_out_size": (_i64, [_LogP]),
    "psig_sig_forward": (_int, [_SigP, _vp, _vp, _vp]),
    "psig_sig_backward_workspace": (_i64, [_SigP]),
    "psig_sig_backward": (_int, [_SigP, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "psig_sig_backward_reproducible": (_int, [_SigP]),
    "psig_logsig_cache_size": (_i64, [_LogP]),
    "psig_logsig_forward": (_int, [_LogP, _vp, _vp, _vp, _vp]),
    "psig_logsig_backward_workspace": (_i64, [_LogP]),
    "psig_logsig_backward": (_int, [_LogP, _vp, _vp, _vp, _vp, _vp, _i64, _vp]),
    "psig_kernel_launches": (_i64, []),
    "psig_bulk_copy_timeouts": (_i64, []),
    "psig_set_bulk_wait_polls": (_int, [_int]),
    "psig_tiled_top_plan": (_int, [_SigP, _int, ctypes.POINTER(ctypes.c_ubyte), ctypes.POINTER(_int)]),
    "psig_closure_source": (_i64, [_SigP, _int, ctypes.c_char_p, _i64, ctypes.POINTER(ctypes.c_int64)]),
    "psig_closure_compile": (_int, [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_char_p, _i64]),
    "psig_closure_available": (_int, []),
    "psig_sig_backward_static": (_int, [_SigP, _vp, _vp, _vp, _vp, _vp]),
    "psig_sig_backward_static_limit": (_i64, []),
    "psig_chen_size": (_i64, [_ChenP]),
    "psig_chen_forward": (_int, [_ChenP, _vp, _vp, _vp, _vp]),
    "psig_chen_backward": (_int, [_ChenP, _vp, _vp, _vp, _vp, _vp, _vp]),
}


def ensure_loaded() -> ctypes.CDLL:
    """Load the native library once; raise ``RuntimeError`` when it is absent or stale."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"pathsig_b200: native library {LIB_PATH} not found. Build it with "
                "`python -c 'import __graft_entry__ as g; g.build()'` or `make -C pathsig_b200/csrc`. "
                "There is no CPU or PyTorch fallback."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        if lib.psig_abi_version() != ABI_VERSION:
            raise RuntimeError(f"pathsig_b200: {LIB_NAME} has ABI {lib.psig_abi_version()}, expected {ABI_VERSION}; rebuild it.")
        _lib = lib
    return _lib


def ensure_binding_loaded() -> ctypes.CDLL:
    """Load the compiled operator registration once (``torch.ops.pathsig_b200.*`` exist afterwards);
    returns a handle for its two plain-C controls."""
    global _binding
    if _binding is not None:
        return _binding
    ensure_loaded()
    with _lock:
        if _binding is not None:
            return _binding
        if not os.path.isfile(BINDING_PATH):
            raise RuntimeError(
                f"pathsig_b200: operator library {BINDING_PATH} not found. Build it with "
                "`python -c 'import __graft_entry__ as g; g.build()'` or `make -C pathsig_b200/csrc`. "
                "There is no Python fallback for the operators."
            )
        import torch
        torch.ops.load_library(BINDING_PATH)
        binding = ctypes.CDLL(BINDING_PATH)
        binding.psig_torch_set_algorithm.restype = None
        binding.psig_torch_set_algorithm.argtypes = [ctypes.c_int]
        binding.psig_torch_get_algorithm.restype = ctypes.c_int
        binding.psig_torch_get_algorithm.argtypes = []
        _binding = binding
    return _binding


def check(status: int, what: str) -> None:
    """Turn a negative PsigStatus into ``RuntimeError`` (mirrors TORCH_CHECK -> RuntimeError)."""
    if status < 0:
        msg = ensure_loaded().psig_status_string(int(status)).decode()
        raise RuntimeError(f"pathsig_b200::{what}: {msg} (status {status})")
