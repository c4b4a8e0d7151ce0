"""Loader of the in-tree sm_100a extension ``picotron_b200/_C*.so``.

The extension is built in-tree (``python setup.py build_ext --inplace`` or
``__graft_entry__.build()``); nothing is JIT-compiled at run time. On a machine with a CUDA device the
extension is mandatory: ops called with CUDA tensors raise if it cannot be imported, they never fall
back to eager PyTorch silently.
"""
from __future__ import annotations

import importlib

_C = None
_ERR = None


def load():
    """Import and return the extension module, or raise with the original import error."""
    global _C, _ERR
    if _C is not None:
        return _C
    if _ERR is None:
        try:
            import torch  # noqa: F401  (libtorch symbols must be loaded first)
            _C = importlib.import_module("picotron_b200._C")
            return _C
        except Exception as e:  # noqa: BLE001
            _ERR = e
    raise RuntimeError(
        "picotron_b200._C (the sm_100a CUDA extension) is not built or failed to load: "
        f"{_ERR!r}. Build it with `python setup.py build_ext --inplace` in the repository root.")


def available() -> bool:
    try:
        load()
        return True
    except RuntimeError:
        return False
