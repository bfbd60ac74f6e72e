"""Loader of the native extension ``fuselink_b200/_C.so``.

The extension is built in-tree by ``python -m fuselink_b200.build``.  On a machine with a GPU a missing or
unloadable extension is an error the first time a CUDA op is used: nothing silently falls back to PyTorch.
"""
from __future__ import annotations

import importlib

C = None
_import_error = None
try:  # pragma: no cover - depends on the build
    import torch  # noqa: F401 - the extension links libtorch: PyTorch has to be initialised before it is loaded
    C = importlib.import_module("fuselink_b200._C")
except Exception as e:  # noqa: BLE001
    _import_error = e


def have_native() -> bool:
    return C is not None


def require_native():
    """Return the extension module or raise with the reason it could not be loaded."""
    if C is None:
        raise RuntimeError(
            "fuselink_b200._C is not available; build it with `python -m fuselink_b200.build` "
            f"(import error: {_import_error!r})"
        )
    return C
