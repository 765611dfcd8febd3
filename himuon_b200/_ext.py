"""Loader for the prebuilt sm_100a extension.

``ext()`` returns the compiled module or raises with a clear message; it never falls back to
another implementation on a GPU machine.  CPU-only machines (the unit-test tier) use the
pure-PyTorch reference ops and never call this.
"""

from __future__ import annotations

import importlib.util
import os

from ._build import EXT_NAME, so_path

_EXT = None
_ERR: Exception | None = None


def ext():
    global _EXT, _ERR
    if _EXT is not None:
        return _EXT
    if _ERR is not None:
        raise RuntimeError(f"himuon_b200: the CUDA extension failed to load earlier: {_ERR}")
    path = so_path()
    try:
        if not os.path.exists(path):
            raise FileNotFoundError(
                f"{path} is missing - run `python -c 'import __graft_entry__ as g; g.build()'` "
                "(or `python -m himuon_b200._build`) to compile it for sm_100a"
            )
        import torch  # noqa: F401  (libtorch symbols must be loaded first)

        spec = importlib.util.spec_from_file_location(EXT_NAME, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _EXT = mod
        return mod
    except Exception as e:  # pragma: no cover - depends on the machine
        _ERR = e
        raise RuntimeError(f"himuon_b200: cannot load the CUDA extension: {e}") from e


def available() -> bool:
    try:
        ext()
        return True
    except Exception:
        return False
