"""``himuon`` - the reference's import name, served by :mod:`himuon_b200`.

``from himuon.optimizers import HiMuon``, ``from himuon.optim import get_optimizer``,
``from himuon.fsdp_bank import wrap_with_banks``, ``from himuon.triton_kernels import XXT`` and the other import
lines of code written against the reference (``src/himuon/``) resolve to this library's modules; ``triton_kernels``
maps to :mod:`himuon_b200.kernels` (the callables are tcgen05 kernels here, the name is kept for compatibility).
"""

import importlib as _importlib
import sys as _sys

import himuon_b200 as _impl

__version__ = _impl.__version__

_RENAMED = {"triton_kernels": "kernels"}
for _name in ("optim", "optimizers", "fsdp_bank", "model", "dataset", "logger", "utils", "models", "ops", "parallel",
              "trainer", "kernels", "triton_kernels"):
    _mod = _importlib.import_module("himuon_b200." + _RENAMED.get(_name, _name))
    _sys.modules[__name__ + "." + _name] = _mod
    globals()[_name] = _mod
# sub-modules that the imports above pulled in (himuon.optimizers.himuon, himuon.fsdp_bank.wrap, ...)
for _key, _mod in list(_sys.modules.items()):
    if _key.startswith("himuon_b200.") and _mod is not None:
        _sys.modules.setdefault(__name__ + _key[len("himuon_b200"):], _mod)
