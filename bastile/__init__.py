"""``import bastile`` for code written against aghilann/bastile.

The implementation lives in :mod:`bastile_b200`; this package only gives it the
reference's import name (src/bastile/__init__.py:18-33), so that
``import bastile; bastile.apply()`` and ``from bastile.ops.rms_norm import rms_norm``
run unchanged.  Every ``bastile.<sub>`` module IS the ``bastile_b200.<sub>`` module
(one registry, one set of patches), not a copy.
"""

import importlib as _importlib
import sys as _sys

import bastile_b200 as _impl
from bastile_b200 import *  # noqa: F401,F403
from bastile_b200 import __all__, __version__  # noqa: F401

for _name in ("autotune", "core", "registry", "ops", "ops.utils", "ops.rms_norm", "ops.rope", "ops.swiglu",
              "ops.fused_linear_cross_entropy"):
    _mod = _importlib.import_module("bastile_b200." + _name)
    _sys.modules[__name__ + "." + _name] = _mod
    if "." not in _name:
        globals()[_name] = _mod
del _name, _mod
