"""Importable alias of the ``iree-turbine_b200`` package directory (hyphens cannot be imported)."""

import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "iree-turbine_b200")
__path__ = [_real]
__file__ = _os.path.join(_real, "__init__.py")
with open(__file__, "rb") as _f:
    exec(compile(_f.read(), __file__, "exec"))
