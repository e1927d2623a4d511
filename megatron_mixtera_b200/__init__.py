"""Import alias for the package that lives in the ``megatron-mixtera_b200/`` directory.

A directory name with a hyphen cannot be imported directly, so this two-line package
points its search path at the real source tree and executes that tree's ``__init__``.
"""
import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "megatron-mixtera_b200")
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _os, _f
