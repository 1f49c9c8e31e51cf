"""Import shim: the package lives in the directory `hyperqwen-rtx4080s32_b200/`, whose name is not a
Python identifier.  This module gives it the importable name `hyperqwen_rtx4080s32_b200` by pointing
`__path__` at that directory and running its `__init__.py` here."""
import os as _os

__package__ = __name__
__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "hyperqwen-rtx4080s32_b200")]
_init = _os.path.join(__path__[0], "__init__.py")
with open(_init, "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), _init, "exec"))
del _os, _init, _f
