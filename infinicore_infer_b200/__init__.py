"""Import name of the framework.

The source tree lives in the sibling folder ``infinicore-infer_b200/`` (a name
that Python cannot import because of the hyphen).  This package points its
search path at that folder and runs its ``__init__``, so that
``import infinicore_infer_b200.config`` resolves to
``infinicore-infer_b200/config``.
"""
import os as _os

_SRC = _os.path.join(
    _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
    "infinicore-infer_b200",
)
if not _os.path.isdir(_SRC):
    raise ImportError(f"framework sources not found at {_SRC}")
__path__ = [_SRC]
with open(_os.path.join(_SRC, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_SRC, "__init__.py"), "exec"))
del _f
