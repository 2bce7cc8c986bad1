"""Import name of the package kept in the folder `xpu-serve_b200/`.

A hyphen cannot appear in an import statement, so this module stands in for the folder:
it points its `__path__` there and runs the folder's `__init__.py` in its own namespace.
`import xpu_serve_b200.engine` then loads `xpu-serve_b200/engine/`.
"""
import os as _os

__package__ = "xpu_serve_b200"
__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "xpu-serve_b200")]
__spec__.submodule_search_locations = __path__   # makes this module a package for the import system
with open(_os.path.join(__path__[0], "__init__.py"), "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
del _f
