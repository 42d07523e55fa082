"""Import shim: the package directory is named `layered-prefill_b200` (not a valid Python
identifier), so `import layered_prefill_b200` resolves to this module, which turns itself into
that package by pointing __path__ at the directory and running its __init__.py."""
import os as _os

__path__ = [_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "layered-prefill_b200")]
__file__ = _os.path.join(__path__[0], "__init__.py")
with open(__file__) as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f
