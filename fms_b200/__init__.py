"""Import name of the library.

The sources live in the folder ``foundation-model-stack_b200`` next to this one.  A hyphen cannot
appear in an ``import`` statement, so this package only redirects its search path there: every
``fms_b200.<sub>`` module is the file ``foundation-model-stack_b200/<sub>``.
"""
import os as _os

_SOURCE_DIR = _os.path.join(
    _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "foundation-model-stack_b200"
)
__path__ = [_SOURCE_DIR]
with open(_os.path.join(_SOURCE_DIR, "__init__.py"), "r", encoding="utf-8") as _f:
    exec(compile(_f.read(), _os.path.join(_SOURCE_DIR, "__init__.py"), "exec"))
del _f
