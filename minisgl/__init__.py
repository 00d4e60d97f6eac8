"""Import shim: ``minisgl`` is the public package name of this engine.

The sources live in the sibling directory ``deepseek-v4-sm80_b200/`` (its name is
not a valid Python identifier), so this package redirects its search path there and
runs that directory's ``__init__``.  ``python -m minisgl``, ``minisgl.llm.LLM`` and
``minisgl.distributed.launch_tensor_parallel`` therefore resolve to the B200 engine.
"""
import os as _os

_SRC = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "deepseek-v4-sm80_b200")
__path__ = [_SRC]
with open(_os.path.join(_SRC, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_SRC, "__init__.py"), "exec"))
del _f
