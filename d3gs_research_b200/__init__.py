"""Importable alias of the ``d3gs-research_b200`` package directory.

The package directory carries the project's name, which contains a hyphen and therefore cannot be
written in an ``import`` statement.  This module makes ``import d3gs_research_b200`` resolve to
it: the package path points at the hyphenated directory and its ``__init__`` is executed here.
"""
import os as _os

_real = _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))), "d3gs-research_b200")
__path__ = [_real]
__file__ = _os.path.join(_real, "__init__.py")
with open(__file__) as _f:
    exec(compile(_f.read(), __file__, "exec"))
del _f
