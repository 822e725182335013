"""``mintext`` - the reference's import name, served by :mod:`mintext_b200`.

``python -m mintext.train --config ...`` and ``import mintext.config`` / ``mintext.models`` / ... resolve to the
modules of the same name in ``mintext_b200`` (the same module objects, not copies).  A directory that is placed
*earlier* on ``sys.path`` and holds another ``mintext`` package (for example an installed copy of the reference that
a comparison harness puts first) still wins the import, because this alias only exists where Python finds this
directory first.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

import mintext_b200 as _impl
from mintext_b200 import *  # noqa: F401,F403

__all__ = getattr(_impl, "__all__", [])
_PREFIX = __name__ + "."


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str):
        self.target = target

    def create_module(self, spec):
        return importlib.import_module(self.target)

    def exec_module(self, module):  # already executed under its own name
        pass


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX) or fullname == _PREFIX + "train":
            return None  # mintext.train is a real module here so that `python -m mintext.train` runs main()
        real = "mintext_b200." + fullname[len(_PREFIX):]
        try:
            found = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if found is None:
            return None
        return importlib.util.spec_from_loader(fullname, _AliasLoader(real), is_package=found.submodule_search_locations is not None)


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
