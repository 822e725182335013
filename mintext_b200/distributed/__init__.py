"""Alias of :mod:`mintext_b200.parallel` under the reference's package name (``mintext.distributed``): the package and
its ``mesh`` / ``partition`` / ``sharding`` submodules are the same module objects under both names."""

import sys as _sys

from mintext_b200.parallel import *  # noqa: F401,F403
from mintext_b200.parallel import mesh, partition, sharding  # noqa: F401

for _name, _mod in (("mesh", mesh), ("partition", partition), ("sharding", sharding)):
    _sys.modules.setdefault(f"{__name__}.{_name}", _mod)
