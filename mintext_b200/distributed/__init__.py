"""Alias of :mod:`mintext_b200.parallel` under the reference's package name (``mintext.distributed``)."""

from mintext_b200.parallel import *  # noqa: F401,F403
from mintext_b200.parallel import mesh, partition, sharding  # noqa: F401
