"""Human file sizes ("5G", "100MB", "1.5g", 1048576) -> bytes (reference: mintext/utils/filesize.py)."""

from __future__ import annotations

import re

_UNITS = {"": 1, "B": 1, "K": 1024, "KB": 1024, "M": 1024 ** 2, "MB": 1024 ** 2, "G": 1024 ** 3, "GB": 1024 ** 3,
          "T": 1024 ** 4, "TB": 1024 ** 4}
_PATTERN = re.compile(r"^\s*([0-9]*\.?[0-9]+)\s*([A-Za-z]*)\s*$")


def parse_file_size(size_str) -> int:
    size = size_str
    if isinstance(size, (int, float)) and not isinstance(size, bool):
        if size < 0:
            raise ValueError(f"File size must be non-negative, got {size}")
        return int(size)
    m = _PATTERN.match(str(size))
    if not m:
        raise ValueError(f"Cannot parse file size: '{size}'")
    unit = m.group(2).upper()
    if unit not in _UNITS:
        raise ValueError(f"Unknown file size unit '{m.group(2)}' in '{size}'")
    return int(float(m.group(1)) * _UNITS[unit])
