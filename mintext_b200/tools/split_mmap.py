"""Split a large ``.bin`` token file into parts at sequence boundaries (the ``.idx`` stays valid: byte pointers are
positions in the logical concatenation of ``prefix.bin.00000``, ``prefix.bin.00001`` ..., which is how the reader
addresses multi-part data).  Reference tool: tools/split_mmap.py.

    python -m mintext_b200.tools.split_mmap --input /data/corpus_text_document --max-file-size 5G [--output PREFIX]
"""

from __future__ import annotations

import argparse
import logging
import shutil
import sys
from pathlib import Path

import numpy as np

from mintext_b200.data.indexed_dataset import MMapIndexedDataset
from mintext_b200.utils.filesize import parse_file_size

_CHUNK = 64 * 1024 * 1024


def plan_parts(pointers: np.ndarray, lengths: np.ndarray, itemsize: int, total_bytes: int, max_bytes: int) -> list[tuple[int, int]]:
    """Byte ranges ``[(start, end), ...]`` that never cut a sequence and stay below ``max_bytes`` when possible."""
    ends = pointers.astype(np.int64) + lengths.astype(np.int64) * itemsize
    parts, start = [], 0
    last_end = 0
    for end in ends.tolist():
        if end - start > max_bytes and last_end > start:
            parts.append((start, last_end))
            start = last_end
        last_end = end
    parts.append((start, total_bytes))
    return parts


def split(input_prefix: str, output_prefix: str, max_bytes: int) -> int:
    bin_path = Path(f"{input_prefix}.bin")
    if not bin_path.exists():
        raise FileNotFoundError(f"Data file not found: {bin_path}")
    size = bin_path.stat().st_size
    if size <= max_bytes:
        logging.info("%s is %d bytes (<= %d): nothing to split", bin_path, size, max_bytes)
        return 1
    ds = MMapIndexedDataset(input_prefix)
    parts = plan_parts(ds._sequence_pointers, ds._sequence_lengths, ds._dtype_size, size, max_bytes)
    with open(bin_path, "rb") as src:
        for i, (a, b) in enumerate(parts):
            with open(f"{output_prefix}.bin.{i:05d}", "wb") as dst:
                src.seek(a)
                left = b - a
                while left > 0:
                    buf = src.read(min(_CHUNK, left))
                    dst.write(buf)
                    left -= len(buf)
            logging.info("part %05d: bytes [%d, %d)", i, a, b)
    if output_prefix != input_prefix:
        shutil.copyfile(f"{input_prefix}.idx", f"{output_prefix}.idx")
    return len(parts)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="Split a .bin file at sequence boundaries")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", default=None)
    ap.add_argument("--max-file-size", default="5G")
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(message)s")
    try:
        n = split(args.input, args.output or args.input, parse_file_size(args.max_file_size))
    except FileNotFoundError as e:
        logging.error("%s", e)
        sys.exit(1)
    logging.info("wrote %d part(s)", n)


if __name__ == "__main__":
    main()
