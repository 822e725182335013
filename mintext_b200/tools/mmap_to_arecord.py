"""Convert a Megatron ``.bin`` / ``.idx`` corpus into per-document record shards (reference: tools/mmap_to_arecord.py).

    python -m mintext_b200.tools.mmap_to_arecord --input /data/corpus_text_document --output /data/corpus_arecord \
        [--max-file-size 1G]
"""

from __future__ import annotations

import argparse
import logging

import numpy as np

from mintext_b200.data.indexed_dataset import MMapIndexedDataset
from mintext_b200.tools.records import ShardedRecordWriter
from mintext_b200.utils.filesize import parse_file_size


def convert(input_prefix: str, output_dir: str, max_bytes: int) -> int:
    ds = MMapIndexedDataset(input_prefix)
    vocab_fits_u16 = ds._dtype.itemsize <= 2
    w = ShardedRecordWriter(output_dir, max_bytes, np.uint16 if vocab_fits_u16 else np.int32)
    for i in range(len(ds)):
        w.write_document(ds[i])
    return len(w.close())


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="mmap (.bin/.idx) -> record shards")
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--max-file-size", default="1G")
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(message)s")
    n = convert(args.input, args.output, parse_file_size(args.max_file_size))
    logging.info("wrote %d shard(s) to %s", n, args.output)


if __name__ == "__main__":
    main()
