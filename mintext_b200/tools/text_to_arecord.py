"""Tokenise text corpora (jsonl, jsonl.gz, parquet, plain text) into per-document record shards, or into a Megatron
``.bin`` / ``.idx`` pair (reference: tools/text_to_arecord.py).

    python -m mintext_b200.tools.text_to_arecord --input data/*.jsonl --tokenizer meta-llama/Llama-3.2-1B \
        --output /data/corpus_arecord [--text-key text] [--workers 8] [--max-file-size 1G] [--append-eos] [--format arecord|mmap]

``.zst`` inputs need the optional ``zstandard`` package.
"""

from __future__ import annotations

import argparse
import glob
import gzip
import io
import json
import logging
import multiprocessing as mp
from pathlib import Path
from typing import Iterator

import numpy as np

from mintext_b200.data.indexed_dataset import write_mmap_dataset
from mintext_b200.tools.records import ShardedRecordWriter
from mintext_b200.utils.filesize import parse_file_size

_TOK = None


def iter_texts(path: str, text_key: str) -> Iterator[str]:
    p = Path(path)
    name = p.name
    if name.endswith(".parquet"):
        import pyarrow.parquet as pq

        for batch in pq.ParquetFile(path).iter_batches(columns=[text_key]):
            for v in batch.column(0).to_pylist():
                if v:
                    yield v
        return
    if name.endswith(".gz"):
        fh = io.TextIOWrapper(gzip.open(path, "rb"), encoding="utf-8")
    elif name.endswith(".zst"):
        import zstandard  # type: ignore

        fh = io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(open(path, "rb")), encoding="utf-8")
    else:
        fh = open(path, encoding="utf-8")
    with fh:
        if ".jsonl" in name or name.endswith(".json"):
            for line in fh:
                line = line.strip()
                if line:
                    v = json.loads(line).get(text_key)
                    if v:
                        yield v
        else:
            for line in fh:
                if line.strip():
                    yield line.rstrip("\n")


def _init_worker(tokenizer_name: str, tokenizer_type: str) -> None:
    global _TOK
    from mintext_b200.data.tokenizer import Tokenizer

    _TOK = Tokenizer(tokenizer_name, tokenizer_type)


def _encode(args):
    text, append_eos = args
    return _TOK.encode(text, add_eos=append_eos)


def convert(inputs: list[str], output: str, tokenizer: str, text_key: str = "text", workers: int = 1,
            max_bytes: int = 1 << 30, append_eos: bool = False, fmt: str = "arecord", tokenizer_type: str = "auto",
            encode_fn=None) -> int:
    """Returns the number of documents written.  ``encode_fn`` (text -> ids) bypasses the tokenizer (tests)."""
    files = sorted(f for pat in inputs for f in glob.glob(pat)) or inputs

    def texts():
        for f in files:
            yield from iter_texts(f, text_key)

    if encode_fn is not None:
        docs = (encode_fn(t) for t in texts())
        pool = None
    elif workers > 1:
        pool = mp.Pool(workers, initializer=_init_worker, initargs=(tokenizer, tokenizer_type))
        docs = pool.imap(_encode, ((t, append_eos) for t in texts()), chunksize=64)
    else:
        _init_worker(tokenizer, tokenizer_type)
        docs = (_encode((t, append_eos)) for t in texts())
        pool = None
    n = 0
    try:
        if fmt == "mmap":
            all_docs = [np.asarray(d, dtype=np.int32) for d in docs if len(d)]
            dtype = np.uint16 if all(int(d.max()) < 65536 for d in all_docs) else np.int32
            write_mmap_dataset(output, all_docs, dtype=dtype)
            n = len(all_docs)
        else:
            first = None
            writer = None
            for d in docs:
                if not len(d):
                    continue
                if writer is None:
                    first = np.asarray(d)
                    writer = ShardedRecordWriter(output, max_bytes, np.uint16 if int(first.max()) < 65536 else np.int32)
                writer.write_document(d)
                n += 1
            if writer is not None:
                writer.close()
    finally:
        if pool is not None:
            pool.close()
            pool.join()
    return n


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="text -> tokenised record shards")
    ap.add_argument("--input", nargs="+", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--tokenizer", "--tokenizer-path", dest="tokenizer", required=True)
    ap.add_argument("--tokenizer-type", default="auto", choices=["auto", "huggingface", "sentencepiece"])
    ap.add_argument("--text-key", default="text")
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--max-file-size", default="1G")
    ap.add_argument("--append-eos", action="store_true")
    ap.add_argument("--format", default="arecord", choices=["arecord", "mmap"])
    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(message)s")
    n = convert(args.input, args.output, args.tokenizer, args.text_key, args.workers,
                parse_file_size(args.max_file_size), args.append_eos, args.format, args.tokenizer_type)
    logging.info("wrote %d documents to %s", n, args.output)


if __name__ == "__main__":
    main()
