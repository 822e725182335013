"""Write a small synthetic JSONL corpus for trying the data pipeline end to end
(reference: tools/generate_sample_jsonl.py).

    python -m mintext_b200.tools.generate_sample_jsonl --output sample.jsonl --num-docs 1000
    python -m mintext_b200.tools.text_to_arecord --input sample.jsonl --tokenizer <name> --output sample_arecord
    python -m mintext_b200.train --config configs/models/test-tiny.yml dataset_type=arecord data_path=sample_arecord
"""

from __future__ import annotations

import argparse
import json
import random

_WORDS = ("the quick brown fox jumps over the lazy dog while a curious model learns patterns from tokens and "
          "gradients flow backward through many layers of attention and feed forward blocks").split()


def generate(path: str, num_docs: int, min_words: int, max_words: int, seed: int, text_key: str = "text") -> None:
    rng = random.Random(seed)
    with open(path, "w") as f:
        for i in range(num_docs):
            n = rng.randint(min_words, max_words)
            f.write(json.dumps({"id": i, text_key: " ".join(rng.choice(_WORDS) for _ in range(n))}) + "\n")


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--output", required=True)
    ap.add_argument("--num-docs", type=int, default=1000)
    ap.add_argument("--min-words", type=int, default=20)
    ap.add_argument("--max-words", type=int, default=400)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--text-key", default="text", help="JSON key of the text field")
    a = ap.parse_args(argv)
    generate(a.output, a.num_docs, a.min_words, a.max_words, a.seed, a.text_key)
    print(f"wrote {a.num_docs} documents to {a.output}")


if __name__ == "__main__":
    main()
