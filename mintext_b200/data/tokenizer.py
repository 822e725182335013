"""Tokenizer wrapper used by the data-preparation tools (reference: mintext/data/tokenizer.py): a HuggingFace
``AutoTokenizer`` (name or local directory) or a SentencePiece ``.model`` file behind one small interface."""

from __future__ import annotations


class Tokenizer:
    def __init__(self, path: str, type: str = "auto"):  # noqa: A002 - the reference's argument names
        """``type``: ``huggingface`` | ``sentencepiece`` | ``auto`` (a ``.model`` file is SentencePiece)."""
        name_or_path, tokenizer_type = path, type
        if tokenizer_type not in ("auto", "huggingface", "sentencepiece"):
            raise ValueError(f"Unknown tokenizer type: {tokenizer_type}")
        self._sp = None
        self._hf = None
        if tokenizer_type == "sentencepiece" or (tokenizer_type == "auto" and str(name_or_path).endswith(".model")):
            import sentencepiece as spm

            self._sp = spm.SentencePieceProcessor(model_file=str(name_or_path))
        else:
            from transformers import AutoTokenizer

            self._hf = AutoTokenizer.from_pretrained(name_or_path)

    def encode(self, text: str, add_eos: bool = False) -> list[int]:
        ids = self._sp.encode(text) if self._sp is not None else self._hf.encode(text, add_special_tokens=False)
        if add_eos and self.eos_id is not None:
            ids = list(ids) + [self.eos_id]
        return list(ids)

    def decode(self, ids) -> str:
        return self._sp.decode(list(ids)) if self._sp is not None else self._hf.decode(list(ids))

    @property
    def vocab_size(self) -> int:
        return self._sp.get_piece_size() if self._sp is not None else len(self._hf)

    @property
    def eos_id(self):
        return self._sp.eos_id() if self._sp is not None else self._hf.eos_token_id

    @property
    def pad_id(self):
        return self._sp.pad_id() if self._sp is not None else self._hf.pad_token_id
