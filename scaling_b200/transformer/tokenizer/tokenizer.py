"""Tokenizer facade over the HF ``tokenizers`` library (src/scaling/transformer/tokenizer/tokenizer.py:7-117).

The facade pins the three things the framework relies on: the end-of-text token id (searched among the
spellings used by the supported vocabularies), a padding id (the same token: it is unused inside documents), and
``encode`` / ``decode`` on plain lists of ids.  ``load_tokenizers`` additionally returns a variant that does not
insert a leading space, which is what prompt-internal text (stop sequences, completions) has to be tokenised with.
"""

from __future__ import annotations

import copy
import json
from pathlib import Path
from typing import Iterable, Optional, Union

from tokenizers import Tokenizer as _HFTokenizer

# checked in this order; the first one present in the vocabulary is the end-of-text token
EOS_CANDIDATES = ("<|end_of_text|>", "<|endoftext|>", "</s>")


class Tokenizer:
    def __init__(self, tokenizer: _HFTokenizer) -> None:
        self.tokenizer = tokenizer
        eos: Optional[int] = None
        for candidate in EOS_CANDIDATES:
            eos = tokenizer.token_to_id(candidate)
            if eos is not None:
                break
        assert eos is not None, "EOS token not defined for the given tokenizer."
        self.eos_token_id: int = eos
        self.padding_token_id: int = eos  # also the placeholder id under image prefixes

    # ------------------------------------------------------------------ constructors
    @classmethod
    def from_file(cls, filename: Union[str, Path]) -> "Tokenizer":
        return cls(_HFTokenizer.from_file(str(filename)))

    @classmethod
    def from_str(cls, json_str: str) -> "Tokenizer":
        return cls(_HFTokenizer.from_str(json_str))

    @classmethod
    def default(cls) -> "Tokenizer":
        """The vocabulary file shipped beside this module, if one was installed there."""
        path = Path(__file__).parent / "alpha-001-128k.json"
        if not path.is_file():
            raise FileNotFoundError(
                f"no default vocabulary at {path}; pass a tokenizer file (Tokenizer.from_file) instead"
            )
        return cls.from_file(path)

    @classmethod
    def from_words(cls, words: Iterable[str], eos_token: str = "<|endoftext|>", unk_token: str = "<unk>") -> "Tokenizer":
        """A whitespace word-level tokenizer over ``words`` - for tests and toy corpora, no training involved."""
        vocab = {eos_token: 0, unk_token: 1}
        for w in words:
            vocab.setdefault(w, len(vocab))
        definition = {
            "version": "1.0", "truncation": None, "padding": None,
            "added_tokens": [{"id": 0, "content": eos_token, "single_word": False, "lstrip": False, "rstrip": False,
                              "normalized": False, "special": True}],
            "normalizer": None, "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None,
            "decoder": None,
            "model": {"type": "WordLevel", "vocab": vocab, "unk_token": unk_token},
        }
        return cls.from_str(json.dumps(definition))

    # ------------------------------------------------------------------ queries
    def __len__(self) -> int:
        return self.tokenizer.get_vocab_size(with_added_tokens=False)

    @property
    def vocab_size(self) -> int:
        return len(self)

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return self.tokenizer.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, token_ids: list[int], skip_special_tokens: bool = True) -> str:
        return self.tokenizer.decode(list(token_ids), skip_special_tokens=skip_special_tokens)


def _without_prefix_space(definition: dict, has_sentencepiece_markers: bool) -> Optional[dict]:
    """Copy of a tokenizer definition with every "insert a leading space" rule switched off; None if it has none."""
    d = copy.deepcopy(definition)
    changed = False
    pre = d.get("pre_tokenizer")
    if pre:
        if pre.get("add_prefix_space", False):
            pre["add_prefix_space"] = False
            changed = True
        if pre.get("type") == "Sequence":
            for part in pre.get("pretokenizers", []):
                if part.get("add_prefix_space", False):
                    part["add_prefix_space"] = False
                    changed = True
    if has_sentencepiece_markers:
        # sentencepiece-style vocabularies prepend a marker in the normalizer and strip one space when decoding
        dec = d.get("decoder")
        if dec and dec.get("type") == "Sequence":
            dec["decoders"] = [x for x in dec["decoders"]
                               if not (x.get("type", "") == "Strip" and x.get("content", "") == " ")]
            changed = True
        norm = d.get("normalizer")
        if norm and norm.get("type") == "Sequence":
            norm["normalizers"] = [x for x in norm["normalizers"] if x.get("type", "") != "Prepend"]
            changed = True
    return d if changed else None


def load_tokenizers(tokenizer_file: Union[str, Path]) -> tuple[Tokenizer, Tokenizer]:
    """``(tokenizer, tokenizer_no_prefix_space)`` from one vocabulary file."""
    tokenizer_file = Path(tokenizer_file)
    tokenizer = Tokenizer.from_file(tokenizer_file)
    with open(tokenizer_file, "r", encoding="UTF-8") as f:
        definition = json.load(f)
    sp = tokenizer.tokenizer.token_to_id("<s>") is not None and tokenizer.tokenizer.token_to_id("<unk>") is not None
    modified = _without_prefix_space(definition, sp)
    if modified is None:
        return tokenizer, tokenizer
    return tokenizer, Tokenizer.from_str(json.dumps(modified))
