"""Tokenizers for the command line.  ``CharTokenizer``: every character is a token, its id is ord(c),
vocabulary 256, begin-of-text 2, end-of-text 3 (fms/utils/tokenizers.py:97-143).  ``get_tokenizer`` also
opens a folder with a ``tokenizer.json`` when the ``tokenizers`` package is there
(fms/utils/tokenizers.py:459-502 chooses among sentencepiece, HF and the character tokenizer)."""
from __future__ import annotations

import os
from typing import List


class BaseTokenizer:
    def __init__(self, bos_id: int, eos_id: int) -> None:
        self.bos_token_id = bos_id
        self.eos_token_id = eos_id

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        raise NotImplementedError

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        raise NotImplementedError

    def vocab_size(self) -> int:
        raise NotImplementedError


class CharTokenizer(BaseTokenizer):
    def __init__(self) -> None:
        super().__init__(2, 3)

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = [ord(ch) if ord(ch) < 256 else 0 for ch in text]
        return [self.bos_token_id] + ids if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        special = {self.bos_token_id, self.eos_token_id} if skip_special_tokens else set()
        return "".join(chr(int(i)) for i in ids if int(i) not in special)

    def vocab_size(self) -> int:
        return 256


class JsonTokenizer(BaseTokenizer):
    """A ``tokenizer.json`` read with the ``tokenizers`` package."""

    def __init__(self, path: str) -> None:
        from tokenizers import Tokenizer  # optional dependency

        self._tok = Tokenizer.from_file(path)
        bos = self._tok.token_to_id("<s>") or self._tok.token_to_id("<|begin_of_text|>") or 1
        eos = self._tok.token_to_id("</s>") or self._tok.token_to_id("<|end_of_text|>") or 2
        super().__init__(bos, eos)

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = self._tok.encode(text, add_special_tokens=False).ids
        return [self.bos_token_id] + ids if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self._tok.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def vocab_size(self) -> int:
        return self._tok.get_vocab_size()


def get_tokenizer(name: str) -> BaseTokenizer:
    if name == "char_tokenizer":
        return CharTokenizer()
    path = os.path.join(name, "tokenizer.json") if os.path.isdir(name) else name
    if os.path.isfile(path) and path.endswith(".json"):
        return JsonTokenizer(path)
    raise ValueError(f'no tokenizer at {name!r}: give "char_tokenizer" or a folder with a tokenizer.json')
