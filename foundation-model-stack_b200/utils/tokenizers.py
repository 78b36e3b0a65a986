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

    # The older four calls of the reference's tokenizers (fms/utils/tokenizers.py:66-91), which its scripts
    # still use: text -> token strings -> ids and back.
    def tokenize(self, text: str) -> List[str]:
        raise NotImplementedError

    def convert_tokens_to_ids(self, tokens):
        raise NotImplementedError

    def convert_ids_to_tokens(self, ids) -> List[str]:
        raise NotImplementedError

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        raise NotImplementedError

    def vocab_size(self) -> int:
        raise NotImplementedError


class CharTokenizer(BaseTokenizer):
    def __init__(self) -> None:
        super().__init__(2, 3)

    def tokenize(self, text: str) -> List[str]:
        return list(text)

    def convert_tokens_to_ids(self, tokens):
        def one(t: str) -> int:
            return ord(t) if len(t) == 1 and ord(t) < 256 else 0

        if isinstance(tokens, str):  # one token gives one id
            if len(tokens) != 1:
                raise RuntimeError("a token of the character tokenizer is one character")
            return one(tokens)
        return [one(t) for t in tokens]

    def convert_ids_to_tokens(self, ids) -> List[str]:
        return [chr(int(i)) for i in ids]

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        return "".join(tokens)

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
        def first_id(names, default):  # an id may be 0: compare with None, not by truth
            found = [i for i in (self._tok.token_to_id(n) for n in names) if i is not None]
            return found[0] if found else default

        super().__init__(first_id(("<s>", "<|begin_of_text|>"), 1), first_id(("</s>", "<|end_of_text|>"), 2))

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = self._tok.encode(text, add_special_tokens=False).ids
        return [self.bos_token_id] + ids if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self._tok.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)

    def tokenize(self, text: str) -> List[str]:
        return self._tok.encode(text, add_special_tokens=False).tokens

    def convert_tokens_to_ids(self, tokens):
        if isinstance(tokens, str):
            return self._tok.token_to_id(tokens)
        return [self._tok.token_to_id(t) for t in tokens]

    def convert_ids_to_tokens(self, ids) -> List[str]:
        return [self._tok.id_to_token(int(i)) for i in ids]

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        return self.decode(self.convert_tokens_to_ids(tokens), skip_special_tokens=False)

    def vocab_size(self) -> int:
        return self._tok.get_vocab_size()


class SentencePieceTokenizer(BaseTokenizer):
    """A sentencepiece ``.model`` file, as the reference reads Meta's tokenizers (fms/utils/tokenizers.py:146-203)."""

    def __init__(self, path: str) -> None:
        from sentencepiece import SentencePieceProcessor  # optional dependency

        self._sp = SentencePieceProcessor(model_file=path)
        super().__init__(self._sp.bos_id(), self._sp.eos_id())

    def tokenize(self, text: str) -> List[str]:
        return self._sp.encode_as_pieces(text)

    def convert_tokens_to_ids(self, tokens):
        return self._sp.piece_to_id(tokens)

    def convert_ids_to_tokens(self, ids) -> List[str]:
        return self._sp.id_to_piece([int(i) for i in ids])

    def convert_tokens_to_string(self, tokens: List[str]) -> str:
        return self._sp.decode_pieces(list(tokens))

    def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
        ids = self._sp.encode(text)
        return [self.bos_token_id] + ids if add_special_tokens and self.bos_token_id >= 0 else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self._sp.decode([int(i) for i in ids])

    def vocab_size(self) -> int:
        return self._sp.vocab_size()


def get_tokenizer(name: str) -> BaseTokenizer:
    """"char_tokenizer", a sentencepiece ``.model`` file, a ``tokenizer.json`` or a folder that holds one of the two
    (fms/utils/tokenizers.py:459-502)."""
    if name == "char_tokenizer":
        return CharTokenizer()
    if os.path.isdir(name):
        for candidate in ("tokenizer.json", "tokenizer.model"):
            if os.path.isfile(os.path.join(name, candidate)):
                name = os.path.join(name, candidate)
                break
    if os.path.isfile(name) and name.endswith(".json"):
        return JsonTokenizer(name)
    if os.path.isfile(name) and name.endswith(".model"):
        return SentencePieceTokenizer(name)
    raise ValueError(f'no tokenizer at {name!r}: give "char_tokenizer", a sentencepiece .model file, a tokenizer.json or '
                     "a folder with one of them")
