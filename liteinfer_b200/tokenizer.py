"""Text <-> token ids.

The reference wraps `transformers.AutoTokenizer` (liteinfer/tokenizer.py:20-48:
`encode` adds no special tokens, `decode` skips them, `eos_token_ids` is a
tuple).  Here a model folder with a `tokenizer.json` is read with the
`tokenizers` library; a folder without one (random weights) gets
`TokenIdTokenizer`, whose "text" is token ids written as decimal numbers with
spaces between them.  `IncrementalDetokenizer` keeps the text of a growing
sequence without decoding the whole prefix each step (tokenizer.py:50-78).
"""

from __future__ import annotations

import json
from pathlib import Path

_REPLACEMENT_CHAR = "�"


def _eos_ids_from_files(model_dir: Path, token_to_id) -> tuple[int, ...]:
    for name in ("generation_config.json", "config.json"):
        path = model_dir / name
        if path.is_file():
            eos = json.loads(path.read_text()).get("eos_token_id")
            if isinstance(eos, list):
                return tuple(int(e) for e in eos)
            if eos is not None:
                return (int(eos),)
    path = model_dir / "tokenizer_config.json"
    if path.is_file() and token_to_id is not None:
        eos = json.loads(path.read_text()).get("eos_token")
        if isinstance(eos, dict):
            eos = eos.get("content")
        if isinstance(eos, str):
            token_id = token_to_id(eos)
            if token_id is not None:
                return (int(token_id),)
    return ()


class TokenIdTokenizer:
    """For models without a vocabulary file: text is ids as decimal numbers, e.g. "5 17 3"."""

    def __init__(self, vocab_size: int, eos_token_ids: tuple[int, ...] = ()) -> None:
        self._vocab_size = vocab_size
        self.eos_token_ids = tuple(eos_token_ids)

    @property
    def vocab_size(self) -> int:
        return self._vocab_size

    def encode(self, text: str) -> list[int]:
        try:
            ids = [int(piece) for piece in text.replace(",", " ").split()]
        except ValueError:
            raise ValueError("this model has no tokenizer.json: give the prompt as token ids, e.g. '5 17 3'") from None
        for i in ids:
            if not 0 <= i < self._vocab_size:
                raise ValueError(f"token id {i} is outside the vocabulary [0, {self._vocab_size})")
        return ids

    def decode(self, token_ids: list[int]) -> str:
        return " ".join(str(i) for i in token_ids)


class FileTokenizer:
    """A `tokenizer.json` read with the `tokenizers` library."""

    def __init__(self, model_dir: Path) -> None:
        from tokenizers import Tokenizer as _Tokenizer

        self._tok = _Tokenizer.from_file(str(model_dir / "tokenizer.json"))
        self.eos_token_ids = _eos_ids_from_files(model_dir, self._tok.token_to_id)

    @property
    def vocab_size(self) -> int:
        return int(self._tok.get_vocab_size())

    def encode(self, text: str) -> list[int]:
        return list(self._tok.encode(text, add_special_tokens=False).ids)

    def decode(self, token_ids: list[int]) -> str:
        return self._tok.decode(list(token_ids), skip_special_tokens=True)


def load_tokenizer(model_dir: str | Path, vocab_size: int, eos_token_ids: tuple[int, ...] = ()):
    model_dir = Path(model_dir)
    if (model_dir / "tokenizer.json").is_file():
        return FileTokenizer(model_dir)
    return TokenIdTokenizer(vocab_size, eos_token_ids or _eos_ids_from_files(model_dir, None))


class IncrementalDetokenizer:
    """The text of a growing list of token ids without decoding all of it at every step.

    A tokenizer's text for a token can depend on its neighbours (spaces, bytes of one character spread over two
    tokens), so new tokens are decoded together with a few settled tokens before them, and what those settled
    tokens decode to alone is cut off the front.  Text that ends in the replacement character is an unfinished
    character: it is held back until the token that completes it has come.  (The reference does the same with a
    prefix offset and a read offset, liteinfer/tokenizer.py:50-78.)
    """

    CONTEXT = 6         # settled tokens decoded again in front of the new ones

    def __init__(self) -> None:
        self.text = ""
        self.settled = 0            # tokens whose text is in `text`

    def _fresh(self, tokenizer, token_ids: list[int]) -> str:
        """What the tokens after the settled ones add to the text."""
        anchor = max(0, self.settled - self.CONTEXT)
        before = tokenizer.decode(token_ids[anchor:self.settled]) if self.settled > anchor else ""
        whole = tokenizer.decode(token_ids[anchor:])
        return whole[len(before):] if len(whole) > len(before) else ""

    def update(self, tokenizer, token_ids: list[int]) -> str:
        if len(token_ids) > self.settled:
            fresh = self._fresh(tokenizer, token_ids)
            if fresh and not fresh.endswith(_REPLACEMENT_CHAR):
                self.text += fresh
                self.settled = len(token_ids)
        return self.text

    def catch_up(self, tokenizer, token_ids: list[int]) -> str:
        """The text of all of `token_ids`, for a detokenizer that was not called at every step: what `update`
        gives, and if the ids end inside a character, everything before that character."""
        text = self.update(tokenizer, token_ids)
        if self.settled == len(token_ids):
            return text
        return text + self._fresh(tokenizer, token_ids).rstrip(_REPLACEMENT_CHAR)
