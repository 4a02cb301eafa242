"""Text <-> token ids: the id tokenizer of folders without a vocabulary, and the incremental detokenizer."""

from __future__ import annotations

import pytest

from liteinfer_b200.tokenizer import IncrementalDetokenizer, TokenIdTokenizer


class ByteTokenizer:
    """One token per byte: characters of several bytes arrive in pieces, as with byte-level vocabularies."""

    def decode(self, token_ids):
        return bytes(token_ids).decode("utf-8", errors="replace")


class SpacingTokenizer:
    """A word per token, but the first token of a text gets no space before it: the text of a token depends on
    what stands before it."""

    def decode(self, token_ids):
        return " ".join(f"w{t}" for t in token_ids)


@pytest.mark.parametrize("text", ["plain ascii", "héllo wörld", "✓ done — ok", "日本語のテキスト", "a🙂b"])
def test_text_grows_token_by_token_and_never_shows_half_a_character(text):
    tok, ids = ByteTokenizer(), list(text.encode("utf-8"))
    inc = IncrementalDetokenizer()
    seen = ""
    for n in range(1, len(ids) + 1):
        now = inc.update(tok, ids[:n])
        assert now.startswith(seen) and "�" not in now and text.startswith(now)
        seen = now
    assert seen == text


def test_catching_up_after_skipped_steps_gives_the_same_text():
    tok, ids = ByteTokenizer(), list("naïve café ✓".encode("utf-8"))
    assert IncrementalDetokenizer().catch_up(tok, ids) == "naïve café ✓"
    cut = ids[:-1]                                   # ends inside the last character
    assert IncrementalDetokenizer().catch_up(tok, cut) == "naïve café "
    stepped = IncrementalDetokenizer()
    stepped.update(tok, ids[:4])
    assert stepped.catch_up(tok, ids) == "naïve café ✓"


def test_text_that_depends_on_the_token_before():
    tok, ids = SpacingTokenizer(), [5, 17, 3, 3, 9, 12, 40, 2, 8, 1]
    inc = IncrementalDetokenizer()
    for n in range(1, len(ids) + 1):
        assert inc.update(tok, ids[:n]) == tok.decode(ids[:n])


def test_token_id_tokenizer():
    tok = TokenIdTokenizer(100, (7,))
    assert tok.encode("5 17, 3") == [5, 17, 3] and tok.decode([5, 17, 3]) == "5 17 3" and tok.eos_token_ids == (7,)
    with pytest.raises(ValueError):
        tok.encode("5 x")
    with pytest.raises(ValueError):
        tok.encode("100")
