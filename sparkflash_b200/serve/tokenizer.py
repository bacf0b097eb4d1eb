"""Tokenizers behind one small interface.

* ``HfTokenizer`` loads a checkpoint's ``tokenizer.json`` (the released model's byte-level BPE with its
  special tokens) through the ``tokenizers`` library.
* ``ByteTokenizer`` is self-contained: ids 0..255 are bytes, the special tokens of the chat encoding follow.
  Synthetic-weight servers, tests and the mock engine use it (no file needed).

Both expose ``token_bytes`` (the byte string of every id) for the constraint automaton and an incremental
detokeniser that never splits a UTF-8 sequence across deltas (reference: crates/sparkflash-api/src/vocab.rs,
tests/tokenizer_seam.rs).
"""
from __future__ import annotations

import re

from .encoding import EOS, SPECIAL_TOKENS


class ByteTokenizer:
    def __init__(self, vocab_size: int | None = None, extra_special: list[str] | None = None):
        self.special = list(SPECIAL_TOKENS) + list(extra_special or [])
        self.special_ids = {s: 256 + i for i, s in enumerate(self.special)}
        self.id_special = {v: k for k, v in self.special_ids.items()}
        self.vocab_size = max(vocab_size or 0, 256 + len(self.special))
        self.eos_id = self.special_ids[EOS]
        self._split = re.compile("(" + "|".join(re.escape(s) for s in sorted(self.special, key=len, reverse=True)) + ")")

    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        out: list[int] = []
        for piece in (self._split.split(text) if allow_special else [text]):
            if allow_special and piece in self.special_ids:
                out.append(self.special_ids[piece])
            else:
                out.extend(piece.encode("utf-8"))
        return out

    def token_bytes(self) -> list[bytes]:
        out = [bytes([i]) for i in range(256)] + [s.encode("utf-8") for s in self.special]
        return out + [b""] * (self.vocab_size - len(out))

    def is_special(self, i: int) -> bool:
        return i in self.id_special

    def decode(self, ids: list[int], skip_special: bool = True) -> str:
        d = StreamDecoder(self, skip_special)
        return "".join(d.push(i) for i in ids) + d.flush()


class HfTokenizer:
    def __init__(self, path: str):
        from tokenizers import Tokenizer
        self.tk = Tokenizer.from_file(path)
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        eos = self.tk.token_to_id(EOS)
        self.eos_id = eos if eos is not None else -1
        self._special = {i for t, i in self.tk.get_vocab(with_added_tokens=True).items() if t.startswith("<｜") or t in ("<think>", "</think>")}
        self._bytes: list[bytes] | None = None

    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        return self.tk.encode(text, add_special_tokens=False).ids

    def is_special(self, i: int) -> bool:
        return i in self._special

    def token_bytes(self) -> list[bytes]:
        if self._bytes is None:
            # byte-level BPE spells bytes through the GPT-2 printable map; invert it
            bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
            cs, n = bs[:], 0
            for b in range(256):
                if b not in bs:
                    bs.append(b); cs.append(256 + n); n += 1
            inv = {chr(c): b for b, c in zip(bs, cs)}
            out = []
            for i in range(self.vocab_size):
                t = self.tk.id_to_token(i) or ""
                if i in self._special:
                    out.append(t.encode("utf-8"))
                else:
                    try:
                        out.append(bytes(inv[ch] for ch in t))
                    except KeyError:
                        out.append(t.encode("utf-8"))
            self._bytes = out
        return self._bytes

    def decode(self, ids: list[int], skip_special: bool = True) -> str:
        return self.tk.decode(ids, skip_special_tokens=skip_special)


class StreamDecoder:
    """Incremental detokeniser over ``token_bytes``: emits only whole UTF-8 sequences."""

    def __init__(self, tok, skip_special: bool = True):
        self.tok, self.skip = tok, skip_special
        self.table = tok.token_bytes()
        self.pending = b""

    def push(self, token_id: int) -> str:
        if self.skip and self.tok.is_special(token_id):
            return self.flush()
        self.pending += self.table[token_id] if 0 <= token_id < len(self.table) else b""
        # longest prefix that is complete UTF-8
        cut = len(self.pending)
        for back in range(1, min(4, len(self.pending)) + 1):
            b = self.pending[-back]
            if b >= 0xC0:      # a lead byte: is its sequence complete?
                need = 2 if b < 0xE0 else 3 if b < 0xF0 else 4
                if back < need:
                    cut = len(self.pending) - back
                break
            if b < 0x80:
                break
        out, self.pending = self.pending[:cut], self.pending[cut:]
        return out.decode("utf-8", "replace")

    def flush(self) -> str:
        out, self.pending = self.pending, b""
        return out.decode("utf-8", "replace")


def load_tokenizer(path: str | None, vocab_size: int | None = None):
    if path:
        return HfTokenizer(path)
    return ByteTokenizer(vocab_size)
