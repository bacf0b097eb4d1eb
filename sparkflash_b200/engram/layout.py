"""Engram layout and hashing: compressed token map, prime buckets, multipliers, n-gram hash ids.

Reference: crates/sparkflash-engram/src/{hash,primes}.rs and docs/architecture/04-engram.md sections 2-5
(normaliser chain, 48 disjoint primes above the engram vocabulary whose per-layer sums are the table row
counts, odd multipliers bounded by int64_max / compressed_vocab / 2, XOR of per-shift products reduced modulo
the bucket prime, look-back blocked by dead positions and the sequence start).
"""
from __future__ import annotations

import ctypes
import re
import unicodedata
from ctypes import c_int, c_int64, c_void_p
from dataclasses import dataclass

import numpy as np

from .. import _lib

DEAD = -1
# multipliers of the released model (layers 1 and 14, compressed vocabulary 99092): numpy's PCG64 stream seeded
# with 10007 * layer_id, bounded draws below 46539438283891, forced odd
RELEASED_MULTIPLIERS = {
    (1, 99092): [76632096046245, 4839876093313, 35959672319349, 73987337458391],
    (14, 99092): [67716810739261, 51510806800915, 30921347202721, 82619226485591],
}
_declared = False


def _L():
    global _declared
    L = _lib.host()
    if not _declared:
        L.sfb_engram_primes.argtypes = [c_int64, c_int, c_int, c_int, c_void_p]
        L.sfb_engram_hash.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]
        L.sfb_engram_pack.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int64, c_int64, c_void_p, c_int]
        _declared = True
    return L


def normalise_token(text: str) -> str:
    t = unicodedata.normalize("NFKC", text)
    t = unicodedata.normalize("NFD", t)
    t = "".join(ch for ch in t if unicodedata.category(ch) != "Mn")       # strip accents
    t = t.lower()
    t = re.sub(r"[ \t\r\n]+", " ", t)
    t = re.sub(r"^ $", "", t)          # a lone space survives the strip below
    t = t.strip()
    return t.replace("", " ")


def build_compressed_token_map(decoded: list[str], raw: list[str] | None = None) -> tuple[np.ndarray, int]:
    """lookup[token_id] = dense id of the token's normalised spelling (first-seen order).  ``decoded``: each
    id decoded alone; ``raw``: the vocabulary strings, used for ids whose decoding is a partial UTF-8 sequence."""
    keys: dict[str, int] = {}
    lookup = np.zeros(len(decoded), dtype=np.int64)
    for i, text in enumerate(decoded):
        if "�" in text:
            key = raw[i] if raw is not None else f"�{i}"
        else:
            key = normalise_token(text) or text
        lookup[i] = keys.setdefault(key, len(keys))
    return lookup, len(keys)


def multipliers(layer_id: int, max_ngram: int, compressed_vocab: int) -> list[int]:
    if (layer_id, compressed_vocab) in RELEASED_MULTIPLIERS and max_ngram == 4:
        return list(RELEASED_MULTIPLIERS[(layer_id, compressed_vocab)])
    bound = max(1, ((2 ** 63 - 1) // compressed_vocab) // 2)
    vals = np.random.default_rng(10007 * layer_id).integers(0, bound, size=(max_ngram,), dtype=np.int64)
    return [int(v) * 2 + 1 for v in vals]


@dataclass
class EngramLayout:
    layer_ids: list[int]
    max_ngram: int
    n_heads: int
    engram_vocab: int
    compressed_vocab: int
    primes: np.ndarray          # [layers, orders, heads]
    offsets: np.ndarray         # [layers, orders, heads]  first row of each bucket inside its layer's table
    rows: list[int]             # rows per layer's table
    mult: np.ndarray            # [layers, max_ngram]

    @classmethod
    def build(cls, layer_ids, max_ngram, n_heads, engram_vocab, compressed_vocab, expect_rows=None) -> "EngramLayout":
        orders = max_ngram - 1
        pr = np.zeros((len(layer_ids), orders, n_heads), dtype=np.int64)
        _L().sfb_engram_primes(engram_vocab, len(layer_ids), orders, n_heads, pr.ctypes.data_as(c_void_p))
        flat = pr.reshape(len(layer_ids), -1)
        offs = (np.cumsum(flat, axis=1) - flat).reshape(pr.shape)
        rows = [int(x) for x in flat.sum(axis=1)]
        if expect_rows is not None and list(expect_rows) != rows:
            raise ValueError(f"prime buckets sum to {rows}, the checkpoint says {list(expect_rows)}: a different layout would rehash the whole table")
        mult = np.array([multipliers(l, max_ngram, compressed_vocab) for l in layer_ids], dtype=np.int64)
        return cls(list(layer_ids), max_ngram, n_heads, engram_vocab, compressed_vocab, pr, offs, rows, mult)

    @property
    def cols(self) -> int:
        return (self.max_ngram - 1) * self.n_heads

    def hash_ids(self, layer_index: int, cache: np.ndarray, positions, pad_id: int) -> np.ndarray:
        """Row ids [n, cols] of ``positions`` given the sequence's compressed-id cache (dead = -1)."""
        cache = np.ascontiguousarray(cache, dtype=np.int64)
        pos = np.ascontiguousarray(positions, dtype=np.int32)
        out = np.zeros((len(pos), self.cols), dtype=np.int64)
        pr = np.ascontiguousarray(self.primes[layer_index].reshape(-1))
        of = np.ascontiguousarray(self.offsets[layer_index].reshape(-1))
        mu = np.ascontiguousarray(self.mult[layer_index])
        _L().sfb_engram_hash(cache.ctypes.data_as(c_void_p), pos.ctypes.data_as(c_void_p), len(pos), self.max_ngram, self.n_heads,
                             pad_id, mu.ctypes.data_as(c_void_p), pr.ctypes.data_as(c_void_p), of.ctypes.data_as(c_void_p),
                             out.ctypes.data_as(c_void_p))
        return out


def hash_ids_reference(layout: EngramLayout, layer_index: int, cache, positions, pad_id: int) -> np.ndarray:
    """Plain transcription of the reference's tensor program for one sequence (python ints, slow)."""
    out = []
    M = 1 << 64
    for p in positions:
        blocked, toks = False, []
        for s in range(layout.max_ngram):
            src = int(cache[max(p - s, 0)])
            blocked = blocked or p < s or src == DEAD
            toks.append(pad_id if blocked else src)
        prods = []
        for s, t in enumerate(toks):
            v = (t * int(layout.mult[layer_index, s])) % M
            prods.append(v - M if v >= M // 2 else v)          # int64 wraparound
        row, rolling = [], prods[0]
        for s in range(1, layout.max_ngram):
            rolling ^= prods[s]
            for h in range(layout.n_heads):
                pr = int(layout.primes[layer_index, s - 1, h])
                row.append(rolling % pr + int(layout.offsets[layer_index, s - 1, h]))
        out.append(row)
    return np.array(out, dtype=np.int64)
