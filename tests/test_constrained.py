"""JSON-schema byte automaton and token masks (reference tests: crates/sparkflash-api/src/constrained.rs unit
tests; docs/serving.md:107-112)."""
import json
import random

import pytest

from sparkflash_b200.serve.constrained import ByteConstraint, Schema, SchemaError, TokenConstraint, TokenVocab


def accepts(schema, text: str) -> bool:
    c = ByteConstraint(Schema(schema))
    return c.feed(text.encode()) and c.can_end


PERSON = {"type": "object", "properties": {"name": {"type": "string"}, "age": {"type": "integer", "minimum": 0, "maximum": 150},
                                              "tags": {"type": "array", "items": {"type": "string", "enum": ["a", "b\"c"]}, "maxItems": 2},
                                              "ok": {"type": "boolean"}, "none": {"type": "null"}},
          "required": ["name", "age"], "additionalProperties": False}


def test_accepts_valid_documents_and_rejects_invalid():
    assert accepts(PERSON, '{"name": "Zoë \\u00e9\\n", "age": 42}')
    assert accepts(PERSON, '{"age":0,"name":"x","tags":["a","b\\"c"],"ok":true,"none":null}')
    assert not accepts(PERSON, '{"name": "x"}')                          # required key missing
    assert not accepts(PERSON, '{"name": "x", "age": 151}')              # above the maximum
    assert not accepts(PERSON, '{"name": "x", "age": 1, "age": 2}')      # a key twice
    assert not accepts(PERSON, '{"name": "x", "age": 1, "extra": 2}')    # closed object
    assert not accepts(PERSON, '{"name": "x", "age": 1, "tags": ["a","a","a"]}')
    assert not accepts(PERSON, '{"name": "x", "age": 1.5}')
    assert not accepts(PERSON, '{"name": "x", "age": 01}')
    assert not accepts(PERSON, '{"name": "x", "age": 1} x')


def test_number_bounds_are_exact_on_the_digits():
    sc = {"type": "number", "minimum": -2.5, "maximum": 10}
    for good in ["-2.5", "-2.49", "0", "10", "9.999999999", "10.0", "-0.0", "3"]:
        assert accepts(sc, good), good
    for bad in ["-2.51", "10.000000001", "11", "-3", "1e1", "100"]:
        assert not accepts(sc, bad), bad
    c = ByteConstraint(Schema({"type": "integer", "minimum": 17, "maximum": 23}))
    assert c.allowed_bytes() == {ord("1"), ord("2")}
    c.feed(b"2")
    assert c.allowed_bytes() == {ord(d) for d in "0123"} and not c.can_end
    with pytest.raises(SchemaError):
        Schema({"type": "integer", "minimum": 1.2, "maximum": 1.8})


def test_open_object_is_any_json_and_random_documents_roundtrip():
    rng = random.Random(0)

    def rand(depth=0):
        k = rng.randrange(7 if depth < 3 else 5)
        if k == 0: return rng.choice([True, False, None])
        if k == 1: return rng.randrange(-1000, 1000)
        if k == 2: return rng.random() * 10 ** rng.randrange(-3, 6)
        if k in (3, 4): return "".join(rng.choice('ab"\\ é\n') for _ in range(rng.randrange(5)))
        if k == 5: return [rand(depth + 1) for _ in range(rng.randrange(4))]
        return {f"k{i}": rand(depth + 1) for i in range(rng.randrange(4))}

    for _ in range(200):
        doc = {"x": rand()}
        for text in (json.dumps(doc), json.dumps(doc, separators=(",", ":"), ensure_ascii=False)):
            assert accepts({"type": "object"}, text), text
    assert not accepts({"type": "object"}, "[1]")
    assert not accepts({"type": "object"}, '{"a": tru}')


def test_refused_keywords_are_typed_errors():
    for bad in [{"type": "string", "pattern": "a+"}, {"anyOf": [{"type": "string"}]}, {"type": ["string", "null"]},
                {"type": "object", "additionalProperties": True}, {}, {"type": "array"}, {"type": "integer", "enum": [1]},
                {"type": "integer", "minimum": 5, "maximum": 4}, {"type": "string", "x-unknown": 1}]:
        with pytest.raises(SchemaError):
            Schema(bad)


def test_masked_greedy_decoding_always_yields_a_valid_document():
    # a byte-pair-ish vocabulary: single bytes plus some multi-byte tokens
    toks = [bytes([b]) for b in range(256)] + [b'{"', b'":', b'", "', b'name', b'age', b'true', b'": ', b'"}', b'12', b'999', b', "', b'""', b"<eos>"]
    eos = len(toks) - 1
    vocab = TokenVocab(toks)
    rng = random.Random(1)
    for trial in range(25):
        c = TokenConstraint(Schema(PERSON), vocab, eos)
        out = b""
        for _ in range(400):
            ids = c.allowed_ids()
            assert ids, out
            # per-rank slices give the same set
            half = vocab.n // 2
            assert ids == c.allowed_ids(0, half) + c.allowed_ids(half, vocab.n)
            # prefer to finish when possible so that the walk terminates
            pick = eos if eos in ids and rng.random() < 0.5 else rng.choice(ids)
            assert c.admits(pick) and c.advance(pick)
            if pick == eos:
                break
            out += toks[pick]
        else:
            continue
        doc = json.loads(out.decode("utf-8", "replace"))
        assert set(doc) >= {"name", "age"} and 0 <= doc["age"] <= 150 and set(doc) <= set(PERSON["properties"])
