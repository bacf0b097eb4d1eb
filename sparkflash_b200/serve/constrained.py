"""Structured outputs: JSON-Schema subset -> byte automaton (csrc/host_constrain.cpp) -> token masks.

The schema front end lives here: it walks the schema, refuses every keyword the automaton does not
enforce (a typed ``SchemaError``, never silently ignored) and feeds the node table to the C++ builder.
Reference behaviour: crates/sparkflash-api/src/constrained.rs:15-80 (supported subset and refusals),
DECISIONS D61/D64 (the surface advertises what it enforces; a dead-ended sequence ends alone).
"""
from __future__ import annotations

import ctypes
import json
from ctypes import c_char_p, c_int, c_void_p
from decimal import Decimal

from .. import _lib

T_ANY, T_OBJECT, T_OPEN_OBJECT, T_ARRAY, T_STRING, T_ENUM, T_INTEGER, T_NUMBER, T_BOOLEAN, T_NULL = range(10)

REFUSED = {
    "pattern", "format", "minLength", "maxLength", "const", "anyOf", "oneOf", "allOf", "not", "if", "then", "else",
    "$ref", "$defs", "definitions", "dependencies", "dependentRequired", "dependentSchemas", "propertyNames",
    "patternProperties", "minProperties", "maxProperties", "exclusiveMinimum", "exclusiveMaximum", "multipleOf",
    "uniqueItems", "contains", "prefixItems", "additionalItems", "unevaluatedProperties",
}
IGNORED = {"title", "description", "$schema", "$id", "default", "examples", "$comment"}


class SchemaError(ValueError):
    """The schema uses something the automaton cannot enforce."""


_declared = False


def _L():
    global _declared
    L = _lib.host()
    if not _declared:
        L.sfb_cst_schema_new.restype = c_void_p
        L.sfb_cst_schema_free.argtypes = [c_void_p]
        L.sfb_cst_node.argtypes = [c_void_p, c_int]
        L.sfb_cst_add_prop.argtypes = [c_void_p, c_int, c_char_p, c_int, c_int, c_int]
        L.sfb_cst_add_option.argtypes = [c_void_p, c_int, c_char_p, c_int]
        L.sfb_cst_set_items.argtypes = [c_void_p, c_int, c_int, c_int, c_int]
        L.sfb_cst_set_bounds.argtypes = [c_void_p, c_int, c_char_p, c_char_p]
        L.sfb_cst_finish.argtypes = [c_void_p, c_int]
        L.sfb_cst_state_new.restype = c_void_p; L.sfb_cst_state_new.argtypes = [c_void_p]
        L.sfb_cst_state_clone.restype = c_void_p; L.sfb_cst_state_clone.argtypes = [c_void_p]
        L.sfb_cst_state_free.argtypes = [c_void_p]
        L.sfb_cst_allowed.argtypes = [c_void_p, c_void_p]
        L.sfb_cst_feed.argtypes = [c_void_p, c_int]
        L.sfb_cst_can_end.argtypes = [c_void_p]
        L.sfb_cst_dead.argtypes = [c_void_p]
        L.sfb_vocab_new.restype = c_void_p; L.sfb_vocab_new.argtypes = [c_int]
        L.sfb_vocab_free.argtypes = [c_void_p]
        L.sfb_vocab_set.argtypes = [c_void_p, c_int, c_char_p, c_int]
        L.sfb_cst_admits.argtypes = [c_void_p, c_void_p, c_int]
        L.sfb_cst_token_mask.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        L.sfb_cst_advance.argtypes = [c_void_p, c_void_p, c_int]
        _declared = True
    return L


def _spell(s: str) -> bytes:
    return json.dumps(s, ensure_ascii=False).encode("utf-8")


def _dec(v) -> bytes:
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise SchemaError("bounds must be numbers")
    d = Decimal(repr(v)) if isinstance(v, float) else Decimal(v)
    return format(d, "f").encode()


class Schema:
    """A compiled schema.  ``Schema.json_object()`` is the open object ``response_format: json_object`` asks for."""

    def __init__(self, schema: dict):
        L = _L()
        self._h = c_void_p(L.sfb_cst_schema_new())
        root = self._compile(schema, "$")
        L.sfb_cst_finish(self._h, root)

    @classmethod
    def json_object(cls) -> "Schema":
        return cls({"type": "object"})

    def __del__(self):
        try:
            _L().sfb_cst_schema_free(self._h)
        except Exception:
            pass

    def _compile(self, sc, path: str) -> int:
        L = _L()
        if sc is True or sc == {}:
            raise SchemaError(f"{path}: a schema that implies no type is refused")
        if not isinstance(sc, dict):
            raise SchemaError(f"{path}: schema must be an object")
        for k in sc:
            if k in REFUSED:
                raise SchemaError(f"{path}: keyword {k!r} is not enforced and therefore refused")
        known = {"type", "properties", "required", "additionalProperties", "items", "minItems", "maxItems", "enum",
                 "minimum", "maximum"} | IGNORED
        for k in sc:
            if k not in known:
                raise SchemaError(f"{path}: unknown keyword {k!r}")
        t = sc.get("type")
        if isinstance(t, list):
            raise SchemaError(f"{path}: a union type needs choice-state masking and is refused")
        if t is None:
            if "properties" in sc or "required" in sc or "additionalProperties" in sc:
                t = "object"
            elif "items" in sc or "minItems" in sc or "maxItems" in sc:
                t = "array"
            elif "enum" in sc and all(isinstance(e, str) for e in sc["enum"]):
                t = "string"
            else:
                raise SchemaError(f"{path}: a schema that implies no type is refused")
        if "enum" in sc and t != "string":
            raise SchemaError(f"{path}: enum is enforced on strings only")
        if t == "object":
            props = sc.get("properties", {})
            req = sc.get("required", [])
            ap = sc.get("additionalProperties")
            if ap is True or isinstance(ap, dict):
                raise SchemaError(f"{path}: additionalProperties other than false is refused")
            if not props and not req and ap is None:
                return L.sfb_cst_node(self._h, T_OPEN_OBJECT)
            for r in req:
                if r not in props:
                    raise SchemaError(f"{path}: required key {r!r} has no schema")
            node = L.sfb_cst_node(self._h, T_OBJECT)
            for name, sub in props.items():
                child = self._compile(sub, f"{path}.{name}")
                b = _spell(name)
                if L.sfb_cst_add_prop(self._h, node, b, len(b), child, int(name in req)):
                    raise SchemaError(f"{path}: more than 63 properties")
            return node
        if t == "array":
            if "items" not in sc:
                raise SchemaError(f"{path}: arrays need items")
            child = self._compile(sc["items"], f"{path}[]")
            node = L.sfb_cst_node(self._h, T_ARRAY)
            mn, mx = int(sc.get("minItems", 0)), int(sc.get("maxItems", -1))
            if mx >= 0 and mn > mx:
                raise SchemaError(f"{path}: minItems above maxItems")
            L.sfb_cst_set_items(self._h, node, child, mn, mx)
            return node
        if t == "string":
            if "enum" in sc:
                if not sc["enum"] or not all(isinstance(e, str) for e in sc["enum"]):
                    raise SchemaError(f"{path}: enum needs string values")
                node = L.sfb_cst_node(self._h, T_ENUM)
                for e in sc["enum"]:
                    b = _spell(e)
                    if L.sfb_cst_add_option(self._h, node, b, len(b)):
                        raise SchemaError(f"{path}: more than 63 enum values")
                return node
            return L.sfb_cst_node(self._h, T_STRING)
        if t in ("integer", "number"):
            node = L.sfb_cst_node(self._h, T_INTEGER if t == "integer" else T_NUMBER)
            mn = _dec(sc["minimum"]) if "minimum" in sc else b""
            mx = _dec(sc["maximum"]) if "maximum" in sc else b""
            if (mn or mx) and L.sfb_cst_set_bounds(self._h, node, mn, mx):
                raise SchemaError(f"{path}: the range holds no value of the type (or is finer than 1e-9)")
            return node
        if t == "boolean":
            return L.sfb_cst_node(self._h, T_BOOLEAN)
        if t == "null":
            return L.sfb_cst_node(self._h, T_NULL)
        raise SchemaError(f"{path}: unknown type {t!r}")


class ByteConstraint:
    """One partially generated document."""

    def __init__(self, schema: Schema, _state=None):
        self.schema = schema
        self._s = c_void_p(_state if _state is not None else _L().sfb_cst_state_new(schema._h))

    def __del__(self):
        try:
            _L().sfb_cst_state_free(self._s)
        except Exception:
            pass

    def clone(self) -> "ByteConstraint":
        return type(self)(self.schema, _L().sfb_cst_state_clone(self._s))

    def allowed_bytes(self) -> set[int]:
        out = (ctypes.c_uint64 * 4)()
        _L().sfb_cst_allowed(self._s, out)
        return {b for b in range(256) if (out[b >> 6] >> (b & 63)) & 1}

    def feed(self, data: bytes) -> bool:
        L = _L()
        for b in data:
            if not L.sfb_cst_feed(self._s, b):
                return False
        return True

    @property
    def can_end(self) -> bool:
        return bool(_L().sfb_cst_can_end(self._s))

    @property
    def dead(self) -> bool:
        return bool(_L().sfb_cst_dead(self._s))


class TokenVocab:
    """Byte strings of every vocabulary id, indexed by first byte on the C++ side."""

    def __init__(self, token_bytes: list[bytes]):
        L = _L()
        self.n = len(token_bytes)
        self._h = c_void_p(L.sfb_vocab_new(self.n))
        for i, b in enumerate(token_bytes):
            L.sfb_vocab_set(self._h, i, b, len(b))

    def __del__(self):
        try:
            _L().sfb_vocab_free(self._h)
        except Exception:
            pass


class TokenConstraint(ByteConstraint):
    """The automaton driven by vocabulary ids (one per constrained sequence on every rank)."""

    def __init__(self, schema: Schema, vocab: TokenVocab | None = None, eos_id: int = -1, _state=None):
        super().__init__(schema, _state)
        self.vocab, self.eos_id = vocab, eos_id

    def clone(self) -> "TokenConstraint":
        return TokenConstraint(self.schema, self.vocab, self.eos_id, _L().sfb_cst_state_clone(self._s))

    def admits(self, token_id: int) -> bool:
        if token_id == self.eos_id:
            return self.can_end
        return bool(_L().sfb_cst_admits(self._s, self.vocab._h, token_id))

    def mask(self, lo: int = 0, hi: int | None = None):
        """(admitted count, uint64 words) for ids [lo, hi): the vocabulary slice of one rank."""
        import numpy as np
        hi = self.vocab.n if hi is None else hi
        words = np.zeros(((hi - lo + 63) // 64,), dtype=np.uint64)
        n = _L().sfb_cst_token_mask(self._s, self.vocab._h, lo, hi, self.eos_id, words.ctypes.data_as(c_void_p))
        return n, words

    def allowed_ids(self, lo: int = 0, hi: int | None = None) -> list[int]:
        import numpy as np
        n, words = self.mask(lo, hi)
        bits = np.unpackbits(words.view(np.uint8), bitorder="little")
        return (np.nonzero(bits)[0] + lo).tolist()

    def advance(self, token_id: int) -> bool:
        if token_id == self.eos_id:
            return self.can_end
        return bool(_L().sfb_cst_advance(self._s, self.vocab._h, token_id))
