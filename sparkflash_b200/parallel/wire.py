"""Binary encoding of control-channel messages: plain data only, nothing executable.

A tick carries numbers, strings, byte strings, lists, tuples, dicts, tensors (vision embeddings) and a
small closed set of record types (requests, vision spans).  The decoder builds exactly those and
refuses everything else, so a frame from an untrusted peer can at worst be rejected - unlike an
unpickler, it never imports a module or calls a constructor that the table below does not name.

Layout: one tag byte, then a tag-specific body; lengths and counts are little-endian u32, integers
i64 (larger ones as decimal text), floats f64.  Tensors travel as dtype name, shape and raw bytes.

Reference: crates/sparkflash-comm/src/control.rs:64 (fixed binary frames Hello/Ready/Request/Token/End/
Error/DeviceTick/DevicePixels).
"""
from __future__ import annotations

import dataclasses
import struct

import torch

_NONE, _TRUE, _FALSE, _INT, _BIGINT, _FLOAT, _STR, _BYTES, _LIST, _TUPLE, _DICT, _TENSOR, _RECORD = range(13)

_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "uint8": torch.uint8,
           "int8": torch.int8, "int32": torch.int32, "int64": torch.int64, "bool": torch.bool, "float64": torch.float64}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}

MAX_DEPTH = 32
MAX_ITEMS = 1 << 24

_records: dict[str, type] = {}


class WireError(ValueError):
    pass


def register(cls: type) -> type:
    """Allow instances of dataclass ``cls`` on the wire (encoded as its name plus its fields)."""
    if not dataclasses.is_dataclass(cls):
        raise TypeError(f"{cls!r} is not a dataclass")
    _records[cls.__name__] = cls
    return cls


def _register_defaults() -> None:
    from ..serve.engine_api import EngineRequest
    register(EngineRequest)
    try:
        from ..serve.vision_glue import VisionSpan
        register(VisionSpan)
    except Exception:      # the vision front end needs optional image codecs; ticks without images do not
        pass


def _enc(o, out: list, depth: int) -> None:
    if depth > MAX_DEPTH:
        raise WireError("message nests too deeply")
    if o is None:
        out.append(bytes([_NONE]))
    elif o is True:
        out.append(bytes([_TRUE]))
    elif o is False:
        out.append(bytes([_FALSE]))
    elif isinstance(o, int):
        if -(1 << 63) <= o < (1 << 63):
            out.append(struct.pack("<Bq", _INT, o))
        else:
            s = str(o).encode()
            out.append(struct.pack("<BI", _BIGINT, len(s)) + s)
    elif isinstance(o, float):
        out.append(struct.pack("<Bd", _FLOAT, o))
    elif isinstance(o, str):
        s = o.encode("utf-8")
        out.append(struct.pack("<BI", _STR, len(s)) + s)
    elif isinstance(o, (bytes, bytearray, memoryview)):
        b = bytes(o)
        out.append(struct.pack("<BI", _BYTES, len(b)) + b)
    elif isinstance(o, (list, tuple)):
        out.append(struct.pack("<BI", _LIST if isinstance(o, list) else _TUPLE, len(o)))
        for x in o:
            _enc(x, out, depth + 1)
    elif isinstance(o, dict):
        out.append(struct.pack("<BI", _DICT, len(o)))
        for k, v in o.items():
            _enc(k, out, depth + 1)
            _enc(v, out, depth + 1)
    elif isinstance(o, torch.Tensor):
        t = o.detach().to("cpu").contiguous()
        name = _DTYPE_NAMES.get(t.dtype)
        if name is None:
            raise WireError(f"tensor dtype {t.dtype} does not travel")
        nb = name.encode()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        out.append(struct.pack("<BB", _TENSOR, len(nb)) + nb + struct.pack("<B", t.dim()) +
                   struct.pack(f"<{t.dim()}q", *t.shape) + struct.pack("<Q", len(raw)) + raw)
    elif dataclasses.is_dataclass(o) and not isinstance(o, type):
        name = type(o).__name__
        if _records.get(name) is not type(o):
            if not _records:
                _register_defaults()
            if _records.get(name) is not type(o):
                raise WireError(f"record type {name} is not registered for the control channel")
        fields = dataclasses.fields(o)
        nb = name.encode()
        out.append(struct.pack("<BB", _RECORD, len(nb)) + nb + struct.pack("<I", len(fields)))
        for f in fields:
            _enc(f.name, out, depth + 1)
            _enc(getattr(o, f.name), out, depth + 1)
    else:
        try:                       # numpy scalars and the like
            import numpy as np
            if isinstance(o, np.integer):
                return _enc(int(o), out, depth)
            if isinstance(o, np.floating):
                return _enc(float(o), out, depth)
            if isinstance(o, np.ndarray):
                return _enc(torch.from_numpy(np.ascontiguousarray(o)), out, depth)
        except ImportError:
            pass
        raise WireError(f"{type(o).__name__} does not travel on the control channel")


def dumps(o) -> bytes:
    out: list = []
    _enc(o, out, 0)
    return b"".join(out)


class _R:
    def __init__(self, b: bytes):
        self.b, self.p = memoryview(b), 0

    def take(self, n: int) -> memoryview:
        if n < 0 or self.p + n > len(self.b):
            raise WireError("truncated frame")
        v = self.b[self.p:self.p + n]
        self.p += n
        return v

    def unpack(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))


def _dec(r: _R, depth: int):
    if depth > MAX_DEPTH:
        raise WireError("message nests too deeply")
    tag = r.unpack("<B")[0]
    if tag == _NONE:
        return None
    if tag == _TRUE:
        return True
    if tag == _FALSE:
        return False
    if tag == _INT:
        return r.unpack("<q")[0]
    if tag == _BIGINT:
        s = bytes(r.take(r.unpack("<I")[0]))
        if len(s) > 128 or not s.lstrip(b"-").isdigit():
            raise WireError("bad integer")
        return int(s)
    if tag == _FLOAT:
        return r.unpack("<d")[0]
    if tag == _STR:
        return bytes(r.take(r.unpack("<I")[0])).decode("utf-8")
    if tag == _BYTES:
        return bytes(r.take(r.unpack("<I")[0]))
    if tag in (_LIST, _TUPLE):
        n = r.unpack("<I")[0]
        if n > MAX_ITEMS:
            raise WireError("sequence too long")
        items = [_dec(r, depth + 1) for _ in range(n)]
        return items if tag == _LIST else tuple(items)
    if tag == _DICT:
        n = r.unpack("<I")[0]
        if n > MAX_ITEMS:
            raise WireError("mapping too long")
        d = {}
        for _ in range(n):
            k = _dec(r, depth + 1)
            if not isinstance(k, (str, int, bool, float, bytes, tuple, type(None))):
                raise WireError("unhashable mapping key")
            d[k] = _dec(r, depth + 1)
        return d
    if tag == _TENSOR:
        name = bytes(r.take(r.unpack("<B")[0])).decode()
        dt = _DTYPES.get(name)
        if dt is None:
            raise WireError(f"unknown tensor dtype {name!r}")
        nd = r.unpack("<B")[0]
        if nd > 8:
            raise WireError("tensor rank too high")
        shape = list(r.unpack(f"<{nd}q")) if nd else []
        nbytes = r.unpack("<Q")[0]
        numel = 1
        for s in shape:
            if s < 0:
                raise WireError("negative tensor extent")
            numel *= s
        if numel * torch.empty((), dtype=dt).element_size() != nbytes:
            raise WireError("tensor bytes do not match its shape")
        raw = bytes(r.take(nbytes))
        if not numel:
            return torch.empty(shape, dtype=dt)
        return torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dt).reshape(shape)
    if tag == _RECORD:
        name = bytes(r.take(r.unpack("<B")[0])).decode()
        if not _records:
            _register_defaults()
        cls = _records.get(name)
        if cls is None:
            raise WireError(f"record type {name!r} is not registered for the control channel")
        n = r.unpack("<I")[0]
        known = {f.name for f in dataclasses.fields(cls)}
        kw = {}
        for _ in range(n):
            k = _dec(r, depth + 1)
            v = _dec(r, depth + 1)
            if k not in known:
                raise WireError(f"{name} has no field {k!r}")
            kw[k] = v
        return cls(**kw)
    raise WireError(f"unknown tag {tag}")


def loads(b: bytes):
    r = _R(b)
    o = _dec(r, 0)
    if r.p != len(r.b):
        raise WireError("trailing bytes after the message")
    return o
