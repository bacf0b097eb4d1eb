"""Weight files: safetensors checkpoints in, per-rank prepared files out and back (csrc/host_weights.cpp).

``SafeTensorsFile`` gives zero-copy torch views of a memory-mapped checkpoint shard.  ``write_rank_file`` /
``load_rank_file`` store a prepared ``DeviceWeights`` (every tensor already sliced for one rank and in the
layout the kernels read) with a digest per tensor; loading is a handful of large parallel reads into pinned
memory followed by one device copy per tensor.  Reference: crates/sparkflash-weights/src/rank_file.rs:15-37,
crates/sparkflash-device/src/converted.rs:15-42, crates/sparkflash-cli/src/convert.rs:15-76.
"""
from __future__ import annotations

import ctypes
import dataclasses
import json
import os
from ctypes import c_char_p, c_int, c_int64, c_uint64, c_void_p

import torch

from .. import _lib

_DT = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "U8": torch.uint8, "I8": torch.int8,
       "I32": torch.int32, "I64": torch.int64, "F8_E4M3": torch.uint8, "F8_E8M0": torch.uint8, "F4": torch.uint8,
       "BOOL": torch.bool, "F64": torch.float64, "I16": torch.int16, "U16": torch.uint16}
_NAME = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.uint8: "U8", torch.int8: "I8",
         torch.int32: "I32", torch.int64: "I64", torch.bool: "BOOL", torch.float64: "F64", torch.int16: "I16"}
_declared = False


def _L():
    global _declared
    L = _lib.host()
    if not _declared:
        L.sfb_weights_last_error.restype = c_char_p
        L.sfb_digest64.restype = c_uint64; L.sfb_digest64.argtypes = [c_void_p, c_uint64]
        L.sfb_st_open.restype = c_void_p; L.sfb_st_open.argtypes = [c_char_p]
        L.sfb_st_close.argtypes = [c_void_p]
        L.sfb_st_count.argtypes = [c_void_p]
        for f in ("sfb_st_name", "sfb_st_dtype", "sfb_rank_name", "sfb_rank_dtype"):
            getattr(L, f).restype = c_char_p; getattr(L, f).argtypes = [c_void_p, c_int]
        L.sfb_st_shape.argtypes = [c_void_p, c_int, c_void_p]
        L.sfb_st_data.restype = c_void_p; L.sfb_st_data.argtypes = [c_void_p, c_int, c_void_p]
        L.sfb_rank_writer_open.restype = c_void_p; L.sfb_rank_writer_open.argtypes = [c_char_p]
        L.sfb_rank_writer_add.argtypes = [c_void_p, c_char_p, c_char_p, c_int, c_void_p, c_void_p, c_uint64]
        L.sfb_rank_writer_close.argtypes = [c_void_p, c_char_p]
        L.sfb_rank_open.restype = c_void_p; L.sfb_rank_open.argtypes = [c_char_p]
        L.sfb_rank_close.argtypes = [c_void_p]
        L.sfb_rank_count.argtypes = [c_void_p]
        L.sfb_rank_meta.restype = c_char_p; L.sfb_rank_meta.argtypes = [c_void_p]
        L.sfb_rank_shape.argtypes = [c_void_p, c_int, c_void_p]
        L.sfb_rank_nbytes.restype = c_uint64; L.sfb_rank_nbytes.argtypes = [c_void_p, c_int]
        L.sfb_rank_read.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int]
        _declared = True
    return L


def _err() -> str:
    return (_L().sfb_weights_last_error() or b"").decode()


def digest64(t: torch.Tensor) -> int:
    t = t.contiguous()
    return int(_L().sfb_digest64(c_void_p(t.data_ptr()), t.numel() * t.element_size()))


class SafeTensorsFile:
    def __init__(self, path: str):
        self._h = _L().sfb_st_open(path.encode())
        if not self._h:
            raise OSError(f"{path}: {_err()}")
        self._h = c_void_p(self._h)
        L = _L()
        self.names = [L.sfb_st_name(self._h, i).decode() for i in range(L.sfb_st_count(self._h))]
        self._index = {n: i for i, n in enumerate(self.names)}

    def close(self):
        if self._h:
            _L().sfb_st_close(self._h)
            self._h = None

    def __contains__(self, name):
        return name in self._index

    def info(self, name: str):
        L = _L()
        i = self._index[name]
        sh = (c_int64 * 8)()
        nd = L.sfb_st_shape(self._h, i, sh)
        return L.sfb_st_dtype(self._h, i).decode(), list(sh[:nd])

    def tensor(self, name: str) -> torch.Tensor:
        """A view of the mapped file (valid while this object lives); sub-byte and 8-bit float types come back as uint8."""
        L = _L()
        i = self._index[name]
        dt, shape = self.info(name)
        nb = c_uint64()
        p = L.sfb_st_data(self._h, i, ctypes.byref(nb))
        if nb.value == 0:
            return torch.empty(shape, dtype=_DT[dt])
        buf = (ctypes.c_uint8 * nb.value).from_address(p)
        flat = torch.frombuffer(buf, dtype=torch.uint8)
        tdt = _DT[dt]
        if dt == "F4" and shape and _prod(shape) == 2 * nb.value:      # two values per byte: the stored last dimension is half the logical one
            shape = shape[:-1] + [shape[-1] // 2]
        return flat.view(tdt).reshape(shape)


def _prod(xs):
    n = 1
    for x in xs:
        n *= x
    return n


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Small writer (tests, synthetic checkpoints): the format is the header length, the JSON table, the data."""
    table, off, blobs = {}, 0, []
    if metadata:
        table["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        table[name] = {"dtype": _NAME[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    head = json.dumps(table, separators=(",", ":")).encode()
    head += b" " * ((8 - len(head) % 8) % 8)
    with open(path, "wb") as f:
        f.write(len(head).to_bytes(8, "little")); f.write(head)
        for b in blobs:
            f.write(b)


def load_checkpoint_dir(path: str) -> tuple[dict[str, torch.Tensor], list[SafeTensorsFile]]:
    """All tensors of every ``*.safetensors`` shard under ``path`` as mapped views (keep the files alive)."""
    files = [SafeTensorsFile(os.path.join(path, f)) for f in sorted(os.listdir(path)) if f.endswith(".safetensors")]
    if not files:
        raise FileNotFoundError(f"no .safetensors shard under {path}")
    out = {}
    for f in files:
        for n in f.names:
            out[n] = f.tensor(n)
    return out, files


# ---- prepared rank files --------------------------------------------------------------------------------------
def _flatten(w) -> tuple[dict[str, torch.Tensor], dict]:
    tensors, scalars = {}, {}
    for f in dataclasses.fields(w):
        v = getattr(w, f.name)
        if f.name in ("cfg", "layers", "mtp_layers"):
            continue
        if isinstance(v, torch.Tensor):
            tensors[f.name] = v
        elif isinstance(v, dict):           # small tables keyed by a flag, e.g. rotary frequencies per layer kind
            for k, t in v.items():
                tensors[f"{f.name}.{int(k)}"] = t
        elif isinstance(v, (int, float, bool, str)) or v is None:
            scalars[f.name] = v
    for group, layers in (("layers", w.layers), ("mtp_layers", getattr(w, "mtp_layers", []))):
        for i, L in enumerate(layers):
            for f in dataclasses.fields(L):
                v = getattr(L, f.name)
                if isinstance(v, torch.Tensor):
                    tensors[f"{group}.{i}.{f.name}"] = v
                elif isinstance(v, (int, float, bool)):
                    scalars[f"{group}.{i}.{f.name}"] = v
    return tensors, scalars


def write_rank_file(path: str, weights, extra_meta: dict | None = None) -> dict:
    """Store a prepared ``DeviceWeights`` (tensors on the CPU).  Returns the table summary."""
    L = _L()
    tensors, scalars = _flatten(weights)
    h = L.sfb_rank_writer_open(path.encode())
    if not h:
        raise OSError(_err())
    h = c_void_p(h)
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        shape = (c_int64 * max(1, t.dim()))(*t.shape)
        if L.sfb_rank_writer_add(h, name.encode(), _NAME[t.dtype].encode(), t.dim(), shape, c_void_p(t.data_ptr()), t.numel() * t.element_size()):
            raise OSError(_err())
    meta = {"format": 1, "rank": weights.rank, "world": weights.world, "config": dataclasses.asdict(weights.cfg),
            "scalars": scalars, **(extra_meta or {})}
    if L.sfb_rank_writer_close(h, json.dumps(meta).encode()):
        raise OSError(_err())
    return {"tensors": len(tensors), "bytes": sum(t.numel() * t.element_size() for t in tensors.values())}


def load_rank_file(path: str, device="cuda", verify: bool = True, threads: int = 16, expect_rank: int | None = None,
                   expect_world: int | None = None):
    """-> DeviceWeights on ``device``.  All payloads land in one pinned staging buffer through parallel reads;
    digests are checked there; then one async copy per tensor."""
    from ..config import ModelConfig
    from ..models.deepseek_v41.prepare import DeviceWeights, LayerW
    L = _L()
    h = L.sfb_rank_open(path.encode())
    if not h:
        raise OSError(f"{path}: {_err()}")
    h = c_void_p(h)
    try:
        meta = json.loads(L.sfb_rank_meta(h).decode())
        if expect_rank is not None and (meta["rank"], meta["world"]) != (expect_rank, expect_world):
            raise ValueError(f"{path} was prepared for rank {meta['rank']}/{meta['world']}, not {expect_rank}/{expect_world}")
        n = L.sfb_rank_count(h)
        offs, total, infos = [], 0, []
        for i in range(n):
            nb = int(L.sfb_rank_nbytes(h, i))
            sh = (c_int64 * 8)()
            nd = L.sfb_rank_shape(h, i, sh)
            infos.append((L.sfb_rank_name(h, i).decode(), L.sfb_rank_dtype(h, i).decode(), list(sh[:nd]), nb))
            offs.append(total)
            total += (nb + 255) // 256 * 256
        on_gpu = torch.device(device).type == "cuda"
        stage = torch.empty((max(total, 1),), dtype=torch.uint8, pin_memory=on_gpu)
        rc = L.sfb_rank_read(h, 0, n, c_void_p(stage.data_ptr()), (c_uint64 * max(1, n))(*offs), threads, int(verify))
        if rc:
            raise OSError(f"{path}: {_err()}")
    finally:
        L.sfb_rank_close(h)
    cfgd = meta["config"]
    cfg = ModelConfig(**{k: (tuple(v) if isinstance(v, list) and k not in _list_fields(ModelConfig) else v) for k, v in cfgd.items()})
    dicts: dict[str, dict] = {}
    tensors = {}
    for (name, dt, shape, nb), off in zip(infos, offs):
        t = stage[off:off + nb].view(_DT[dt]).reshape(shape)
        t = t.to(device, non_blocking=True) if on_gpu else t.clone()
        head, _, tail = name.partition(".")
        if head not in ("layers", "mtp_layers") and tail.isdigit():
            dicts.setdefault(head, {})[bool(int(tail))] = t
        else:
            tensors[name] = t
    if on_gpu:
        torch.cuda.synchronize()
    sc = meta["scalars"]
    groups = {}
    for group in ("layers", "mtp_layers"):
        nl = 1 + max((int(k.split(".")[1]) for k in tensors if k.startswith(group + ".")), default=-1)
        layers = []
        for i in range(nl):
            Lw = LayerW()
            pre = f"{group}.{i}."
            for k, v in tensors.items():
                if k.startswith(pre):
                    setattr(Lw, k[len(pre):], v)
            for k, v in sc.items():
                if k.startswith(pre):
                    setattr(Lw, k[len(pre):], v)
            layers.append(Lw)
        groups[group] = layers
    kw = {f.name: tensors.get(f.name, sc.get(f.name)) for f in dataclasses.fields(DeviceWeights) if f.name not in ("cfg", "layers", "mtp_layers")}
    kw = {k: v for k, v in kw.items() if v is not None or k in ("embed",)}
    kw.update(dicts)
    kw.update(cfg=cfg, **groups)
    return DeviceWeights(**kw)


def _list_fields(cls) -> set[str]:
    out = set()
    for f in dataclasses.fields(cls):
        if "list" in str(f.type):
            out.add(f.name)
    return out
