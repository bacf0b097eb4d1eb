"""Engram tables: packing into per-rank shard files, loading a shard (device memory, or pinned host memory
the GPU reads in place), lookups and the gated residual.

B200 placement: the two tables are 188.8 GiB of FP8 rows.  With 8 ranks a row-range shard is 23.6 GiB per GPU
and lives in HBM; with fewer ranks the shard stays in pinned host memory mapped into the device address
space, and the gather kernel reads the 24 rows per token over PCIe.  Either way the kernel sees one pointer.
Reference: crates/sparkflash-engram/src/{packer,paged,store}.rs, docs/architecture/04-engram.md section 7
(row sharding, tail padded with weight 0 / scale 1, out-of-range rows contribute zeros and the ranks' partial
lookups are summed).
"""
from __future__ import annotations

import ctypes
import json
import os
from ctypes import c_float, c_int, c_int64, c_longlong, c_void_p

import numpy as np
import torch

from .. import _lib
from ..codecs import e4m3_decode, ue8m0_decode
from .layout import _L as _host

STRIDE = 272          # 256 e4m3 + 8 ue8m0 + 8 pad: 16-byte aligned rows
MANIFEST = "engram_manifest.json"


def shard_range(rows: int, rank: int, world: int) -> tuple[int, int]:
    per = -(-rows // world)
    return rank * per, per


def pack_table(weight: torch.Tensor, scale: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """uint8 [per, STRIDE] shard of one table (weight uint8 [rows, width], scale uint8 [rows, width/32])."""
    rows, width = weight.shape
    first, per = shard_range(rows, rank, world)
    out = torch.empty((per, STRIDE), dtype=torch.uint8)
    w, s = weight.contiguous(), scale.contiguous()
    rc = _host().sfb_engram_pack(c_void_p(w.data_ptr()), c_void_p(s.data_ptr()), rows, width, first, per, c_void_p(out.data_ptr()), STRIDE)
    if rc:
        raise ValueError("row stride too small for the row")
    return out


def pack(source_dir: str, out_dir: str, world: int = 1, dry_run: bool = False) -> dict:
    """``pack-engram``: read ``engram.{layer}.embed.weight|scale`` from the checkpoint shards under ``source_dir``
    and write ``engram-L{layer}-rank{r}-of-{world}.bin`` files plus a manifest."""
    from ..weights.files import load_checkpoint_dir
    ck, keep = load_checkpoint_dir(source_dir)
    layers = sorted({int(n.split(".")[1]) for n in ck if n.startswith("engram.") and n.endswith(".embed.weight")})
    rep = {"files": [], "bytes": 0, "layers": layers, "world": world, "stride": STRIDE, "rows": {}}
    os.makedirs(out_dir, exist_ok=True)
    for l in layers:
        w, s = ck[f"engram.{l}.embed.weight"], ck[f"engram.{l}.embed.scale"]
        rep["rows"][str(l)] = int(w.shape[0])
        for r in range(world):
            name = f"engram-L{l}-rank{r}-of-{world}.bin"
            first, per = shard_range(w.shape[0], r, world)
            rep["files"].append(name)
            rep["bytes"] += per * STRIDE
            if not dry_run:
                pack_table(w, s, r, world).numpy().tofile(os.path.join(out_dir, name))
    if not dry_run:
        with open(os.path.join(out_dir, MANIFEST), "w") as f:
            json.dump(rep, f, indent=1)
    for k in keep:
        k.close()
    return rep


class EngramShard:
    """One rank's rows of one layer's table."""

    def __init__(self, packed: torch.Tensor, rows_total: int, rank: int, world: int, device="cuda", resident: bool = True):
        self.first, self.per = shard_range(rows_total, rank, world)
        assert packed.shape == (self.per, STRIDE)
        self.width = 256
        dev = torch.device(device)
        if dev.type == "cuda" and not resident:
            self.host = packed.pin_memory()                # the kernel reads it in place through the mapped address
            self.data = self.host
            self.ptr = self.host.data_ptr()                # pinned memory is addressable from the device (UVA)
        else:
            self.data = packed.to(dev)
            self.ptr = self.data.data_ptr()
        self.lookups = 0

    @classmethod
    def from_file(cls, path: str, rows_total: int, rank: int, world: int, **kw) -> "EngramShard":
        per = shard_range(rows_total, rank, world)[1]
        arr = np.fromfile(path, dtype=np.uint8).reshape(per, STRIDE)
        return cls(torch.from_numpy(arr), rows_total, rank, world, **kw)

    def gather(self, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """ids int64 [n, cols] (device) -> bf16 [n, cols*width]; rows outside this shard give zeros."""
        n, cols = ids.shape
        if out is None:
            out = torch.empty((n, cols * self.width), dtype=torch.bfloat16, device=ids.device)
        self.lookups += n * cols
        if ids.device.type == "cuda":
            from ..ops import native as N
            rc = _lib.cuda().sfb_engram_gather(c_void_p(self.ptr), c_longlong(self.first), c_longlong(self.per), c_int(STRIDE),
                                               N._p(ids), c_int(n), c_int(cols), c_int(self.width), N._p(out), N._stream())
            N._check(rc, "engram_gather")
            return out
        out.copy_(gather_reference(self.data, self.first, ids).to(torch.bfloat16))
        return out


def gather_reference(packed: torch.Tensor, first: int, ids: torch.Tensor) -> torch.Tensor:
    """fp32 [n, cols*256]: dequantised rows; ids outside [first, first+per) give zeros."""
    per = packed.shape[0]
    loc = ids - first
    ok = (loc >= 0) & (loc < per)
    rows = packed[loc.clamp(0, per - 1).reshape(-1)]
    w = e4m3_decode(rows[:, :256]).reshape(-1, 8, 32)
    s = ue8m0_decode(rows[:, 256:264]).reshape(-1, 8, 1)
    v = (w * s).reshape(ids.shape[0], ids.shape[1], 256) * ok.unsqueeze(-1)
    return v.reshape(ids.shape[0], -1)


def gate_reference(h: torch.Tensor, kv: torch.Tensor, w: torch.Tensor, token_mask: torch.Tensor | None, eps: float) -> torch.Tensor:
    """h fp32 [n, hc, d]; kv [n, (hc+1)*d]; w = q_weight*k_weight fp32 [hc, d] -> new h."""
    n, hc, d = h.shape
    kv = kv.float()
    key, value = kv[:, :hc * d].reshape(n, hc, d), kv[:, hc * d:]
    rstd = torch.rsqrt(h.pow(2).mean(-1) + eps) * torch.rsqrt(key.pow(2).mean(-1) + eps)
    dot = (h * w * key).sum(-1) * rstd * d ** -0.5
    gate = torch.sigmoid(torch.copysign(torch.sqrt(dot.abs().clamp_min(1e-6)), dot))
    if token_mask is not None:
        gate = gate * token_mask.reshape(n, 1).to(gate.dtype)
    return h + gate.unsqueeze(-1) * value.unsqueeze(1)


def gate(h: torch.Tensor, kv: torch.Tensor, w: torch.Tensor, token_mask: torch.Tensor | None, eps: float) -> None:
    """In place on the device."""
    from ..ops import native as N
    n, hc, d = h.shape
    rc = _lib.cuda().sfb_engram_gate(N._p(h), N._p(kv), N._p(w), N._p(token_mask) if token_mask is not None else None,
                                     c_int(n), c_int(hc), c_int(d), c_float(eps), N._stream())
    N._check(rc, "engram_gate")
