"""Evidence artefacts of a run: the run header (what exactly ran), logits dumps for the numerics gates, and per-step
timing records.

A number without its provenance cannot be compared later: the header names the arm, the collective path, the build (a
digest of the native sources), the configuration digest, the GPUs and the NCCL environment, and is written beside every
dump and benchmark record.

Reference: crates/sparkflash-deepseek-forward/src/run_header.rs (arm / collective path / NCCL env), logits_dump.rs (D40),
chain_timing.rs (timing JSON), tp4_token.rs (token envelopes).
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
import time
from pathlib import Path

import torch

_PKG = Path(__file__).resolve().parent.parent


def build_id() -> str:
    """Digest of the native sources (what the shared libraries were built from)."""
    h = hashlib.sha256()
    for f in sorted((_PKG / "csrc").glob("*")):
        if f.suffix in (".cu", ".cuh", ".cpp", ".h"):
            h.update(f.name.encode()); h.update(f.read_bytes())
    return h.hexdigest()[:16]


def run_header(engine=None, settings=None, extra: dict | None = None) -> dict:
    hdr = {"framework": "sparkflash_b200", "build_id": build_id(), "time_unix": int(time.time()),
           "torch": torch.__version__, "cuda": torch.version.cuda,
           "nccl_env": {k: v for k, v in os.environ.items() if k.startswith("NCCL_")},
           "sfb_env": {k: v for k, v in os.environ.items() if k.startswith("SFB_") and "KEY" not in k and "TOKEN" not in k}}
    if torch.cuda.is_available():
        p = torch.cuda.get_device_properties(torch.cuda.current_device())
        hdr["gpu"] = {"name": p.name, "sms": p.multi_processor_count, "memory_gb": round(p.total_memory / 1e9, 1),
                      "capability": f"{p.major}.{p.minor}"}
    if engine is not None:
        comm = getattr(engine, "comm", None)
        hdr["engine"] = {"arm": getattr(engine, "arm", None), "world": getattr(engine, "world", 1), "rank": getattr(engine, "rank", 0),
                         "max_rows": getattr(engine, "max_rows", None), "max_lanes": getattr(engine, "max_lanes", None),
                         "collective": getattr(comm, "name", "none") if comm is not None else "none",
                         "cuda_graphs": getattr(engine, "use_graphs", None),
                         "moe_mode": getattr(getattr(engine, "w", None), "moe_mode", None),
                         "model": getattr(getattr(engine, "cfg", None), "name", None)}
    if settings is not None and hasattr(settings, "digest"):
        hdr["settings_digest"] = settings.digest()
    if extra:
        hdr.update(extra)
    return hdr


MAGIC = b"SFBLOGIT"


class LogitsDump:
    """Append-only binary dump of fp32 logits rows: ``MAGIC | u32 header length | header JSON`` then records of
    ``i64 step | i32 row | i32 position | i32 n | n x f32``.  Read back with ``read``."""

    def __init__(self, path: str, header: dict):
        self.f = open(path, "wb")
        h = json.dumps(header).encode()
        self.f.write(MAGIC + struct.pack("<I", len(h)) + h)
        self.records = 0

    def add(self, step: int, row: int, position: int, logits: torch.Tensor) -> None:
        v = logits.detach().float().cpu().contiguous()
        self.f.write(struct.pack("<qiii", step, row, position, v.numel()) + v.numpy().tobytes())
        self.records += 1

    def close(self) -> None:
        self.f.close()

    @staticmethod
    def read(path: str):
        b = Path(path).read_bytes()
        if b[:8] != MAGIC:
            raise ValueError("not a logits dump")
        hl = struct.unpack("<I", b[8:12])[0]
        header = json.loads(b[12:12 + hl])
        p, recs = 12 + hl, []
        while p < len(b):
            step, row, pos, n = struct.unpack("<qiii", b[p:p + 20])
            p += 20
            recs.append((step, row, pos, torch.frombuffer(bytearray(b[p:p + 4 * n]), dtype=torch.float32)))
            p += 4 * n
        return header, recs


def compare_dumps(a: str, b: str) -> dict:
    """Position-by-position comparison of two dumps of the same forced token sequence: the bars of the served numerics gate."""
    _, ra = LogitsDump.read(a)
    _, rb = LogitsDump.read(b)
    if len(ra) != len(rb):
        raise ValueError(f"dumps hold {len(ra)} and {len(rb)} records")
    max_abs = mean_abs = kl = 0.0
    top1 = 0
    for (sa, wa, pa, la), (sb, wb, pb, lb) in zip(ra, rb):
        if (sa, wa, pa) != (sb, wb, pb) or la.numel() != lb.numel():
            raise ValueError(f"record mismatch at step {sa}/{sb}")
        d = (la - lb).abs()
        max_abs = max(max_abs, float(d.max())); mean_abs += float(d.mean())
        pa_, pb_ = torch.log_softmax(la, 0), torch.log_softmax(lb, 0)
        kl += float((pa_.exp() * (pa_ - pb_)).sum())
        top1 += int(la.argmax()) == int(lb.argmax())
    n = max(1, len(ra))
    return {"records": len(ra), "max_abs": max_abs, "mean_abs": mean_abs / n, "kl": kl / n, "top1": top1 / n}


class TimingLog:
    """Per-step timing records as JSON lines (step, rows, device ms, host ms), with the run header first."""

    def __init__(self, path: str, header: dict):
        self.f = open(path, "w")
        self.f.write(json.dumps({"header": header}) + "\n")

    def add(self, step: int, rows: int, device_ms: float, host_ms: float | None = None, **kw) -> None:
        self.f.write(json.dumps({"step": step, "rows": rows, "device_ms": device_ms, "host_ms": host_ms, **kw}) + "\n")

    def close(self) -> None:
        self.f.close()
