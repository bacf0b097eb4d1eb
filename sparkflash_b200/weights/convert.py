"""Offline conversion: a checkpoint directory (``config.json`` + ``*.safetensors``) -> one prepared file per
rank plus a manifest.  Reference: crates/sparkflash-cli/src/convert.rs:15-76 (options: world size, ranks,
verify, inspect), crates/sparkflash-device/src/converted.rs (convert_checkpoint / verify / inspect).
"""
from __future__ import annotations

import json
import os
import time

from ..config import config_from_hf
from . import files as F

MANIFEST = "manifest.json"


def rank_path(out_dir: str, rank: int, world: int) -> str:
    return os.path.join(out_dir, f"rank{rank}-of-{world}.sfb")


def convert(src_dir: str, out_dir: str, world: int = 1, ranks: list[int] | None = None, verify: bool = True,
            progress=None, moe_mode: str = "tp") -> dict:
    from ..models.deepseek_v41 import prepare as P
    with open(os.path.join(src_dir, "config.json")) as f:
        cfg = config_from_hf(json.load(f))
    ck, keep = F.load_checkpoint_dir(src_dir)
    os.makedirs(out_dir, exist_ok=True)
    ranks = list(range(world)) if ranks is None else ranks
    man_path = os.path.join(out_dir, MANIFEST)
    manifest = {"format": 1, "model": cfg.name, "world": world, "moe_mode": moe_mode, "source": os.path.abspath(src_dir), "ranks": {}}
    if os.path.exists(man_path):
        with open(man_path) as f:
            old = json.load(f)
        if old.get("world") == world:
            manifest["ranks"] = old.get("ranks", {})
    for i, r in enumerate(ranks):
        t0 = time.time()
        w = P.prepare_from_checkpoint(ck, cfg, r, world, device="cpu", moe_mode=moe_mode)
        path = rank_path(out_dir, r, world)
        info = F.write_rank_file(path, w, {"source": os.path.basename(os.path.abspath(src_dir))})
        if verify:
            F.load_rank_file(path, device="cpu", verify=True, expect_rank=r, expect_world=world)
        manifest["ranks"][str(r)] = {"file": os.path.basename(path), "bytes": os.path.getsize(path), "tensors": info["tensors"],
                                     "seconds": round(time.time() - t0, 3), "verified": bool(verify)}
        if progress:
            progress(i + 1, len(ranks), os.path.basename(path))
    with open(man_path, "w") as f:
        json.dump(manifest, f, indent=1)
    for k in keep:
        k.close()
    return manifest


def inspect(path: str, verify_weights: bool = False) -> dict:
    w = F.load_rank_file(path, device="cpu", verify=verify_weights)
    tensors, scalars = F._flatten(w)
    return {"rank": w.rank, "world": w.world, "model": w.cfg.name, "tensors": len(tensors),
            "bytes": sum(t.numel() * t.element_size() for t in tensors.values()), "verified": verify_weights,
            "largest": sorted(((t.numel() * t.element_size(), n) for n, t in tensors.items()), reverse=True)[:5]}


def export_synthetic_checkpoint(out_dir: str, cfg, seed: int = 0, shard_bytes: int = 1 << 30) -> None:
    """Write a synthetic checkpoint in the released layout (config.json + shards): the input of ``convert`` in
    tests and on machines without the released weights."""
    from ..config import config_to_hf
    from ..models.deepseek_v41 import weights as W
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(config_to_hf(cfg), f, indent=1)
    ck = W.synthetic_checkpoint(cfg, seed)
    shard, size, idx = {}, 0, 0
    for name, t in ck.items():
        shard[name] = t
        size += t.numel() * t.element_size()
        if size >= shard_bytes:
            F.write_safetensors(os.path.join(out_dir, f"model-{idx:05d}.safetensors"), shard); shard, size, idx = {}, 0, idx + 1
    if shard:
        F.write_safetensors(os.path.join(out_dir, f"model-{idx:05d}.safetensors"), shard)
