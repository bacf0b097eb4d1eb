"""Model hub cache: from a model id to a checkpoint directory, listing what a node can serve, and a resumable download
with an injectable fetcher (tests and offline machines pass their own; the default uses urllib).

The cache has the layout ``huggingface_hub`` writes::

    <cache>/models--<org>--<name>/refs/main          commit hash that ``main`` points at
    <cache>/models--<org>--<name>/snapshots/<hash>/  the checkout (symlinks into blobs/ or plain files)
    <cache>/models--<org>--<name>/blobs/             file contents, named by digest

Reference behaviour: crates/sparkflash-web/src/hf.rs (list:144, preferred_cached:181, lookup:215, fit_cached:284,
families:406, search:559, inspect:642), crates/sparkflash-weights/src/hub.rs (cache directory, id to snapshot).
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import urllib.request
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Iterable

from ..config import full_config
from ..models.registry import MODELS
from . import fit

ID_RE = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]*/[A-Za-z0-9][A-Za-z0-9._-]*$")

# config.json ``model_type`` -> the family of the model table that serves it
MODEL_TYPES = {
    "deepseek_v41": "deepseek", "deepseek_v3": "deepseek", "qwen4_exp": "qwen", "qwen4_exp_text": "qwen", "qwen3_5_moe": "qwen",
    "qwen3_5_moe_text": "qwen", "glm5_next": "glm", "dory": "dory", "inkling2": "inkling",
}


def default_cache_dir(env=None) -> Path:
    env = os.environ if env is None else env
    if env.get("HF_HUB_CACHE"):
        return Path(env["HF_HUB_CACHE"])
    if env.get("HF_HOME"):
        return Path(env["HF_HOME"]) / "hub"
    return Path(env.get("HOME", "/root")) / ".cache" / "huggingface" / "hub"


def is_model_id(s: str) -> bool:
    return bool(ID_RE.match(s)) and not os.path.exists(s)


def repo_folder(model_id: str) -> str:
    return "models--" + model_id.replace("/", "--")


def folder_id(folder: str) -> str | None:
    if not folder.startswith("models--"):
        return None
    parts = folder[len("models--"):].split("--")
    return "/".join(parts) if len(parts) == 2 and all(parts) else None


def snapshot_of(repo: Path) -> Path | None:
    """The snapshot ``refs/main`` names, else the most recently modified one."""
    ref = repo / "refs" / "main"
    snaps = repo / "snapshots"
    if ref.is_file():
        p = snaps / ref.read_text().strip()
        if p.is_dir():
            return p
    if snaps.is_dir():
        cands = sorted((d for d in snaps.iterdir() if d.is_dir()), key=lambda d: d.stat().st_mtime)
        if cands:
            return cands[-1]
    return None


def resolve(cache: Path, model_id: str) -> Path | None:
    return snapshot_of(Path(cache) / repo_folder(model_id))


@dataclass
class CachedModel:
    id: str
    path: str
    model_type: str | None
    family: str | None
    served_by: str | None          # entry of the model table, when a device engine or an oracle serves the family
    weight_bytes: int
    shards: int
    complete: bool                 # every shard the index names is present
    problems: list[str] = field(default_factory=list)
    fit: dict | None = None

    def as_dict(self) -> dict:
        return asdict(self)


def _family_entry(family: str | None):
    if family is None:
        return None
    best = None
    for m in MODELS.values():
        if m.family == family and (best is None or (m.status == "device" and best.status != "device")):
            best = m
    return best


def describe(model_id: str, snap: Path) -> CachedModel:
    problems: list[str] = []
    model_type = None
    cfg = snap / "config.json"
    if cfg.is_file():
        try:
            model_type = json.loads(cfg.read_text()).get("model_type")
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            problems.append(f"config.json does not parse: {e}")
    else:
        problems.append("no config.json")
    family = MODEL_TYPES.get(model_type or "")
    if model_type and family is None:
        problems.append(f"model_type {model_type!r} has no engine here")
    files = sorted(snap.glob("*.safetensors"))
    wanted: set[str] = set()
    idx = snap / "model.safetensors.index.json"
    if idx.is_file():
        try:
            wanted = set(json.loads(idx.read_text()).get("weight_map", {}).values())
        except json.JSONDecodeError as e:
            problems.append(f"shard index does not parse: {e}")
    have = {f.name for f in files if f.exists()}
    missing = sorted(wanted - have)
    if missing:
        problems.append(f"{len(missing)} of {len(wanted)} shards missing (first: {missing[0]})")
    if not files:
        problems.append("no safetensors shards")
    entry = _family_entry(family)
    return CachedModel(model_id, str(snap), model_type, family, entry.name if entry else None,
                       sum(f.stat().st_size for f in files if f.exists()), len(files), bool(files) and not missing, problems)


def list_cached(cache: Path) -> list[CachedModel]:
    cache = Path(cache)
    out = []
    if not cache.is_dir():
        return out
    for d in sorted(cache.iterdir()):
        mid = folder_id(d.name)
        snap = snapshot_of(d) if mid else None
        if mid and snap:
            out.append(describe(mid, snap))
    return out


def lookup(cache: Path, model_id: str) -> CachedModel | None:
    snap = resolve(cache, model_id)
    return describe(model_id, snap) if snap else None


def fit_cached(m: CachedModel, world: int, gpu_gb: float = 180.0, context: int = 131072, lanes: int = 16) -> dict:
    """Whether the cached model fits on ``world`` GPUs.  The flagship family uses the per-tensor estimator; other
    families are judged on their stored bytes split evenly plus a tenth for caches and workspace."""
    if m.family == "deepseek":
        rep = fit.estimate(full_config(), world, context, lanes, gpu_gb).as_dict()
        rep["evidence"] = "per-tensor estimate of the flagship layout"
        return rep
    per = m.weight_bytes / max(world, 1) * 1.1 / 1e9
    return {"world": world, "total_gb": round(per, 2), "capacity_gb": gpu_gb, "fits": per <= gpu_gb * 0.95,
            "evidence": "stored bytes split evenly over the ranks, plus 10 %"}


def judge_cached(models: Iterable[CachedModel], world: int, gpu_gb: float = 180.0) -> None:
    for m in models:
        m.fit = fit_cached(m, world, gpu_gb)


def preferred_cached(models: list[CachedModel], wanted_id: str | None = None) -> CachedModel | None:
    """The model a fresh console offers first: the configured id when it is cached and complete, else the complete
    model of a device-served family with the most bytes, else any complete one."""
    ok = [m for m in models if m.complete and not m.problems]
    for m in ok:
        if m.id == wanted_id:
            return m
    dev = [m for m in ok if m.served_by and MODELS[m.served_by].status == "device"]
    pool = dev or ok
    return max(pool, key=lambda m: m.weight_bytes) if pool else None


def families() -> list[dict]:
    out: dict[str, dict] = {}
    for m in MODELS.values():
        f = out.setdefault(m.family, {"family": m.family, "models": [], "model_types": sorted(k for k, v in MODEL_TYPES.items() if v == m.family)})
        f["models"].append({"name": m.name, "status": m.status, "summary": m.summary})
    return list(out.values())


# ---- remote side: every network access goes through ``fetch(url, headers) -> (status, headers, iterator of bytes)`` ----------------

Fetcher = Callable[[str, dict], tuple]


def url_fetch(url: str, headers: dict) -> tuple:
    req = urllib.request.Request(url, headers=headers)
    r = urllib.request.urlopen(req, timeout=30)

    def chunks():
        while True:
            b = r.read(1 << 20)
            if not b:
                return
            yield b
    return r.status, dict(r.headers), chunks()


def _json(fetch: Fetcher, url: str, token: str | None):
    st, _, body = fetch(url, {"Authorization": f"Bearer {token}"} if token else {})
    data = b"".join(body)
    if st != 200:
        raise RuntimeError(f"{url}: HTTP {st}")
    return json.loads(data)


def search(query: str, fetch: Fetcher = url_fetch, endpoint: str = "https://huggingface.co", token: str | None = None, limit: int = 20) -> list[dict]:
    rows = _json(fetch, f"{endpoint}/api/models?search={urllib.request.quote(query)}&limit={limit}", token)
    return [{"id": r.get("id") or r.get("modelId"), "downloads": r.get("downloads"), "tags": r.get("tags", [])} for r in rows]


def inspect(model_id: str, fetch: Fetcher = url_fetch, endpoint: str = "https://huggingface.co", token: str | None = None,
            cache: Path | None = None, world: int = 8) -> dict:
    """What the hub says about a model (files with sizes, model_type) and, when it is cached, the local state."""
    if not ID_RE.match(model_id):
        raise ValueError(f"{model_id!r} is not an org/name model id")
    info = _json(fetch, f"{endpoint}/api/models/{model_id}?blobs=true", token)
    files = [{"name": s["rfilename"], "size": s.get("size") or (s.get("lfs") or {}).get("size"), "sha256": (s.get("lfs") or {}).get("sha256")}
             for s in info.get("siblings", [])]
    mt = (info.get("config") or {}).get("model_type")
    out = {"id": model_id, "sha": info.get("sha"), "model_type": mt, "family": MODEL_TYPES.get(mt or ""), "files": files,
           "weight_bytes": sum(f["size"] or 0 for f in files if f["name"].endswith(".safetensors"))}
    if cache is not None:
        c = lookup(cache, model_id)
        out["cached"] = c.as_dict() if c else None
    per = out["weight_bytes"] / max(world, 1) * 1.1 / 1e9
    out["fit"] = {"world": world, "gb_per_gpu": round(per, 2), "fits": per <= 180 * 0.95}
    return out


WANTED = re.compile(r"(\.safetensors|\.json|\.txt|\.model|\.jinja)$")


def download(model_id: str, cache: Path, fetch: Fetcher = url_fetch, endpoint: str = "https://huggingface.co", token: str | None = None,
             progress: Callable[[dict], None] | None = None) -> Path:
    """Fetch every weight, config and tokenizer file of ``model_id`` into the cache layout.  A partly written file
    (``<name>.incomplete``) is resumed with a Range request; a file whose size (and sha256, when the hub gives one)
    already matches is skipped.  Returns the snapshot directory."""
    meta = inspect(model_id, fetch, endpoint, token)
    sha = meta["sha"] or "main"
    repo = Path(cache) / repo_folder(model_id)
    snap = repo / "snapshots" / sha
    snap.mkdir(parents=True, exist_ok=True)
    (repo / "refs").mkdir(exist_ok=True)
    files = [f for f in meta["files"] if WANTED.search(f["name"]) and ".." not in Path(f["name"]).parts and not f["name"].startswith("/")]
    total, done = sum(f["size"] or 0 for f in files), 0
    hdr = {"Authorization": f"Bearer {token}"} if token else {}
    for f in files:
        dst = snap / f["name"]
        dst.parent.mkdir(parents=True, exist_ok=True)
        if dst.is_file() and (f["size"] is None or dst.stat().st_size == f["size"]):
            done += dst.stat().st_size
            continue
        part = dst.with_name(dst.name + ".incomplete")
        have = part.stat().st_size if part.is_file() else 0
        st, _, body = fetch(f"{endpoint}/{model_id}/resolve/{sha}/{f['name']}", hdr | ({"Range": f"bytes={have}-"} if have else {}))
        if st == 200:
            have = 0                                   # the server ignored the range: start over
        elif st != 206:
            raise RuntimeError(f"{f['name']}: HTTP {st}")
        with open(part, "ab" if have else "wb") as out:
            for chunk in body:
                out.write(chunk)
                have += len(chunk)
                if progress:
                    progress({"file": f["name"], "bytes": done + have, "total": total})
        if f["size"] is not None and have != f["size"]:
            raise RuntimeError(f"{f['name']}: got {have} bytes, the hub lists {f['size']}")
        if f.get("sha256"):
            h = hashlib.sha256()
            with open(part, "rb") as r:
                for blk in iter(lambda: r.read(1 << 22), b""):
                    h.update(blk)
            if h.hexdigest() != f["sha256"]:
                part.unlink()
                raise RuntimeError(f"{f['name']}: sha256 mismatch")
        part.replace(dst)
        done += have
    (repo / "refs" / "main").write_text(sha)
    return snap
