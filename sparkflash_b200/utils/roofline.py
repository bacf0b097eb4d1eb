"""Per-kernel-class roofline accounting of a rows step, without a profiler.

``timed_step`` runs one eager step with a CUDA event after every launch the wrappers issue and returns (launch name,
microseconds) in order; ``account`` groups the launches into classes (dense projections, expert gate/up, expert down,
attention, indexer, seams, head, rest), computes for each class the bytes it must move and the FLOPs it must do for this
step from the prepared weights and the step's shape, and reports measured time, roofline time (the slower of bytes /
measured copy bandwidth and FLOPs / measured GEMM rate) and the fraction achieved.  The peaks come from
``MEASURED_PEAKS.json`` at the repository root when present (``hbm_gbs``, ``bf16_tflops_sustained``), else the fallback
figures of this pool.  ``python -m sparkflash_b200 roofline --rows 1024`` prints the table.

Event timing in eager mode includes each launch's gap to its predecessor (a few microseconds): the classes that matter at
many rows are hundreds of microseconds, the one-row figures are upper bounds.
Reference behaviour: scripts/probes/sparkdash_decode.py and docs/performance.md (per-component step budgets against the
memory roofline), crates/sparkflash-kernels roofline notes per launcher.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from ..runtime import segments

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}

CLASSES = (
    ("moe_gate_up", ("umma_gate_up", "moe_gate_up")),
    ("moe_down", ("umma_down", "moe_down", "moe_combine")),
    ("moe_plan", ("moe_plan", "moe_permute", "router", "expert_remap")),
    ("attention", ("attn_",)),
    ("indexer", ("index_", "select_topk", "hsi_")),
    ("sampler", ("sample",)),
    ("seams", ("seam_", "fold_slots", "fold_push", "push_rows", "tap_mean")),
    ("kv", ("qkv_post", "compress_append", "rope_table", "embed")),
    ("dense", ("umma_", "gemv", "splitk", "quant_rows")),
)


def peaks(root: str | Path | None = None) -> dict:
    p = Path(root) if root else Path(__file__).resolve().parents[2]
    f = p / "MEASURED_PEAKS.json"
    if f.is_file():
        try:
            d = json.loads(f.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained") or d["bf16_tflops"]),
                    "source": "measured"}
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


def classify(name: str) -> str:
    for cls, keys in CLASSES:
        if any(k in name for k in keys):
            return cls
    return "rest"


class _TimedLog(segments.LaunchLog):
    def __init__(self):
        super().__init__()
        self.events: list[torch.cuda.Event] = []

    def note(self, name: str) -> None:
        super().note(name)
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.events.append(e)


def timed_step(engine, tokens, lanes, positions, **kw) -> list[tuple[str, float]]:
    """One eager step (the engine must have been built with ``use_graphs=False``) with an event after every launch."""
    start = torch.cuda.Event(enable_timing=True)
    log = _TimedLog()
    prev = segments.install(log)
    try:
        torch.cuda.synchronize()
        start.record()
        engine.step(tokens, lanes, positions, **kw)
        torch.cuda.synchronize()
    finally:
        segments.install(prev)
    out, last = [], start
    for name, ev in zip(log.items, log.events):
        out.append((name, last.elapsed_time(ev) * 1e3))
        last = ev
    return out


@dataclass
class ClassWork:
    bytes: float = 0.0
    flops: float = 0.0


def _nbytes(*ts) -> float:
    return float(sum(t.numel() * t.element_size() for t in ts if t is not None))


def work_model(engine, n: int, context: int, head_rows: int = 0) -> dict[str, ClassWork]:
    """Bytes and FLOPs a step of ``n`` rows at ``context`` cached tokens must move and do on this rank, per class.  Weights
    count once per step (experts: the distinct experts the rows can touch, at most the resident pool); activations and KV
    reads count where they dominate (attention)."""
    cfg, w = engine.cfg, engine.w
    d = cfg.hidden_size
    out = {c: ClassWork() for c, _ in CLASSES}
    out["rest"] = ClassWork()
    E_res = w.layers[0].w13.shape[0] if w.layers and w.layers[0].w13 is not None else 0
    touched = min(E_res, n * cfg.top_k) if E_res else 0
    for L in w.layers:
        dense_w = _nbytes(L.wqkv_a, L.wqkv_a_sf, L.wq_b, L.wq_b_sf, L.wo_a, L.wo_a_sf, L.wo_b, L.wo_b_sf, L.aux_w, L.gate_w)
        out["dense"].bytes += dense_w + n * d * 2 * 6
        dense_rows = sum(t.shape[0] * t.shape[1] for t in (L.wqkv_a, L.wq_b, L.wo_a, L.wo_b) if t is not None)
        out["dense"].flops += 2.0 * n * dense_rows
        if L.w13 is not None:
            per_gu = _nbytes(L.w13[0], L.w13_sf[0]) if L.w13_sf is not None else _nbytes(L.w13[0])
            per_dn = _nbytes(L.w2[0], L.w2_sf[0]) if L.w2_sf is not None else _nbytes(L.w2[0])
            out["moe_gate_up"].bytes += touched * per_gu + _nbytes(L.s13, L.s13_sf)
            out["moe_down"].bytes += touched * per_dn + _nbytes(L.s2, L.s2_sf)
            il = w.il or cfg.moe_inter
            pairs = n * (cfg.top_k + (1 if L.s13 is not None else 0))
            out["moe_gate_up"].flops += 2.0 * pairs * 2 * il * d
            out["moe_down"].flops += 2.0 * pairs * il * d
        out["seams"].bytes += 2 * n * cfg.hc_mult * d * 2 * 2 + _nbytes(L.hc_attn_fn, L.hc_ffn_fn)
    # attention: every row reads its window and its selected compressed entries once per head group
    hd = cfg.head_dim
    heads = cfg.n_heads // max(1, w.world)
    for li, ratio in enumerate(cfg.compress_ratios[:len(w.layers)]):
        keys = min(cfg.window, context)
        if ratio:
            keys += min(cfg.index_topk, max(1, context // (4 if ratio == 2 else 128)))
        out["attention"].bytes += n * keys * hd * (1.0 if not ratio else 0.6)
        out["attention"].flops += 2.0 * n * heads * keys * hd * 2
    if head_rows:      # the vocabulary head is a bf16 tensor-core GEMM like the other projections: counted with them
        out["dense"].bytes += _nbytes(w.head)
        out["dense"].flops += 2.0 * w.head.shape[0] * d * head_rows
    return out


def account(timings: list[tuple[str, float]], work: dict[str, ClassWork], pk: dict | None = None) -> list[dict]:
    pk = pk or peaks()
    by: dict[str, list[float]] = {}
    for name, us in timings:
        by.setdefault(classify(name), []).append(us)
    rows = []
    for cls, ts in sorted(by.items(), key=lambda kv: -sum(kv[1])):
        wk = work.get(cls, ClassWork())
        t_mem = wk.bytes / (pk["hbm_gbs"] * 1e9) * 1e6
        t_cmp = wk.flops / (pk["bf16_tflops_sustained"] * 1e12) * 1e6
        roof = max(t_mem, t_cmp)
        meas = sum(ts)
        rows.append({"class": cls, "launches": len(ts), "measured_us": round(meas, 1), "bytes_mb": round(wk.bytes / 1e6, 1),
                     "gflop": round(wk.flops / 1e9, 1), "roofline_us": round(roof, 1), "bound": "memory" if t_mem >= t_cmp else "compute",
                     "fraction_of_" + pk["source"]: round(roof / meas, 3) if meas > 0 and roof > 0 else None})
    return rows


def format_table(rows: list[dict]) -> str:
    if not rows:
        return "(no launches)"
    keys = list(rows[0].keys())
    lines = ["| " + " | ".join(keys) + " |", "|" + "---|" * len(keys)]
    for r in rows:
        lines.append("| " + " | ".join(str(r[k]) for k in keys) + " |")
    return "\n".join(lines)
