"""Node facts and the setup report: what this node has (GPUs, the NVLink matrix between them, driver, free disk,
the built libraries) and whether the plan can run on it.  Facts are read, never set; every source is injectable so the
analysis runs on recorded text.

The unit is one NVSwitch node, so the "fabric" to check is the GPU-to-GPU matrix: every pair of the GPUs a plan uses must
be connected by NVLink (``NV#`` in ``nvidia-smi topo -m``), otherwise the fused collectives would cross PCIe.

Reference behaviour: crates/sparkflash-web/src/inspect.rs (parse_facts:232, analyze:577, Finding:485, SetupReport:545),
crates/sparkflash-web/src/discovery.rs (NodeReport:69).
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
from dataclasses import asdict, dataclass, field
from pathlib import Path

from . import hub, panel


@dataclass
class GpuFact:
    index: int
    name: str
    memory_mib: int
    free_mib: int
    sm: str


@dataclass
class NodeFacts:
    host: str = "localhost"
    driver: str | None = None
    gpus: list[GpuFact] = field(default_factory=list)
    links: dict = field(default_factory=dict)          # (i, j) -> "NV18", "PIX", "SYS", ...
    disk_free_gb: dict = field(default_factory=dict)   # path -> GB
    libraries: dict = field(default_factory=dict)      # name -> bool
    errors: list[str] = field(default_factory=list)

    def as_dict(self) -> dict:
        d = asdict(self)
        d["links"] = {f"{i}-{j}": v for (i, j), v in self.links.items()}
        return d


def parse_gpu_csv(text: str) -> tuple[list[GpuFact], str | None]:
    """``nvidia-smi --query-gpu=index,name,memory.total,memory.free,compute_cap,driver_version --format=csv,noheader,nounits``"""
    gpus, driver = [], None
    for line in text.strip().splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 6 or not f[0].isdigit():
            continue
        gpus.append(GpuFact(int(f[0]), f[1], int(float(f[2])), int(float(f[3])), f[4].replace(".", "")))
        driver = f[5]
    return gpus, driver


def parse_topo(text: str) -> dict:
    """The GPU block of ``nvidia-smi topo -m``: a header row of GPU names, then one row per GPU."""
    links = {}
    lines = [ln for ln in text.splitlines() if ln.strip()]
    header = None
    for ln in lines:
        cells = re.sub(r"\x1b\[[0-9;]*m", "", ln).split()
        if header is None:
            if cells and cells[0].startswith("GPU0"):
                header = [c for c in cells if re.fullmatch(r"GPU\d+", c)]
            continue
        if not cells or not re.fullmatch(r"GPU\d+", cells[0]):
            continue
        i = int(cells[0][3:])
        for j, c in enumerate(cells[1:1 + len(header)]):
            if c != "X":
                links[(i, j)] = c
    return links


def _run(argv: list[str]) -> str:
    return subprocess.run(argv, capture_output=True, text=True, timeout=20, check=True).stdout


def gather(run=_run, paths: list[str] | None = None) -> NodeFacts:
    f = NodeFacts(host=os.uname().nodename)
    try:
        f.gpus, f.driver = parse_gpu_csv(run(["nvidia-smi", "--query-gpu=index,name,memory.total,memory.free,compute_cap,driver_version",
                                              "--format=csv,noheader,nounits"]))
    except Exception as e:                                         # noqa: BLE001
        f.errors.append(f"nvidia-smi query: {type(e).__name__}: {e}")
    try:
        f.links = parse_topo(run(["nvidia-smi", "topo", "-m"]))
    except Exception as e:                                         # noqa: BLE001
        f.errors.append(f"nvidia-smi topo: {type(e).__name__}: {e}")
    for p in paths or []:
        q = Path(p)
        while not q.exists() and q != q.parent:
            q = q.parent
        try:
            f.disk_free_gb[p] = round(shutil.disk_usage(q).free / 1e9, 1)
        except OSError as e:
            f.errors.append(f"{p}: {e}")
    lib = Path(__file__).resolve().parent.parent / "lib"
    f.libraries = {n: (lib / n).is_file() for n in ("libsfb_cuda.so", "libsfb_host.so")}
    return f


@dataclass
class Finding:
    severity: str          # "ok" | "warn" | "fail"
    check: str
    message: str
    fix: str = ""


@dataclass
class SetupReport:
    findings: list[Finding]

    def ok(self) -> bool:
        return not any(f.severity == "fail" for f in self.findings)

    def as_dict(self) -> dict:
        return {"ok": self.ok(), "findings": [asdict(f) for f in self.findings]}


def analyze(plan: "panel.Plan", facts: NodeFacts, weight_bytes: int | None = None) -> SetupReport:
    out: list[Finding] = []
    W = plan.engine.world
    for e in facts.errors:
        out.append(Finding("warn", "facts", e))
    # GPUs
    if len(facts.gpus) < W:
        out.append(Finding("fail", "gpus", f"the plan wants {W} GPUs, this node shows {len(facts.gpus)}", "lower engine.world"))
    else:
        out.append(Finding("ok", "gpus", f"{len(facts.gpus)} GPUs visible, {W} used"))
    used = facts.gpus[:W]
    wrong = [g for g in used if g.sm != "100"]
    if wrong:
        out.append(Finding("fail", "arch", f"GPU {wrong[0].index} is sm_{wrong[0].sm}; the kernels are built for sm_100a only"))
    busy = [g for g in used if g.free_mib < 0.9 * g.memory_mib]
    if busy:
        out.append(Finding("warn", "memory", f"GPU {busy[0].index} has {busy[0].free_mib} of {busy[0].memory_mib} MiB free: another process holds memory"))
    # links between every pair the plan uses
    if W > 1 and facts.links:
        bad = [(i, j, facts.links.get((i, j), "?")) for i in range(W) for j in range(W) if i != j and not str(facts.links.get((i, j), "")).startswith("NV")]
        if bad:
            i, j, v = bad[0]
            out.append(Finding("fail", "nvlink", f"GPU {i} and GPU {j} are connected by {v}, not NVLink ({len(bad)} such pairs)",
                               "choose GPUs of one NVSwitch domain with CUDA_VISIBLE_DEVICES"))
        else:
            out.append(Finding("ok", "nvlink", f"all {W * (W - 1) // 2} GPU pairs are NVLink-connected"))
    elif W > 1:
        out.append(Finding("warn", "nvlink", "no topology matrix could be read"))
    # libraries
    for name, have in facts.libraries.items():
        if not have:
            out.append(Finding("fail", "build", f"{name} is not built", "python -m sparkflash_b200._build"))
    # model source
    if not plan.model.synthetic:
        try:
            ck = plan.resolve_checkpoint()
            out.append(Finding("ok", "checkpoint", f"checkpoint at {ck}"))
            if weight_bytes is None:
                weight_bytes = sum(f.stat().st_size for f in ck.glob("*.safetensors"))
        except panel.PlanError as e:
            sev = "warn" if hub.ID_RE.match(plan.model.id) else "fail"
            out.append(Finding(sev, "checkpoint", str(e), "run the download step" if sev == "warn" else "set model.checkpoint"))
        if plan.requires_conversion():
            need = (weight_bytes or 0) * 1.05 / 1e9
            free = facts.disk_free_gb.get(str(panel.expand(plan.paths.converted)))
            if free is not None and need and free < need:
                out.append(Finding("fail", "disk", f"conversion writes ≈{need:.0f} GB, {free:.0f} GB free under {plan.paths.converted}"))
            else:
                out.append(Finding("warn", "convert", f"rank files for {plan.conversion_scope()} are not there yet", "run the convert step"))
        else:
            out.append(Finding("ok", "convert", f"rank files present in {plan.converted_path()}"))
    # memory fit
    if used:
        from ..config import full_config, reduced_config, tiny_config
        from . import fit
        cfg = {"tiny": tiny_config, "reduced": lambda: reduced_config(128, 40)}.get(plan.model.synthetic, full_config)()
        rep = fit.estimate(cfg, W, plan.engine.context, plan.engine.lanes, min(g.memory_mib for g in used) * 1.048576 / 1000)
        out.append(Finding("ok" if rep.fits else "fail", "fit", f"{rep.total_gb:.1f} GB of {rep.capacity_gb:.0f} GB per GPU "
                           f"(weights {rep.weights_gb:.1f}, KV {rep.kv_gb:.1f}); up to {rep.max_lanes_that_fit} lanes fit",
                           "" if rep.fits else "lower engine.lanes or engine.context, or raise engine.world"))
    return SetupReport(out)
