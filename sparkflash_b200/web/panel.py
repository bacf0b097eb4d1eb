"""Control-panel plan: one TOML file describes what to serve (model, engine shape, paths, web and stats settings); the
panel validates it, derives the environment and the command lines of every operator action (download, convert, start /
stop / status of the server, doctor) and shows them before it runs them.  One node with N GPUs behind NVSwitch is the
unit here, so there are no SSH destinations or fabric rails to plan: a rank is a local process bound to one GPU.

Reference behaviour: crates/sparkflash-web/src/config.rs (SparkConfig:359, validate:744, launch_env:1644,
requires_conversion:1458, world_size:1378), crates/sparkflash-web/src/commands.rs (CommandSpec:30, convert_command:71,
serve_action_command:273, download_command:374).
"""
from __future__ import annotations

import os
import shlex
import sys
import tomllib
from dataclasses import asdict, dataclass, field
from pathlib import Path

from ..config import ENV_INTERNAL, ENV_TABLE
from ..models.registry import MODELS
from . import hub


class PlanError(ValueError):
    pass


@dataclass
class ModelPlan:
    id: str = "deepseek-v4.1-flash"            # an org/name hub id, or an entry of the model table
    checkpoint: str = ""                       # directory of safetensors shards; empty = resolve ``id`` in the hub cache
    synthetic: str = ""                        # "tiny" | "reduced" | "full": random weights of that shape instead of a checkpoint
    tokenizer: str = ""


@dataclass
class EnginePlan:
    world: int = 8
    moe_mode: str = "tp"                       # "tp": experts sliced by width; "ep": whole experts per rank
    lanes: int = 16
    context: int = 131072
    max_rows: int = 1024
    drafting: bool = True                      # the model's own draft stages when the weights carry them, prompt look-up otherwise
    draft_depth: int = 4
    collective: str = "fused"                  # "fused": this package's NVLink kernels; "nccl": the baseline arm
    lane_budget_gb: int = 0
    arm: str = "tc"


@dataclass
class PathsPlan:
    converted: str = "~/.cache/sparkflash_b200/converted"
    hub_cache: str = ""
    stats: str = "~/.cache/sparkflash_b200/stats.json"
    pid_file: str = "~/.cache/sparkflash_b200/serve.pid"
    log: str = "~/.cache/sparkflash_b200/serve.log"


@dataclass
class WebPlan:
    host: str = "127.0.0.1"
    port: int = 8080
    server_host: str = "127.0.0.1"
    server_port: int = 8000
    control_port: int = 29600
    api_key_env: str = "SFB_API_KEY"           # the NAME of the variable; a key never sits in the file


@dataclass
class StatsPlan:
    interval_s: float = 2.0
    history_s: float = 86400.0
    flush_s: float = 300.0


@dataclass
class Plan:
    model: ModelPlan = field(default_factory=ModelPlan)
    engine: EnginePlan = field(default_factory=EnginePlan)
    paths: PathsPlan = field(default_factory=PathsPlan)
    web: WebPlan = field(default_factory=WebPlan)
    stats: StatsPlan = field(default_factory=StatsPlan)
    env: dict = field(default_factory=dict)    # extra SFB_* settings for the server processes

    # ---- file ----------------------------------------------------------------------------------------------------
    @classmethod
    def from_toml(cls, text: str) -> "Plan":
        try:
            raw = tomllib.loads(text)
        except tomllib.TOMLDecodeError as e:
            raise PlanError(f"not valid TOML: {e}") from None
        p = cls()
        for name, part in (("model", p.model), ("engine", p.engine), ("paths", p.paths), ("web", p.web), ("stats", p.stats)):
            for k, v in raw.pop(name, {}).items():
                if not hasattr(part, k):
                    raise PlanError(f"[{name}] has no setting {k!r}")
                want = type(getattr(part, k))
                if want is float and isinstance(v, int):
                    v = float(v)
                if not isinstance(v, want) or (want is int and isinstance(v, bool)):
                    raise PlanError(f"[{name}] {k} wants {want.__name__}, got {type(v).__name__}")
                setattr(part, k, v)
        p.env = {str(k): str(v) for k, v in raw.pop("env", {}).items()}
        if raw:
            raise PlanError(f"unknown section(s): {', '.join(sorted(raw))}")
        p.validate()
        return p

    @classmethod
    def load(cls, path) -> "Plan":
        return cls.from_toml(Path(path).read_text())

    def to_toml(self) -> str:
        def val(v):
            if isinstance(v, bool):
                return "true" if v else "false"
            if isinstance(v, (int, float)):
                return repr(v)
            return '"' + str(v).replace("\\", "\\\\").replace('"', '\\"') + '"'
        out = []
        for name in ("model", "engine", "paths", "web", "stats"):
            out.append(f"[{name}]")
            out += [f"{k} = {val(v)}" for k, v in asdict(getattr(self, name)).items()]
            out.append("")
        if self.env:
            out.append("[env]")
            out += [f"{k} = {val(v)}" for k, v in sorted(self.env.items())]
            out.append("")
        return "\n".join(out)

    def save(self, path) -> None:
        path = Path(path)
        tmp = path.with_name(path.name + ".tmp")
        tmp.write_text(self.to_toml())
        tmp.replace(path)

    # ---- rules ---------------------------------------------------------------------------------------------------
    def validate(self) -> None:
        e, m = self.engine, self.model
        if e.world not in (1, 2, 4, 8):
            raise PlanError(f"engine.world = {e.world}: a node serves on 1, 2, 4 or 8 GPUs")
        if e.moe_mode not in ("tp", "ep"):
            raise PlanError(f"engine.moe_mode = {e.moe_mode!r}: tp or ep")
        if e.collective not in ("fused", "nccl"):
            raise PlanError(f"engine.collective = {e.collective!r}: fused or nccl")
        if e.arm not in ("tc", "cuda"):
            raise PlanError(f"engine.arm = {e.arm!r}: tc or cuda")
        if not 1 <= e.lanes <= 256:
            raise PlanError("engine.lanes must be in 1..256")
        if e.context < 1024 or e.context > (1 << 20):
            raise PlanError("engine.context must be in 1,024..1,048,576")
        if e.max_rows not in (64, 128, 256, 512, 1024, 2048):
            raise PlanError("engine.max_rows must be one of 64, 128, 256, 512, 1024, 2048")
        if not 0 <= e.draft_depth <= 8:
            raise PlanError("engine.draft_depth must be in 0..8")
        if m.synthetic not in ("", "tiny", "reduced", "full"):
            raise PlanError(f"model.synthetic = {m.synthetic!r}: tiny, reduced or full")
        if not m.synthetic and not m.checkpoint and not hub.ID_RE.match(m.id) and m.id not in MODELS:
            raise PlanError(f"model.id = {m.id!r} is neither an org/name hub id nor an entry of the model table")
        if self.web.port == self.web.server_port and self.web.host == self.web.server_host:
            raise PlanError("web.port and web.server_port collide")
        known = set(ENV_TABLE) | set(ENV_INTERNAL)
        for k in self.env:
            if not k.startswith("SFB_"):
                raise PlanError(f"[env] {k}: only SFB_* settings are passed to the server")
            if k not in known:
                raise PlanError(f"[env] {k} is not a setting of this package")

    # ---- derived -------------------------------------------------------------------------------------------------
    def world_size(self) -> int:
        return self.engine.world

    def is_solo(self) -> bool:
        return self.engine.world == 1

    def family(self) -> str | None:
        if self.model.id in MODELS:
            return MODELS[self.model.id].family
        return None

    def hub_cache_dir(self) -> Path:
        return expand(self.paths.hub_cache) if self.paths.hub_cache else hub.default_cache_dir()

    def resolve_checkpoint(self) -> Path:
        if self.model.synthetic:
            raise PlanError("a synthetic model has no checkpoint")
        if self.model.checkpoint:
            p = expand(self.model.checkpoint)
            if not p.is_dir():
                raise PlanError(f"model.checkpoint {p} is not a directory")
            return p
        if hub.ID_RE.match(self.model.id):
            snap = hub.resolve(self.hub_cache_dir(), self.model.id)
            if snap is None:
                raise PlanError(f"{self.model.id} is not in the hub cache {self.hub_cache_dir()} (download it first)")
            return snap
        raise PlanError(f"model.id = {self.model.id!r} names a family, not a checkpoint: set model.checkpoint or an org/name id")

    def conversion_scope(self) -> str:
        """Folder name of the converted rank files: they depend on the model, the world size and the expert split."""
        tag = self.model.id.replace("/", "--")
        return f"{tag}-w{self.engine.world}-{self.engine.moe_mode}"

    def converted_path(self) -> Path:
        return expand(self.paths.converted) / self.conversion_scope()

    def requires_conversion(self) -> bool:
        if self.model.synthetic:
            return False
        d = self.converted_path()
        return not all((d / f"rank{r}-of-{self.engine.world}.sfb").is_file() for r in range(self.engine.world))

    def launch_env(self) -> dict:
        e = {"SFB_MOE_MODE": self.engine.moe_mode, "SFB_COLLECTIVE": self.engine.collective, "SFB_MAX_LANES": str(self.engine.lanes),
             "SFB_MAX_CONTEXT": str(self.engine.context), "SFB_MAX_ROWS": str(self.engine.max_rows),
             "SFB_SPECULATION": "1" if self.engine.drafting else "0", "SFB_SPEC_DEPTH": str(self.engine.draft_depth), "SFB_ARM": self.engine.arm}
        e.update(self.env)
        return e

    def server_url(self) -> str:
        return f"http://{self.web.server_host}:{self.web.server_port}"

    def as_dict(self) -> dict:
        return {k: asdict(getattr(self, k)) for k in ("model", "engine", "paths", "web", "stats")} | {"env": dict(self.env)}


def expand(path: str) -> Path:
    return Path(os.path.expanduser(os.path.expandvars(path)))


# ---- command lines ---------------------------------------------------------------------------------------------------

@dataclass
class CommandSpec:
    label: str
    kind: str
    argv: list[str]
    env: dict = field(default_factory=dict)
    cwd: str | None = None

    def display(self) -> str:
        """The line an operator could paste into a shell: environment first, every word quoted where it needs it."""
        env = " ".join(f"{k}={shlex.quote(v)}" for k, v in sorted(self.env.items()))
        return (env + " " if env else "") + " ".join(shlex.quote(a) for a in self.argv)

    def as_dict(self) -> dict:
        return {"label": self.label, "kind": self.kind, "argv": self.argv, "env": self.env, "cwd": self.cwd, "display": self.display()}


PY = sys.executable or "python"


def download_command(p: Plan) -> CommandSpec:
    if not hub.ID_RE.match(p.model.id):
        raise PlanError(f"model.id = {p.model.id!r} is not an org/name hub id: nothing to download")
    return CommandSpec("Download the checkpoint", "download", [PY, "-m", "sparkflash_b200.web.app", "download", p.model.id,
                                                               "--cache", str(p.hub_cache_dir())])


def convert_command(p: Plan) -> CommandSpec:
    argv = [PY, "-m", "sparkflash_b200", "convert", "--output-dir", str(p.converted_path()), "--tp-world-size", str(p.engine.world),
            "--expert-split", p.engine.moe_mode]
    if p.model.synthetic:
        argv += ["--synthetic", "tiny" if p.model.synthetic == "tiny" else "full"]
    else:
        argv += ["--checkpoint", str(p.resolve_checkpoint())]
    return CommandSpec("Convert to per-rank files", "convert", argv)


def inspect_command(p: Plan) -> CommandSpec:
    return CommandSpec("Inspect the converted files", "inspect", [PY, "-m", "sparkflash_b200", "convert", "--inspect", str(p.converted_path())])


def doctor_command(p: Plan) -> CommandSpec:
    argv = [PY, "-m", "sparkflash_b200", "doctor", "--gpus", str(p.engine.world)]
    if not p.model.synthetic:
        argv += ["--weights", str(p.converted_path())]
    return CommandSpec("Check this node", "doctor", argv)


SERVE_ACTIONS = {"launch": ("Start server", "Launch all ranks"), "stop": ("Stop server", "Stop all ranks"),
                 "status": ("Check server status", "Check rank status")}


def serve_action_command(p: Plan, action: str) -> CommandSpec:
    """launch: one detached supervisor (it starts one process per GPU); stop: SIGTERM to exactly the recorded process
    group (rank 0 drains first); status: is the recorded group alive, and does the server answer its health route."""
    if action not in SERVE_ACTIONS:
        raise PlanError(f"unknown serve action {action!r}")
    label = SERVE_ACTIONS[action][0 if p.is_solo() else 1]
    sup = [PY, "-m", "sparkflash_b200.serve.supervisor", action, "--pid-file", str(expand(p.paths.pid_file))]
    if action == "launch":
        argv = sup + ["--gpus", str(p.engine.world), "--log", str(expand(p.paths.log)), "--master-port", str(p.web.control_port + 1), "--",
                      "--host", p.web.server_host, "--port", str(p.web.server_port), "--control-port", str(p.web.control_port), "--model-id", p.model.id]
        if p.model.synthetic:
            argv += ["--synthetic", p.model.synthetic]
        else:
            argv += ["--weights", str(p.converted_path())]
        if p.model.tokenizer:
            argv += ["--tokenizer", str(expand(p.model.tokenizer))]
        if p.engine.lane_budget_gb:
            argv += ["--lane-budget-gb", str(p.engine.lane_budget_gb)]
        return CommandSpec(label, action, argv, p.launch_env())
    if action == "status":
        sup += ["--url", p.server_url()]
    return CommandSpec(label, action, sup)


def workflow(p: Plan) -> list[CommandSpec]:
    """The steps from this plan to a serving node, in order, leaving out what is already done."""
    steps = [doctor_command(p)]
    if not p.model.synthetic and not p.model.checkpoint and hub.ID_RE.match(p.model.id) and hub.resolve(p.hub_cache_dir(), p.model.id) is None:
        steps.append(download_command(p))
    if p.requires_conversion():
        steps.append(convert_command_lazy(p))
    steps.append(serve_action_command(p, "launch"))
    return steps


def convert_command_lazy(p: Plan) -> CommandSpec:
    """convert_command, tolerating a checkpoint that an earlier step of the workflow will download."""
    try:
        return convert_command(p)
    except PlanError:
        snap = p.hub_cache_dir() / hub.repo_folder(p.model.id) / "snapshots" / "<downloaded>"
        return CommandSpec("Convert to per-rank files", "convert", [PY, "-m", "sparkflash_b200", "convert", "--checkpoint", str(snap), "--output-dir",
                                                                     str(p.converted_path()), "--tp-world-size", str(p.engine.world), "--expert-split", p.engine.moe_mode])
