"""Numerics registry gate: nothing about a configuration's arithmetic changes unless it was declared.

Each registry entry names a configuration (model + world size), its numerics version and the digest of the
CPU oracle's output on a fixed prompt suite (greedy tokens and the bit patterns of the first-step logits).  The
gate recomputes the digest; a mismatch without a version bump is a failure.  ``--update`` writes a new digest
only together with a bumped version and a declaration line.  Reference: docs/NUMERICS.md sections 1-5,
scripts/numerics.py, scripts/numerical-gate.sh.

    python -m sparkflash_b200.gates.numerics [--update --declare "split-K order of wo_b changed"]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys
import tomllib

REGISTRY = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "numerics", "registry.toml")
PROMPTS = [[3, 17, 99, 250, 4, 4, 81], [500, 501, 502, 503, 504, 505, 506, 507, 508, 509, 510, 511], [7] * 20]
N_NEW = 6


def reference_digest(config_name: str, world: int) -> str:
    import torch
    from ..config import tiny_config, tiny_mla_v3_config
    from ..models.deepseek_v41 import oracle as O, weights as W
    cfg = {"tiny-csa2": tiny_config, "tiny-mla-v3": tiny_mla_v3_config}[config_name]()
    ck = W.synthetic_checkpoint(cfg, 0)
    orc = O.Oracle(cfg, W.dequantize_checkpoint(ck, cfg) if hasattr(W, "dequantize_checkpoint") else ck, world)
    h = hashlib.sha256()
    for p in PROMPTS:
        p = [t % cfg.vocab_size for t in p]
        out = orc.generate(p, N_NEW)
        toks, logits = (out if isinstance(out, tuple) else (out, None))
        h.update(repr(list(map(int, toks))).encode())
        if logits is not None:
            h.update(torch.as_tensor(logits[0]).float().contiguous().numpy().tobytes())
    return h.hexdigest()[:32]


def load_registry(path: str = REGISTRY) -> dict:
    with open(path, "rb") as f:
        return tomllib.load(f)


def write_registry(reg: dict, path: str = REGISTRY) -> None:
    lines = ["# Numerics registry: one entry per served configuration.  Edited only by `gates.numerics --update`.", ""]
    for name, e in reg["config"].items():
        lines += [f'[config."{name}"]', f'model = "{e["model"]}"', f'world = {e["world"]}', f'version = {e["version"]}',
                  f'digest = "{e["digest"]}"', "declared = [", *[f'  "{d}",' for d in e.get("declared", [])], "]", ""]
    with open(path, "w") as f:
        f.write("\n".join(lines))


def check(reg: dict, compute=reference_digest) -> list[str]:
    problems = []
    for name, e in reg["config"].items():
        got = compute(e["model"], e["world"])
        if got != e["digest"]:
            problems.append(f"{name}: digest {got} differs from the registered {e['digest']} (version {e['version']}): "
                            f"an undeclared change of arithmetic")
        if len(e.get("declared", [])) != e["version"]:
            problems.append(f"{name}: version {e['version']} needs exactly {e['version']} declaration line(s)")
    return problems


def update(reg: dict, declaration: str, compute=reference_digest) -> list[str]:
    changed = []
    for name, e in reg["config"].items():
        got = compute(e["model"], e["world"])
        if got != e["digest"]:
            e["digest"], e["version"] = got, e["version"] + 1
            e.setdefault("declared", []).append(declaration)
            changed.append(name)
    return changed


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--update", action="store_true")
    ap.add_argument("--declare", default="")
    a = ap.parse_args(argv)
    reg = load_registry()
    if a.update:
        if not a.declare.strip():
            print("numerics: --update needs --declare \"what changed and why\"", file=sys.stderr)
            return 2
        ch = update(reg, a.declare.strip())
        write_registry(reg)
        print(f"numerics: bumped {ch or 'nothing'}")
        return 0
    problems = check(reg)
    for p in problems:
        print("numerics: " + p, file=sys.stderr)
    print(f"numerics: {len(reg['config'])} configuration(s), {len(problems)} problem(s)")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
