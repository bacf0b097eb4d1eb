#!/usr/bin/env python
"""Everything that can be checked without a GPU, in the order a contributor wants to hear about it:

  1. the native build for sm_100a (nvcc cross-compiles without a device) and the host library;
  2. the ABI check (ci/check_abi.py) and the source rules (ci/check_sources.py);
  3. the parts catalogue against the built library (every catalogued entry point is exported);
  4. the env-override table: every SFB_* variable the sources read is declared in config.ENV_TABLE;
  5. the CPU test tiers (pytest -m "not gpu").

    python ci/host_gates.py [--skip-tests]

Reference: ci/host-gates.py, ci/check_features.py of the reference.
"""
from __future__ import annotations

import argparse
import re
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "ci"))


def gate_build() -> str:
    from sparkflash_b200 import _build
    t0 = time.time()
    out = _build.build()
    for p in out.values():
        if not p.exists():
            raise RuntimeError(f"{p} was not built")
    return f"built in {time.time() - t0:.1f}s"


def gate_abi() -> str:
    import check_abi
    if check_abi.main() != 0:
        raise RuntimeError("ABI mismatch between native entry points and Python callers")
    return "argument counts agree"


def gate_sources() -> str:
    import check_sources
    problems = check_sources.scan()
    if problems:
        raise RuntimeError("; ".join(problems[:5]))
    return "no forbidden construct"


def gate_catalogue() -> str:
    from sparkflash_b200.ops.plan import KernelResolver
    missing = KernelResolver().missing()
    if missing:
        raise RuntimeError(f"catalogued entry points not exported: {missing[:5]}")
    return "every catalogued entry point is exported"


def env_reads() -> set[str]:
    """SFB_* names read through os.environ in the package and the root scripts."""
    names = set()
    pat = re.compile(r"environ(?:\.get|\.setdefault)?\s*[\(\[]\s*[\"'](SFB_[A-Z0-9_]+)[\"']")
    for f in list((ROOT / "sparkflash_b200").rglob("*.py")) + [ROOT / "bench.py", ROOT / "step_demo.py"]:
        names |= set(pat.findall(f.read_text()))
    return names


def gate_env_table() -> str:
    from sparkflash_b200 import config
    table = getattr(config, "ENV_TABLE", None)
    declared = set(table) if isinstance(table, dict) else {getattr(e, "name", e[0] if isinstance(e, tuple) else e) for e in (table or [])}
    undeclared = sorted(n for n in env_reads() if n not in declared and n not in config.ENV_INTERNAL)
    if undeclared:
        raise RuntimeError(f"environment variables read but not declared in config.ENV_TABLE: {undeclared}")
    return f"{len(declared)} declared overrides cover every SFB_* read"


def gate_tests() -> str:
    r = subprocess.run([sys.executable, "-m", "pytest", "tests", "-x", "-q", "-m", "not gpu"], cwd=ROOT, capture_output=True, text=True)
    tail = (r.stdout.strip().splitlines() or [""])[-1]
    if r.returncode != 0:
        raise RuntimeError(tail + "\n" + r.stdout[-2000:])
    return tail


GATES = [("build", gate_build), ("abi", gate_abi), ("sources", gate_sources), ("catalogue", gate_catalogue), ("env-table", gate_env_table),
         ("tests", gate_tests)]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--skip-tests", action="store_true")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    failed = 0
    for name, fn in GATES:
        if (args.skip_tests and name == "tests") or (args.only and name not in args.only.split(",")):
            continue
        try:
            print(f"[ ok ] {name}: {fn()}")
        except Exception as e:
            failed += 1
            print(f"[FAIL] {name}: {e}")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
