"""Performance regression gate and collective-count check.

``perf``: compare a bench.py JSON line against a committed baseline with a tolerance; a drop beyond it fails.
``collectives``: the number of cross-rank exchanges of one step is fixed by the architecture (two sublayer
seams per layer plus the sampler); more than that means somebody added a hidden collective.  Reference:
scripts/perf_regression_gate.py, scripts/check-collective-count.py.

    python -m sparkflash_b200.gates.perf perf --result BENCH.json [--baseline perf_baseline.json] [--tolerance 0.03]

The default baseline is ``gates/perf_baseline.json`` (B200 figures of bench.py's defaults at 1, 2 and 8 GPUs).
    python -m sparkflash_b200.gates.perf collectives --layers 40 --counted 81
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def expected_collectives(n_layers: int) -> int:
    return 2 * n_layers + 1


def check_collectives(n_layers: int, counted: int) -> list[str]:
    want = expected_collectives(n_layers)
    return [] if counted == want else [f"{counted} exchanges per step, the architecture needs exactly {want} (2 per layer + sampler)"]


def check_perf(result: dict, baseline: dict, tolerance: float = 0.03) -> list[str]:
    problems = []
    key = f'{result.get("metric")}@{result.get("n_gpus")}'
    base = baseline.get(key)
    if base is None:
        return [f"no baseline for {key}"]
    hib = result.get("higher_is_better", True)
    v, b = float(result["value"]), float(base["value"])
    worse = v < b * (1 - tolerance) if hib else v > b * (1 + tolerance)
    if worse:
        problems.append(f"{key}: {v:.4g} vs baseline {b:.4g} ({(v / b - 1) * 100:+.1f}%, tolerance {tolerance * 100:.0f}%)")
    clocks = result.get("clocks") or {}
    if any(r in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown") for r in clocks.get("reasons", [])):
        problems.append(f"{key}: measured under thermal or hardware slowdown; take it again")
    if base.get("config") and result.get("config") and base["config"].get("model") != result["config"].get("model"):
        problems.append(f"{key}: model {result['config'].get('model')} differs from the baseline's {base['config'].get('model')}")
    return problems


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("perf"); p.add_argument("--result", required=True); p.add_argument("--baseline", default=os.path.join(os.path.dirname(__file__), "perf_baseline.json")); p.add_argument("--tolerance", type=float, default=0.03)
    c = sub.add_parser("collectives"); c.add_argument("--layers", type=int, required=True); c.add_argument("--counted", type=int, required=True)
    a = ap.parse_args(argv)
    if a.cmd == "perf":
        with open(a.result) as f:
            lines = [l for l in f.read().splitlines() if l.strip().startswith("{")]
        problems = check_perf(json.loads(lines[-1]), json.load(open(a.baseline)), a.tolerance)
    else:
        problems = check_collectives(a.layers, a.counted)
    for pr in problems:
        print("gate: " + pr, file=sys.stderr)
    print(f"gate: {len(problems)} problem(s)")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
