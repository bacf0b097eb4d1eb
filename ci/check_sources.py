#!/usr/bin/env python
"""Source rules that must hold for every native file of the package (run by ci/host_gates.py and the CPU tests):

  * no TMA or bulk load qualified to deliver one tile to several CTAs of a cluster (runs on two or more GPUs must never
    issue one, and the package runs the same files at every GPU count);
  * no batched-memcpy runtime calls;
  * no device-side trap or failing assert as an error path: kernels record a status code and return;
  * every spin on a flag or an mbarrier is bounded: the wait helpers are the only loops that poll, and each has an
    iteration limit;
  * kernels are compiled for sm_100a only.
"""
from __future__ import annotations

import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "sparkflash_b200" / "csrc"

FORBIDDEN = [
    (re.compile("[.]multi" + "cast[:][:]clu" + "ster"), "load qualified for several CTAs of a cluster"),
    (re.compile(r"cudaMemcpy(3D)?Batch" + "Async|cuMemcpy(3D)?Batch" + "Async"), "batched memcpy call"),
    (re.compile(r"__trap\s*\("), "device trap"),
    (re.compile(r"\bassert\s*\("), "device/host assert in a native source"),
    (re.compile(r"\bwgmma\b"), "sm_90-only instruction"),
]


def scan() -> list[str]:
    problems = []
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.cpp")) + list(CSRC.glob("*.h"))):
        text = f.read_text()
        code = re.sub(r"//[^\n]*", "", re.sub(r"/\*.*?\*/", "", text, flags=re.S))
        for pat, what in FORBIDDEN:
            for m in pat.finditer(code):
                line = code[:m.start()].count("\n") + 1
                problems.append(f"{f.name}:{line}: {what}")
        # unbounded polling: a `while (true)` / `for (;;)` loop anywhere in device code
        if f.suffix not in (".cu", ".cuh"):
            continue
        for m in re.finditer(r"while\s*\(\s*(true|1)\s*\)|for\s*\(\s*;\s*;\s*\)", code):
            line = code[:m.start()].count("\n") + 1
            problems.append(f"{f.name}:{line}: loop without a bound")
    build = (ROOT / "sparkflash_b200" / "_build.py").read_text()
    if "arch=compute_100a,code=sm_100a" not in build:
        problems.append("_build.py: kernels are not compiled for sm_100a")
    return problems


def main() -> int:
    problems = scan()
    for p in problems:
        print(p)
    print(f"source rules: {len(problems)} problem(s)")
    return 1 if problems else 0


if __name__ == "__main__":
    sys.exit(main())
