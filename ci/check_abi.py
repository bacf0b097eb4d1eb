#!/usr/bin/env python
"""Static check of the C ABI between the native sources and their Python callers.

Every exported entry point (`extern "C"` functions named sfb_* in sparkflash_b200/csrc) is called from Python through
ctypes, which checks nothing: a wrapper that passes one argument too many or too few still "works" until the callee
reads a pointer from the wrong register.  This script parses both sides and compares the argument counts:

  * C side: the parameter list of every sfb_* definition inside an extern "C" region;
  * Python side: every call `<expr>.sfb_name(...)` in the package and the tests (ast), and every
    `.sfb_name.argtypes = [...]` declaration.

Exit status 1 on any mismatch or on a Python call of a symbol no source defines.

Reference: ci/check-m4-abi-size.sh, ci/verify-m4-abi-split.py and crates/sparkflash-kernels/src/m4_abi/scanner.rs of the
reference (a source scanner that proves the .cu signatures match the frozen launcher ABI).
"""
from __future__ import annotations

import ast
import re
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "sparkflash_b200" / "csrc"


def _strip_comments(src: str) -> str:
    src = re.sub(r"/\*.*?\*/", lambda m: " " * len(m.group(0)), src, flags=re.S)
    return re.sub(r"//[^\n]*", "", src)


def c_signatures() -> dict[str, tuple[int, str]]:
    """name -> (parameter count, file) for every sfb_* function defined (with a body) in the native sources."""
    out: dict[str, tuple[int, str]] = {}
    pat = re.compile(r"\b(sfb_[A-Za-z0-9_]+)\s*\(")
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cpp"))):
        src = _strip_comments(f.read_text())
        for m in pat.finditer(src):
            name = m.group(1)
            i = m.end()
            depth, j = 1, i
            while j < len(src) and depth:
                depth += {"(": 1, ")": -1}.get(src[j], 0)
                j += 1
            params = src[i:j - 1]
            k = j
            while k < len(src) and src[k] in " \t\r\n":
                k += 1
            if k >= len(src) or src[k] != "{":
                continue                      # a call or a declaration, not a definition
            # a definition is preceded by a return type on the same statement, not by an operator or a dot
            before = src[max(0, m.start() - 40):m.start()].rstrip()
            if not before or before[-1] in ".>=(,!&|+-*/" and not before.endswith("*"):
                continue
            p = params.strip()
            if p in ("", "void"):
                n = 0
            else:
                n, d = 1, 0
                for ch in p:
                    d += {"(": 1, "<": 1, ")": -1, ">": -1}.get(ch, 0)
                    if ch == "," and d == 0:
                        n += 1
            out.setdefault(name, (n, f.name))
    return out


def python_calls() -> list[tuple[str, int, str, int]]:
    """(symbol, argument count, file, line) of every `.sfb_*(...)` call; argtypes declarations count as calls of that arity."""
    found = []
    files = list((ROOT / "sparkflash_b200").rglob("*.py")) + list((ROOT / "tests").glob("*.py")) + [ROOT / "bench.py"]
    for f in files:
        try:
            tree = ast.parse(f.read_text())
        except SyntaxError as e:
            found.append(("<syntax error>", -1, str(f), e.lineno or 0))
            continue
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr.startswith("sfb_"):
                if any(isinstance(a, ast.Starred) for a in node.args):
                    continue
                found.append((node.func.attr, len(node.args), str(f.relative_to(ROOT)), node.lineno))
            if isinstance(node, ast.Assign) and len(node.targets) == 1:
                t = node.targets[0]
                if (isinstance(t, ast.Attribute) and t.attr == "argtypes" and isinstance(t.value, ast.Attribute)
                        and t.value.attr.startswith("sfb_") and isinstance(node.value, (ast.List, ast.Tuple))):
                    found.append((t.value.attr, len(node.value.elts), str(f.relative_to(ROOT)), node.lineno))
    return found


def main() -> int:
    sigs = c_signatures()
    bad = []
    for name, n, f, line in python_calls():
        if name not in sigs:
            bad.append(f"{f}:{line}: {name} is not defined in any native source")
        elif sigs[name][0] != n:
            bad.append(f"{f}:{line}: {name} called with {n} arguments, {sigs[name][1]} defines {sigs[name][0]}")
    for b in bad:
        print(b)
    print(f"checked {len(sigs)} native entry points against their Python callers: {len(bad)} problem(s)")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
