"""In-tree native build.

Two shared libraries with a plain C ABI (loaded through ctypes, see ``_lib.py``):

* ``lib/libsfb_host.so``  - g++: codecs, CPU oracle ops, scheduler core, lane planner, radix cache,
  constrained-decoding automaton, tool-call parser, Engram hash, rank-file converter/loader.
* ``lib/libsfb_cuda.so``  - nvcc for sm_100a only: every device kernel and its launcher, the
  symmetric-memory helpers and the lane (virtual memory) allocator.

Objects are rebuilt only when the hash of the source (plus headers and flags) changes, so importing
the package on a machine that received the built tree does not compile anything.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "lib"
OBJDIR = ROOT / "lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
    "-Xcompiler", "-Wno-unused-function",
]
if os.environ.get("SFB_KERNEL_MARKS") == "1":      # in-kernel phase marks (utils/kernel_marks.py): a measurement build
    NVCC_FLAGS.append("-DSFB_KERNEL_MARKS")
GXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("SFB_NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set SFB_NVCC)")


def _headers_digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _digest(src: Path, flags: list[str], hdr: str) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    h.update(" ".join(flags).encode())
    h.update(hdr.encode())
    return h.hexdigest()


def _compile_one(cmd: list[str], src: Path, obj: Path, stamp: Path, digest: str, verbose: bool) -> str:
    if obj.exists() and stamp.exists() and stamp.read_text() == digest:
        return f"[up-to-date] {src.name}"
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = OBJDIR / (src.name + ".log")
    log.write_text(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    if verbose:
        sys.stderr.write(r.stderr)
    return f"[built] {src.name}"


def build(verbose: bool = False, force: bool = False) -> dict[str, Path]:
    """Compile every native source for sm_100a / the host and link both libraries."""
    LIBDIR.mkdir(exist_ok=True)
    OBJDIR.mkdir(exist_ok=True)
    hdr = _headers_digest()
    nvcc = _nvcc()
    cuda_srcs = sorted(CSRC.rglob("*.cu"))
    host_srcs = sorted(CSRC.rglob("*.cpp"))
    jobs = []
    cuda_objs, host_objs = [], []
    for s in cuda_srcs:
        o = OBJDIR / (s.stem + ".cu.o")
        cuda_objs.append(o)
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
        jobs.append((cmd, s, o, OBJDIR / (s.stem + ".cu.stamp"), _digest(s, NVCC_FLAGS, hdr)))
    for s in host_srcs:
        o = OBJDIR / (s.stem + ".cpp.o")
        host_objs.append(o)
        cmd = ["g++", *GXX_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)]
        jobs.append((cmd, s, o, OBJDIR / (s.stem + ".cpp.stamp"), _digest(s, GXX_FLAGS, hdr)))
    if force:
        for j in jobs:
            if j[3].exists():
                j[3].unlink()
    with ThreadPoolExecutor(max_workers=max(2, (os.cpu_count() or 4))) as ex:
        results = list(ex.map(lambda j: _compile_one(*j, verbose), jobs))
    rebuilt = any(r.startswith("[built]") for r in results)
    if verbose:
        print("\n".join(results))
    out = {"host": LIBDIR / "libsfb_host.so", "cuda": LIBDIR / "libsfb_cuda.so"}
    if rebuilt or not out["host"].exists():
        subprocess.run(["g++", "-shared", "-o", str(out["host"]), *map(str, host_objs), "-pthread"],
                       check=True)
    if rebuilt or not out["cuda"].exists():
        subprocess.run([nvcc, "-shared", "-o", str(out["cuda"]), *map(str, cuda_objs),
                        "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"],
                       check=True)
    return out


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, as printed by ``-Xptxas -v`` at build."""
    out = []
    for log in sorted(OBJDIR.glob("*.cu.log")):
        out.append(f"== {log.name}")
        out.append(log.read_text())
    return "\n".join(out)


if __name__ == "__main__":
    libs = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    for k, v in libs.items():
        print(k, v, v.stat().st_size)
