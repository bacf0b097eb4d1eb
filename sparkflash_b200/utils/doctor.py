"""``doctor``: read-only checks of the box before serving (reference: crates/sparkflash-cli doctor subcommand;
docs/serving.md).  Nothing here changes a setting of a GPU: clocks, power limits and modes are only read."""
from __future__ import annotations

import os
import shutil
from dataclasses import dataclass


@dataclass
class Check:
    name: str
    ok: bool
    detail: str
    fatal: bool = True


def run_checks(nvml=None, need_gpus: int = 1, weights_dir: str | None = None, world: int = 1) -> list[Check]:
    """``nvml``: an object with the pynvml query functions (a fake in tests)."""
    out: list[Check] = []
    from .. import _build
    libdir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
    for lib in ("libsfb_cuda.so", "libsfb_host.so"):
        p = os.path.join(libdir, lib)
        out.append(Check(f"native library {lib}", os.path.exists(p), p if os.path.exists(p) else "missing: run python -m sparkflash_b200._build"))
    out.append(Check("nvcc", shutil.which("nvcc") is not None or os.path.exists("/usr/local/cuda/bin/nvcc"), "needed only to rebuild the kernels", fatal=False))
    try:
        if nvml is None:
            import pynvml as nvml
        nvml.nvmlInit()
        n = nvml.nvmlDeviceGetCount()
        out.append(Check("GPU count", n >= need_gpus, f"{n} visible, {need_gpus} needed"))
        drv = nvml.nvmlSystemGetDriverVersion()
        out.append(Check("driver", True, drv if isinstance(drv, str) else drv.decode(), fatal=False))
        for i in range(min(n, max(need_gpus, 1))):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            name = nvml.nvmlDeviceGetName(h)
            name = name if isinstance(name, str) else name.decode()
            major, minor = nvml.nvmlDeviceGetCudaComputeCapability(h)
            out.append(Check(f"gpu{i} architecture", (major, minor) == (10, 0), f"{name} sm_{major}{minor} (kernels are built for sm_100a only)"))
            mem = nvml.nvmlDeviceGetMemoryInfo(h)
            out.append(Check(f"gpu{i} memory", mem.total >= 170 * 2 ** 30, f"{mem.free / 2 ** 30:.0f} GiB free of {mem.total / 2 ** 30:.0f}", fatal=False))
            sm, mx = nvml.nvmlDeviceGetClockInfo(h, 1), nvml.nvmlDeviceGetMaxClockInfo(h, 1)
            out.append(Check(f"gpu{i} SM clock", True, f"{sm} MHz now, {mx} MHz max (read only)", fatal=False))
            try:
                reasons = nvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                bad = reasons & (0x8 | 0x40 | 0x20)        # hw slowdown, hw thermal, sw thermal
                out.append(Check(f"gpu{i} throttle", bad == 0, f"reasons mask 0x{reasons:x}", fatal=False))
            except Exception:
                pass
    except Exception as e:
        out.append(Check("NVML", False, f"{type(e).__name__}: {e}"))
    try:
        import torch
        import torch.distributed as dist
        out.append(Check("torch CUDA", torch.cuda.is_available(), torch.__version__))
        out.append(Check("NCCL backend", dist.is_nccl_available(), "torch.distributed", fatal=world > 1))
        if torch.cuda.is_available() and world > 1:
            ok = all(torch.cuda.can_device_access_peer(0, j) for j in range(1, min(world, torch.cuda.device_count())))
            out.append(Check("peer access", ok, "GPU 0 can map its peers' memory (needed by the fused collectives)"))
    except Exception as e:
        out.append(Check("torch", False, f"{type(e).__name__}: {e}"))
    if weights_dir:
        from ..weights.convert import MANIFEST, rank_path
        man = os.path.join(weights_dir, MANIFEST)
        out.append(Check("weights manifest", os.path.exists(man), man))
        for r in range(world):
            p = rank_path(weights_dir, r, world)
            out.append(Check(f"rank file {r}", os.path.exists(p), p))
    return out


def report(checks: list[Check]) -> tuple[str, bool]:
    lines, ok = [], True
    for c in checks:
        mark = "ok  " if c.ok else ("FAIL" if c.fatal else "warn")
        ok = ok and (c.ok or not c.fatal)
        lines.append(f"[{mark}] {c.name}: {c.detail}")
    return "\n".join(lines), ok
