"""Start, stop and query a serving group on this node.

``launch`` starts the ranks detached from the caller (a session of their own, output to a log file) — one process when
``--gpus 1``, else ``torch.distributed.run`` with one process per GPU on 127.0.0.1 — and records the leader's process id,
which is also the id of the group's process group.  ``stop`` sends SIGTERM to exactly that recorded group (rank 0 drains
its requests, says goodbye on the control channel, the followers leave) and waits for it to end; nothing is ever
signalled by name or pattern.  ``status`` says whether the recorded group is alive and whether the server answers
``/health``.

Reference behaviour: scripts/serve-four-node.sh (launch | stop | status), crates/sparkflash-web/src/commands.rs:227-300.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
import urllib.request
from pathlib import Path


def _read_pid(pid_file: Path) -> int | None:
    try:
        rec = json.loads(pid_file.read_text())
        return int(rec["pgid"])
    except (OSError, ValueError, KeyError, json.JSONDecodeError):
        return None


def _alive(pgid: int) -> bool:
    try:
        os.killpg(pgid, 0)
        return True
    except ProcessLookupError:
        return False
    except PermissionError:
        return True


def command_line(gpus: int, master_port: int, serve_args: list[str]) -> list[str]:
    if gpus == 1:
        return [sys.executable, "-m", "sparkflash_b200", "serve", *serve_args]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
            "--master-port", str(master_port), "-m", "sparkflash_b200", "serve", *serve_args]


def launch(pid_file: Path, gpus: int, log: Path, master_port: int, serve_args: list[str], popen=subprocess.Popen) -> dict:
    old = _read_pid(pid_file)
    if old is not None and _alive(old):
        return {"ok": False, "error": f"a serving group is already running (process group {old})"}
    pid_file.parent.mkdir(parents=True, exist_ok=True)
    log.parent.mkdir(parents=True, exist_ok=True)
    argv = command_line(gpus, master_port, serve_args)
    with open(log, "ab") as out:
        p = popen(argv, stdout=out, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL, start_new_session=True)
    pid_file.write_text(json.dumps({"pgid": p.pid, "argv": argv, "started": time.time(), "log": str(log), "gpus": gpus}))
    return {"ok": True, "pgid": p.pid, "argv": argv, "log": str(log)}


def stop(pid_file: Path, wait_s: float = 60.0, kill=os.killpg) -> dict:
    pgid = _read_pid(pid_file)
    if pgid is None:
        return {"ok": True, "state": "not running (no record)"}
    if not _alive(pgid):
        pid_file.unlink(missing_ok=True)
        return {"ok": True, "state": "not running (stale record removed)"}
    kill(pgid, signal.SIGTERM)
    t0 = time.monotonic()
    while time.monotonic() - t0 < wait_s:
        if not _alive(pgid):
            pid_file.unlink(missing_ok=True)
            return {"ok": True, "state": "stopped", "seconds": round(time.monotonic() - t0, 1)}
        time.sleep(0.2)
    return {"ok": False, "state": f"process group {pgid} still draining after {wait_s:.0f}s"}


def status(pid_file: Path, url: str | None = None) -> dict:
    pgid = _read_pid(pid_file)
    out = {"recorded": pgid is not None, "alive": bool(pgid is not None and _alive(pgid)), "pgid": pgid}
    if url:
        try:
            with urllib.request.urlopen(url.rstrip("/") + "/health", timeout=2) as r:
                out["health"] = json.loads(r.read())
                out["serving"] = True
        except Exception as e:                                     # noqa: BLE001 - any failure means "not serving"
            out["serving"] = False
            out["health_error"] = f"{type(e).__name__}: {e}"
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="sparkflash_b200.serve.supervisor")
    ap.add_argument("action", choices=["launch", "stop", "status"])
    ap.add_argument("--pid-file", default=os.path.expanduser("~/.cache/sparkflash_b200/serve.pid"))
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--log", default=os.path.expanduser("~/.cache/sparkflash_b200/serve.log"))
    ap.add_argument("--master-port", type=int, default=29601)
    ap.add_argument("--url")
    ap.add_argument("--wait", type=float, default=60.0)
    ap.add_argument("serve_args", nargs=argparse.REMAINDER, help="after --: arguments of `sparkflash_b200 serve`")
    a = ap.parse_args(argv)
    rest = a.serve_args[1:] if a.serve_args[:1] == ["--"] else a.serve_args
    if a.action == "launch":
        rep = launch(Path(a.pid_file), a.gpus, Path(a.log), a.master_port, rest)
    elif a.action == "stop":
        rep = stop(Path(a.pid_file), a.wait)
    else:
        rep = status(Path(a.pid_file), a.url)
    print(json.dumps(rep))
    return 0 if rep.get("ok", True) else 1


if __name__ == "__main__":
    sys.exit(main())
