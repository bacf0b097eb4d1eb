"""Control panel backend: node discovery (local GPUs through NVML, read only), the fit estimator, job records for
convert runs, and a stats proxy to a running server.  ``python -m sparkflash_b200.web.app --port 8080``.
Reference: crates/sparkflash-web/src/{api,discovery,fit,jobs,stats}.rs (docs/web.md)."""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
import threading
import time
import urllib.request
import uuid

from starlette.applications import Starlette
from starlette.requests import Request
from starlette.responses import HTMLResponse, JSONResponse
from starlette.routing import Route

from ..config import full_config, reduced_config
from . import fit

PAGE = """<!doctype html><title>sparkflash_b200</title><h1>sparkflash_b200 control panel</h1>
<p>JSON endpoints: <a href=/api/nodes>/api/nodes</a>, <a href="/api/fit?world=8&context=131072&lanes=32">/api/fit</a>,
<a href=/api/jobs>/api/jobs</a>, <a href=/api/stats>/api/stats</a></p>"""


def discover(nvml=None) -> list[dict]:
    out = []
    try:
        if nvml is None:
            import pynvml as nvml
        nvml.nvmlInit()
        for i in range(nvml.nvmlDeviceGetCount()):
            h = nvml.nvmlDeviceGetHandleByIndex(i)
            name = nvml.nvmlDeviceGetName(h)
            mem = nvml.nvmlDeviceGetMemoryInfo(h)
            out.append({"index": i, "name": name if isinstance(name, str) else name.decode(), "memory_gb": round(mem.total / 1e9, 1),
                        "free_gb": round(mem.free / 1e9, 1), "sm": "%d%d" % tuple(nvml.nvmlDeviceGetCudaComputeCapability(h))})
    except Exception as e:
        out.append({"error": f"{type(e).__name__}: {e}"})
    return out


class Jobs:
    def __init__(self):
        self.jobs: dict[str, dict] = {}

    def start(self, argv: list[str]) -> str:
        jid = uuid.uuid4().hex[:12]
        rec = {"id": jid, "argv": argv, "state": "running", "progress": None, "started": time.time(), "log": []}
        self.jobs[jid] = rec

        def run():
            p = subprocess.Popen([sys.executable, "-m", "sparkflash_b200", *argv], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
            for line in p.stdout:
                line = line.rstrip()
                if line.startswith("@progress "):
                    rec["progress"] = json.loads(line[10:])
                else:
                    rec["log"] = (rec["log"] + [line])[-50:]
            rec["state"] = "done" if p.wait() == 0 else "failed"
            rec["finished"] = time.time()
        threading.Thread(target=run, daemon=True).start()
        return jid


def create_app(server_url: str = "http://127.0.0.1:8000", nvml=None) -> Starlette:
    jobs = Jobs()

    async def index(request: Request):
        return HTMLResponse(PAGE)

    async def nodes(request: Request):
        return JSONResponse({"nodes": [{"host": "localhost", "gpus": discover(nvml)}]})

    async def fit_route(request: Request):
        qp = request.query_params
        world, ctx, lanes = int(qp.get("world", 8)), int(qp.get("context", 131072)), int(qp.get("lanes", 32))
        experts = int(qp.get("experts", 0))
        cfg = reduced_config(experts, int(qp.get("layers", 40))) if experts else full_config()
        rep = fit.estimate(cfg, world, ctx, lanes, float(qp.get("gpu_gb", 180)), qp.get("engram", "0") == "1")
        return JSONResponse(rep.as_dict())

    async def jobs_route(request: Request):
        if request.method == "POST":
            body = await request.json()
            if body.get("kind") != "convert":
                return JSONResponse({"error": "only convert jobs are offered"}, status_code=400)
            argv = ["convert", "--checkpoint", body["checkpoint"], "--output-dir", body["output_dir"], "--tp-world-size", str(body.get("world", 1))]
            if body.get("synthetic"):
                argv += ["--synthetic", body["synthetic"]]
            return JSONResponse({"id": jobs.start(argv)})
        return JSONResponse({"jobs": [{k: v for k, v in j.items() if k != "log"} | {"log_tail": j["log"][-5:]} for j in jobs.jobs.values()]})

    async def stats(request: Request):
        try:
            with urllib.request.urlopen(server_url.rstrip("/") + "/v1/cluster/stats", timeout=2) as r:
                return JSONResponse(json.loads(r.read()))
        except Exception as e:
            return JSONResponse({"serving": False, "error": f"{type(e).__name__}: {e}"}, status_code=502)

    return Starlette(routes=[Route("/", index), Route("/api/nodes", nodes), Route("/api/fit", fit_route),
                             Route("/api/jobs", jobs_route, methods=["GET", "POST"]), Route("/api/stats", stats)])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1"); ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--server", default="http://127.0.0.1:8000")
    a = ap.parse_args(argv)
    import uvicorn
    uvicorn.run(create_app(a.server), host=a.host, port=a.port, log_level="warning")
    return 0


if __name__ == "__main__":
    sys.exit(main())
