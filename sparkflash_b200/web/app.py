"""Control panel backend: node discovery (local GPUs through NVML, read only), the fit estimator, the plan file with
its derived command lines, the hub cache and downloads, node facts with a setup report, job records for the operator
actions, and serving statistics with history.  ``python -m sparkflash_b200.web.app --port 8080 [--plan plan.toml]``;
``python -m sparkflash_b200.web.app download <org/name> --cache <dir>`` fetches a checkpoint into the hub cache.
Reference: crates/sparkflash-web/src/{api,commands,config,discovery,fit,hf,inspect,jobs,run,stats}.rs (docs/web.md)."""
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
from . import fit, hub, node, panel
from . import stats as stats_mod

PAGE = """<!doctype html><title>sparkflash_b200</title><h1>sparkflash_b200 control panel</h1>
<p>JSON endpoints: <a href=/api/nodes>/api/nodes</a>, <a href="/api/fit?world=8&context=131072&lanes=32">/api/fit</a>,
<a href=/api/jobs>/api/jobs</a>, <a href=/api/stats>/api/stats</a>, <a href=/api/stats/history>/api/stats/history</a>,
<a href=/api/plan>/api/plan</a>, <a href=/api/commands>/api/commands</a>, <a href=/api/hub>/api/hub</a>, <a href=/api/setup>/api/setup</a></p>"""


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

    def start(self, argv: list[str], env: dict | None = None, raw: bool = False, kind: str = "convert") -> str:
        """``argv`` are arguments of ``python -m sparkflash_b200`` unless ``raw`` (then the full command line)."""
        jid = uuid.uuid4().hex[:12]
        rec = {"id": jid, "kind": kind, "argv": argv, "state": "running", "progress": None, "started": time.time(), "log": []}
        self.jobs[jid] = rec
        full = list(argv) if raw else [sys.executable, "-m", "sparkflash_b200", *argv]
        import os
        child_env = {**os.environ, **(env or {})}

        def run():
            p = subprocess.Popen(full, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=child_env)
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


def create_app(server_url: str = "http://127.0.0.1:8000", nvml=None, plan_path: str | None = None, facts_source=None,
               fetch=hub.url_fetch, history: "stats_mod.History | None" = None) -> Starlette:
    jobs = Jobs()
    state = {"plan": panel.Plan.load(plan_path) if plan_path and __import__("os").path.exists(plan_path) else panel.Plan()}
    if plan_path is None or not __import__("os").path.exists(plan_path or ""):
        state["plan"].web.server_host, state["plan"].web.server_port = _split_url(server_url)
    hist = history or stats_mod.History(state["plan"].stats.interval_s, state["plan"].stats.history_s, state["plan"].stats.flush_s)

    def facts():
        return facts_source() if facts_source else node.gather(paths=[str(panel.expand(state["plan"].paths.converted))])

    async def plan_route(request: Request):
        if request.method == "PUT":
            try:
                new = panel.Plan.from_toml((await request.body()).decode())
            except (panel.PlanError, UnicodeDecodeError) as e:
                return JSONResponse({"error": str(e)}, status_code=400)
            state["plan"] = new
            if plan_path:
                new.save(plan_path)
        p = state["plan"]
        return JSONResponse({"plan": p.as_dict(), "toml": p.to_toml(), "requires_conversion": p.requires_conversion(),
                             "conversion_scope": p.conversion_scope(), "launch_env": p.launch_env()})

    async def commands_route(request: Request):
        p = state["plan"]
        out = {"workflow": [c.as_dict() for c in panel.workflow(p)]}
        for a in panel.SERVE_ACTIONS:
            out[a] = panel.serve_action_command(p, a).as_dict()
        return JSONResponse(out)

    async def run_route(request: Request):
        """Run one derived command as a job: {"kind": "doctor" | "download" | "convert" | "launch" | "stop" | "status"}.
        Only command lines derived from the plan are ever run; the request cannot supply its own."""
        kind = (await request.json()).get("kind")
        p = state["plan"]
        try:
            spec = {"doctor": panel.doctor_command, "download": panel.download_command, "convert": panel.convert_command,
                    "inspect": panel.inspect_command}[kind](p) if kind not in panel.SERVE_ACTIONS else panel.serve_action_command(p, kind)
        except KeyError:
            return JSONResponse({"error": f"unknown command kind {kind!r}"}, status_code=400)
        except panel.PlanError as e:
            return JSONResponse({"error": str(e)}, status_code=409)
        return JSONResponse({"id": jobs.start(spec.argv, spec.env, raw=True, kind=spec.kind), "display": spec.display()})

    async def hub_route(request: Request):
        p = state["plan"]
        models = hub.list_cached(p.hub_cache_dir())
        hub.judge_cached(models, p.engine.world)
        pref = hub.preferred_cached(models, p.model.id)
        return JSONResponse({"cache": str(p.hub_cache_dir()), "models": [m.as_dict() for m in models], "preferred": pref.id if pref else None,
                             "families": hub.families()})

    async def hub_inspect(request: Request):
        mid = request.path_params["model_id"]
        try:
            return JSONResponse(hub.inspect(mid, fetch, cache=state["plan"].hub_cache_dir(), world=state["plan"].engine.world))
        except ValueError as e:
            return JSONResponse({"error": str(e)}, status_code=400)
        except Exception as e:                                     # noqa: BLE001 - offline or unknown model
            return JSONResponse({"error": f"{type(e).__name__}: {e}"}, status_code=502)

    async def setup_route(request: Request):
        f = facts()
        return JSONResponse({"facts": f.as_dict(), "report": node.analyze(state["plan"], f).as_dict()})

    async def history_route(request: Request):
        qp = request.query_params
        return JSONResponse({"summary": hist.summary(float(qp.get("summary_s", 60))),
                             "points": hist.window(float(qp.get("seconds", 3600)), int(qp.get("points", 300)))})

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

    app = Starlette(routes=[Route("/", index), Route("/api/nodes", nodes), Route("/api/fit", fit_route),
                            Route("/api/jobs", jobs_route, methods=["GET", "POST"]), Route("/api/stats", stats),
                            Route("/api/plan", plan_route, methods=["GET", "PUT"]), Route("/api/commands", commands_route),
                            Route("/api/run", run_route, methods=["POST"]), Route("/api/hub", hub_route),
                            Route("/api/hub/inspect/{model_id:path}", hub_inspect), Route("/api/setup", setup_route),
                            Route("/api/stats/history", history_route)])
    app.state.history, app.state.jobs, app.state.panel = hist, jobs, state
    return app


def _split_url(url: str) -> tuple[str, int]:
    from urllib.parse import urlparse
    u = urlparse(url)
    return u.hostname or "127.0.0.1", u.port or 8000


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv[:1] == ["download"]:
        ap = argparse.ArgumentParser(prog="sparkflash_b200.web.app download")
        ap.add_argument("model_id"); ap.add_argument("--cache", default=str(hub.default_cache_dir()))
        ap.add_argument("--endpoint", default="https://huggingface.co"); ap.add_argument("--token-env", default="HF_TOKEN")
        a = ap.parse_args(argv[1:])
        import os
        last = [0.0]

        def progress(p):
            if time.time() - last[0] > 1.0:
                last[0] = time.time()
                print("@progress " + json.dumps(p), flush=True)
        snap = hub.download(a.model_id, hub.Path(a.cache), endpoint=a.endpoint, token=os.environ.get(a.token_env), progress=progress)
        print(json.dumps({"snapshot": str(snap)}))
        return 0
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1"); ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--server", default="http://127.0.0.1:8000"); ap.add_argument("--plan", help="TOML plan file (created on first save)")
    a = ap.parse_args(argv)
    import uvicorn
    app = create_app(a.server, plan_path=a.plan)
    app.state.history.start(stats_mod.http_source(app.state.panel["plan"].server_url()))
    uvicorn.run(app, host=a.host, port=a.port, log_level="warning")
    return 0


if __name__ == "__main__":
    sys.exit(main())
