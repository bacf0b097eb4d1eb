"""Control panel: plan file, derived commands, hub cache and download (scripted fetcher, no network), node facts from
recorded text, stats history, supervisor.  Reference: crates/sparkflash-web/src tests (config, commands, hf, inspect, stats)."""
import hashlib
import json
import os
import signal

import pytest
from starlette.testclient import TestClient

from sparkflash_b200.serve import supervisor
from sparkflash_b200.web import app as webapp, hub, node, panel, stats


def test_plan_roundtrip_rules_and_commands(tmp_path):
    p = panel.Plan()
    p.model.synthetic = "reduced"; p.engine.world = 4; p.engine.moe_mode = "ep"; p.env["SFB_SEED"] = "7"
    p.paths.converted = str(tmp_path / "conv"); p.paths.pid_file = str(tmp_path / "serve.pid"); p.paths.log = str(tmp_path / "serve.log")
    q = panel.Plan.from_toml(p.to_toml())
    assert q.as_dict() == p.as_dict()
    assert q.launch_env()["SFB_MOE_MODE"] == "ep" and q.launch_env()["SFB_SEED"] == "7"
    assert not q.requires_conversion()                               # synthetic weights need no rank files
    launch = panel.serve_action_command(q, "launch")
    assert "sparkflash_b200.serve.supervisor" in launch.argv and "--gpus" in launch.argv and launch.argv[launch.argv.index("--gpus") + 1] == "4"
    assert "SFB_MOE_MODE=ep" in launch.display() and "--synthetic reduced" in launch.display()
    assert panel.serve_action_command(q, "stop").argv[3] == "stop"
    for bad in ("[engine]\nworld = 3\n", "[engine]\nworld = true\n", "[engine]\nnope = 1\n", "[env]\nPATH = \"x\"\n", "[env]\nSFB_NOPE = \"1\"\n",
                "[model]\nid = \"not a model\"\n", "[what]\na = 1\n", "x = = 1"):
        with pytest.raises(panel.PlanError):
            panel.Plan.from_toml(bad)
    # a real checkpoint: conversion is wanted until every rank file exists
    ck = tmp_path / "ck"; ck.mkdir()
    q.model.synthetic = ""; q.model.checkpoint = str(ck); q.model.id = "acme/flash"
    assert q.requires_conversion() and "--checkpoint" in panel.convert_command(q).argv
    d = q.converted_path(); d.mkdir(parents=True)
    for r in range(4):
        (d / f"rank{r}-of-4.sfb").write_bytes(b"x")
    assert not q.requires_conversion()
    assert [c.kind for c in panel.workflow(q)] == ["doctor", "launch"]


def _make_cached(cache, mid, model_type="deepseek_v41", shards=2, drop=None):
    snap = cache / hub.repo_folder(mid) / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    (cache / hub.repo_folder(mid) / "refs").mkdir()
    (cache / hub.repo_folder(mid) / "refs" / "main").write_text("abc123")
    (snap / "config.json").write_text(json.dumps({"model_type": model_type}))
    names = [f"model-{i:05d}-of-{shards:05d}.safetensors" for i in range(1, shards + 1)]
    (snap / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {f"t{i}": n for i, n in enumerate(names)}}))
    for n in names:
        if n != drop:
            (snap / n).write_bytes(b"\0" * 1000)
    return snap


def test_hub_cache_listing_and_preference(tmp_path):
    cache = tmp_path / "hub"; cache.mkdir()
    _make_cached(cache, "acme/flash")
    _make_cached(cache, "acme/broken", drop="model-00002-of-00002.safetensors")
    _make_cached(cache, "acme/other", model_type="llama")
    (cache / "datasets--x--y").mkdir()
    ms = {m.id: m for m in hub.list_cached(cache)}
    assert set(ms) == {"acme/flash", "acme/broken", "acme/other"}
    assert ms["acme/flash"].complete and ms["acme/flash"].family == "deepseek" and ms["acme/flash"].served_by == "deepseek-v4.1-flash"
    assert not ms["acme/broken"].complete and "missing" in ms["acme/broken"].problems[0]
    assert ms["acme/other"].family is None and "no engine" in ms["acme/other"].problems[0]
    assert hub.preferred_cached(list(ms.values())).id == "acme/flash"
    assert hub.resolve(cache, "acme/flash").name == "abc123" and hub.lookup(cache, "nope/none") is None
    assert hub.is_model_id("acme/flash") and not hub.is_model_id("/abs/path") and not hub.is_model_id("a/b/c")
    hub.judge_cached(ms.values(), world=8)
    assert ms["acme/flash"].fit["fits"] is True
    assert {f["family"] for f in hub.families()} >= {"deepseek", "qwen", "glm", "inkling", "dory"}


class FakeHub:
    """fetch(url, headers) over an in-memory repository; honours Range; can cut a body short once."""

    def __init__(self, files: dict[str, bytes], sha="feedbeef"):
        self.files, self.sha, self.calls, self.cut = files, sha, [], None

    def __call__(self, url, headers):
        self.calls.append((url, dict(headers)))
        if "/api/models/" in url:
            sib = [{"rfilename": n, "size": len(b), "lfs": {"sha256": hashlib.sha256(b).hexdigest(), "size": len(b)}} for n, b in self.files.items()]
            return 200, {}, iter([json.dumps({"sha": self.sha, "config": {"model_type": "deepseek_v41"}, "siblings": sib}).encode()])
        name = url.split(f"/resolve/{self.sha}/")[1]
        body = self.files[name]
        start = int(headers["Range"].split("=")[1].rstrip("-")) if "Range" in headers else 0
        data = body[start:]
        if self.cut == name:
            self.cut = None
            data = data[:len(data) // 2]
        return (206 if start else 200), {}, iter([data[i:i + 7] for i in range(0, len(data), 7)])


def test_download_resumes_and_verifies(tmp_path):
    files = {"config.json": b'{"model_type": "deepseek_v41"}', "model-00001-of-00001.safetensors": bytes(range(256)) * 4,
             "tokenizer.json": b"{}", "README.md": b"skip me", "../evil.json": b"{}"}
    fh = FakeHub(files)
    fh.cut = "model-00001-of-00001.safetensors"
    cache = tmp_path / "hub"
    with pytest.raises(RuntimeError, match="got 512 bytes"):
        hub.download("acme/flash", cache, fetch=fh)
    part = cache / hub.repo_folder("acme/flash") / "snapshots" / "feedbeef" / "model-00001-of-00001.safetensors.incomplete"
    assert part.stat().st_size == 512
    seen = []
    snap = hub.download("acme/flash", cache, fetch=fh, progress=seen.append)
    assert any(h.get("Range") == "bytes=512-" for _, h in fh.calls)          # resumed, not restarted
    assert (snap / "model-00001-of-00001.safetensors").read_bytes() == files["model-00001-of-00001.safetensors"]
    assert not (snap / "README.md").exists() and not (snap.parent / "evil.json").exists() and not part.exists()
    assert seen and seen[-1]["total"] == sum(len(files[n]) for n in ("config.json", "model-00001-of-00001.safetensors", "tokenizer.json"))
    assert hub.lookup(cache, "acme/flash").complete
    n = len(fh.calls)
    hub.download("acme/flash", cache, fetch=fh)                              # everything present: only the metadata call
    assert len(fh.calls) == n + 1
    files["tokenizer.json"] = b"{ }"                                         # the hub's copy changed size: fetched again
    hub.download("acme/flash", cache, fetch=fh)
    assert (snap / "tokenizer.json").read_bytes() == b"{ }"
    with pytest.raises(ValueError):
        hub.inspect("not-an-id", fh)


TOPO = """\tGPU0\tGPU1\tGPU2\tGPU3\tNIC0\tCPU Affinity\tNUMA Affinity
GPU0\t X \tNV18\tNV18\tNV18\tSYS\t0-55\t0
GPU1\tNV18\t X \tNV18\tNV18\tSYS\t0-55\t0
GPU2\tNV18\tNV18\t X \tPIX\tSYS\t56-111\t1
GPU3\tNV18\tNV18\tPIX\t X \tSYS\t56-111\t1
NIC0\tSYS\tSYS\tSYS\tSYS\t X

Legend:
"""
CSV = "\n".join(f"{i}, NVIDIA B200, 183359, {183000 if i else 90000}, 10.0, 580.159" for i in range(4))


def test_node_facts_and_setup_report(tmp_path):
    def run(argv):
        return TOPO if "topo" in argv else CSV
    f = node.gather(run=run, paths=[str(tmp_path / "conv")])
    assert len(f.gpus) == 4 and f.driver == "580.159" and f.links[(0, 1)] == "NV18" and f.links[(2, 3)] == "PIX"
    p = panel.Plan(); p.model.synthetic = "reduced"; p.engine.world = 2; p.engine.lanes = 4
    rep = node.analyze(p, f)
    kinds = {x.check: x.severity for x in rep.findings}
    assert kinds["gpus"] == "ok" and kinds["nvlink"] == "ok" and kinds["memory"] == "warn" and kinds["fit"] == "ok"
    p.engine.world = 4
    rep = node.analyze(p, f)
    bad = [x for x in rep.findings if x.check == "nvlink"][0]
    assert bad.severity == "fail" and "PIX" in bad.message and not rep.ok()
    p.engine.world = 8
    assert [x for x in node.analyze(p, f).findings if x.check == "gpus"][0].severity == "fail"


def test_stats_history_rates_downsampling_and_idle_flush(tmp_path):
    now = [1000.0]
    h = stats.History(interval_s=1.0, history_s=100.0, flush_s=10.0, path=tmp_path / "s.json", clock=lambda: now[0])
    tok = 0
    for i in range(50):
        now[0] += 1.0
        tok += 40
        h.add({"generated_tokens": tok, "scheduler": {"running": 2 if i < 45 else 0, "waiting": 0}})
        if i < 45:
            assert not (tmp_path / "s.json").exists()                       # never written while requests run
    assert (tmp_path / "s.json").exists()
    pts = h.window(100, points=10)
    assert len(pts) == 10 and all(abs(p["tok_s"] - 40) < 1e-6 for p in pts[1:]) and pts[-1]["tokens_total"] == tok
    assert h.summary(20)["tok_s_peak"] == pytest.approx(40)
    h.add({"generated_tokens": 5, "scheduler": {"running": 0, "waiting": 0}})   # a restart: the counter went back, no negative rate
    assert h.window(5)[-1]["tok_s"] == 0
    assert h.sample(lambda: (_ for _ in ()).throw(OSError("down"))) is None and h.errors == 1
    h2 = stats.History(interval_s=1.0, history_s=100.0, path=tmp_path / "s.json", clock=lambda: now[0])
    assert len(h2.ring) >= 45                                                # history survives a restart of the panel


def test_supervisor_records_the_group_and_signals_exactly_it(tmp_path):
    pidf, log = tmp_path / "run" / "serve.pid", tmp_path / "run" / "serve.log"
    started = []

    class P:
        pid = os.getpgid(0)                                                  # a process group that is certainly alive: ours

    def popen(argv, **kw):
        started.append((argv, kw))
        return P()
    rep = supervisor.launch(pidf, 4, log, 29999, ["--synthetic", "reduced"], popen=popen)
    assert rep["ok"] and "--nproc-per-node=4" in rep["argv"] and started[0][1]["start_new_session"] is True
    assert supervisor.launch(pidf, 4, log, 29999, [], popen=popen)["ok"] is False          # already running
    assert supervisor.status(pidf)["alive"] is True
    sent = []
    rep = supervisor.stop(pidf, wait_s=0.3, kill=lambda pg, sig: sent.append((pg, sig)))
    assert sent == [(P.pid, signal.SIGTERM)] and rep["ok"] is False         # our own group does not exit
    pidf.write_text(json.dumps({"pgid": 2 ** 22 - 3}))                       # a group that does not exist
    assert "stale" in supervisor.stop(pidf)["state"] and not pidf.exists()
    assert supervisor.command_line(1, 1, ["--mock"])[1:4] == ["-m", "sparkflash_b200", "serve"]


def test_panel_routes(tmp_path):
    cache = tmp_path / "hub"; cache.mkdir()
    _make_cached(cache, "acme/flash")
    planf = tmp_path / "plan.toml"
    facts = node.gather(run=lambda argv: TOPO if "topo" in argv else CSV)
    c = TestClient(webapp.create_app(plan_path=str(planf), facts_source=lambda: facts, fetch=FakeHub({"config.json": b"{}"})))
    p = panel.Plan(); p.model.id = "acme/flash"; p.engine.world = 2; p.paths.hub_cache = str(cache); p.paths.converted = str(tmp_path / "conv")
    r = c.put("/api/plan", content=p.to_toml())
    assert r.status_code == 200 and r.json()["requires_conversion"] is True and planf.exists()
    assert c.put("/api/plan", content="[engine]\nworld = 5\n").status_code == 400
    cmds = c.get("/api/commands").json()
    assert [w["kind"] for w in cmds["workflow"]] == ["doctor", "convert", "launch"] and "supervisor" in cmds["stop"]["display"]
    hubr = c.get("/api/hub").json()
    assert hubr["preferred"] == "acme/flash" and hubr["models"][0]["fit"]["world"] == 2
    assert c.get("/api/hub/inspect/acme/flash").json()["cached"]["complete"] is True
    assert c.get("/api/hub/inspect/bad id").status_code == 400
    setup = c.get("/api/setup").json()
    assert any(f["check"] == "convert" and f["severity"] == "warn" for f in setup["report"]["findings"])
    assert c.post("/api/run", json={"kind": "rm -rf"}).status_code == 400
    assert c.get("/api/stats/history").json()["summary"]["samples"] == 0
