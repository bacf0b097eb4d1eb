"""CLI, doctor (against a fake NVML), convert, settings, served benchmark client over the mock engine."""
import asyncio
import json
import types

import pytest

from sparkflash_b200 import cli, config as CF
from sparkflash_b200.utils import doctor


class FakeNvml:
    def __init__(self, n=2, cc=(10, 0), reasons=0):
        self.n, self.cc, self.reasons = n, cc, reasons
        self.writes = []

    def nvmlInit(self): pass
    def nvmlDeviceGetCount(self): return self.n
    def nvmlSystemGetDriverVersion(self): return "580.159"
    def nvmlDeviceGetHandleByIndex(self, i): return i
    def nvmlDeviceGetName(self, h): return "NVIDIA B200"
    def nvmlDeviceGetCudaComputeCapability(self, h): return self.cc
    def nvmlDeviceGetMemoryInfo(self, h): return types.SimpleNamespace(total=183359 * 2 ** 20, free=180000 * 2 ** 20)
    def nvmlDeviceGetClockInfo(self, h, k): return 1200
    def nvmlDeviceGetMaxClockInfo(self, h, k): return 1965
    def nvmlDeviceGetCurrentClocksEventReasons(self, h): return self.reasons

    def __getattr__(self, name):          # any setter the doctor might call would land here: it must call none
        if "Set" in name or "Reset" in name:
            raise AssertionError(f"doctor tried to change a GPU setting: {name}")
        raise AttributeError(name)


def test_doctor_reads_but_never_sets():
    checks = doctor.run_checks(FakeNvml(2), need_gpus=2)
    byname = {c.name: c for c in checks}
    assert byname["GPU count"].ok and byname["gpu0 architecture"].ok and byname["gpu1 throttle"].ok
    checks = doctor.run_checks(FakeNvml(1, cc=(9, 0), reasons=0x40), need_gpus=2)
    byname = {c.name: c for c in checks}
    assert not byname["GPU count"].ok and not byname["gpu0 architecture"].ok and not byname["gpu0 throttle"].ok
    text, ok = doctor.report(checks)
    assert not ok and "[FAIL] GPU count" in text and "[warn] gpu0 throttle" in text


def test_convert_cli_roundtrip(tmp_path, capsys):
    src, out = str(tmp_path / "ck"), str(tmp_path / "out")
    assert cli.main(["convert", "--synthetic", "tiny", "--checkpoint", src, "--output-dir", out, "--tp-world-size", "2"]) == 0
    text = capsys.readouterr().out
    assert text.count("@progress") == 2 and "wrote 2 rank file(s)" in text
    man = json.load(open(out + "/manifest.json"))
    assert man["world"] == 2 and man["ranks"]["1"]["verified"]
    assert cli.main(["convert", "--inspect", out + "/rank1-of-2.sfb", "--verify-weights"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["rank"] == 1 and rep["world"] == 2 and rep["verified"]
    # only one rank re-converted: the manifest keeps the other
    assert cli.main(["convert", "--checkpoint", src, "--output-dir", out, "--tp-world-size", "2", "--ranks", "0", "--no-verify"]) == 0
    man = json.load(open(out + "/manifest.json"))
    assert set(man["ranks"]) == {"0", "1"} and not man["ranks"]["0"]["verified"]
    with pytest.raises(ValueError, match="unknown key"):
        CF.config_from_hf({"dim": 256, "brand_new_knob": 1})


def test_models_table_and_settings(capsys, tmp_path):
    assert cli.main(["models"]) == 0
    out = capsys.readouterr().out
    assert "deepseek-v4.1-flash" in out and "inkling-2-small" in out and "dory-1.0-4b" in out
    s = CF.Settings().apply_env({"SFB_MAX_LANES": "8", "SFB_COLLECTIVE": "nccl", "HOME": "/x"})
    assert s.engine.max_lanes == 8 and s.parallel.collective == "nccl"
    with pytest.raises(ValueError, match="unknown setting"):
        CF.Settings().apply_env({"SFB_TYPO": "1"})
    with pytest.raises(ValueError):
        CF.Settings().apply_env({"SFB_COLLECTIVE": "mpi"})
    p = tmp_path / "s.toml"
    p.write_text("[engine]\nmax_rows = 32\n[parallel]\nmoe_mode = \"ep\"\n")
    s2 = CF.Settings().apply_dict(CF.load_toml(str(p)))
    assert s2.engine.max_rows == 32 and s2.digest() != CF.Settings().digest()
    with pytest.raises(ValueError):
        CF.Settings().apply_dict({"engine": {"nope": 1}})


def test_served_benchmark_client_over_mock():
    import httpx
    from sparkflash_b200.serve.bench_client import run_async
    from sparkflash_b200.serve.engine_api import MockEngine
    from sparkflash_b200.serve.server import Server
    from sparkflash_b200.serve.tokenizer import ByteTokenizer
    tok = ByteTokenizer()
    srv = Server(MockEngine(tok, lambda p: tok.encode("x" * 40), lanes=4, queue=8, delay=0.001))
    out = asyncio.run(run_async("http://t", 4, 8, 64, 32, transport=httpx.ASGITransport(app=srv.app)))
    assert out["ok"] == 8 and out["aggregate_tok_s"] > 0 and out["ttft_p50_s"] <= out["ttft_p99_s"]


def test_fit_estimator_and_control_panel(tmp_path):
    import time as _t
    from starlette.testclient import TestClient
    from sparkflash_b200.web import app as WA, fit
    full = CF.full_config()
    one = fit.estimate(full, 1, 131072, 32)
    eight = fit.estimate(full, 8, 1048576, 32)
    assert not one.fits and one.weights_gb > 180            # the whole model does not fit one GPU
    assert eight.fits and eight.weights_gb < 60 and eight.max_lanes_that_fit >= 32
    assert fit.estimate(CF.reduced_config(128, 40), 1, 65536, 16).fits
    assert fit.kv_bytes_per_lane(full, 1 << 20) > 20 * fit.kv_bytes_per_lane(full, 1 << 14) / 2
    c = TestClient(WA.create_app(nvml=FakeNvml(2)))
    assert len(c.get("/api/nodes").json()["nodes"][0]["gpus"]) == 2
    r = c.get("/api/fit?world=8&context=1048576&lanes=32").json()
    assert r["fits"] and r["world"] == 8
    assert c.get("/api/stats").status_code == 502            # nothing is serving
    jid = c.post("/api/jobs", json={"kind": "convert", "synthetic": "tiny", "checkpoint": str(tmp_path / "ck"), "output_dir": str(tmp_path / "o"), "world": 1}).json()["id"]
    for _ in range(200):
        j = [x for x in c.get("/api/jobs").json()["jobs"] if x["id"] == jid][0]
        if j["state"] != "running":
            break
        _t.sleep(0.1)
    assert j["state"] == "done" and j["progress"]["done"] == 1
    assert c.post("/api/jobs", json={"kind": "rm -rf"}).status_code == 400


def test_plan_and_inkling_subcommands(capsys):
    assert cli.main(["plan", "--world", "4", "--moe-mode", "ep"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert rep["world"] == 4 and rep["heads_per_rank"] == 16 and rep["gb_per_rank"] > 10
    assert set(rep["step_plans"]) >= {"1", "16", "1024"}
    assert cli.main(["inkling-tp4", "--world", "4", "--tokens", "5"]) == 0
    rep = json.loads(capsys.readouterr().out)
    assert set(rep["max_abs_vs_unsplit"]) == {"experts", "intermediate", "rows"}


def test_pack_engram_subcommand_resolves_its_packer():
    import inspect
    src = inspect.getsource(cli._pack_engram)
    assert "engram import store" in src
    from sparkflash_b200.engram import store
    assert hasattr(store, "pack")
