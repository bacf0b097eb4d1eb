"""Numerics registry, identity gates over the fake engine, perf and collective-count gates (reference:
scripts/tests/ unit tests of numerics.py, perf_regression_gate.py, check-collective-count.py)."""
import copy

from sparkflash_b200.gates import identity, numerics, perf


def test_registry_matches_the_oracle_and_detects_undeclared_changes(tmp_path):
    reg = numerics.load_registry()
    assert set(reg["config"]) >= {"tiny-csa2/tp1", "tiny-csa2/tp2"}
    one = {"config": {"tiny-csa2/tp2": reg["config"]["tiny-csa2/tp2"]}}
    assert numerics.check(one) == []
    fake = lambda model, world: "f" * 32
    bad = numerics.check(copy.deepcopy(one), compute=fake)
    assert len(bad) == 1 and "undeclared" in bad[0]
    upd = copy.deepcopy(one)
    assert numerics.update(upd, "reassociation: test", compute=fake) == ["tiny-csa2/tp2"]
    e = upd["config"]["tiny-csa2/tp2"]
    assert e["version"] == 1 and e["declared"] == ["reassociation: test"] and e["digest"] == "f" * 32
    assert numerics.check(upd, compute=fake) == []
    p = tmp_path / "r.toml"
    numerics.write_registry(upd, str(p))
    assert numerics.load_registry(str(p)) == upd
    assert numerics.main(["--update"]) == 2            # an update without a declaration is refused


def test_identity_gates_pass_on_a_correct_engine_and_catch_a_broken_one():
    from sparkflash_b200.serve.driver import DeviceDriver, FakeRowsEngine
    from sparkflash_b200.serve.tokenizer import ByteTokenizer
    tok = ByteTokenizer(300)

    def make(broken=False):
        def f(**kw):
            lanes = kw.pop("max_lanes", 4)
            eng = FakeRowsEngine(max_lanes=lanes, max_rows=8)
            if broken:                                  # an engine whose output depends on how many rows share a step
                orig = eng.step
                eng.step = lambda tokens, *a, **k: [(t + len(tokens)) % 90 + 32 for t in orig(tokens, *a, **k)]
            return DeviceDriver(eng, tok, eos_id=10 ** 9, max_lanes=lanes, **kw)
        return f
    prompts = [list(range(40, 60)), [65, 66, 67] * 8]
    res = identity.run_gates(make(), prompts, n_new=8)
    assert all(res.values()), res
    res = identity.run_gates(make(broken=True), prompts, n_new=8)
    assert not res["batch_invariance"] or not res["chunk_width"]


def test_perf_and_collective_gates():
    base = {"decode_tok_s@1": {"value": 130.0, "config": {"model": "m"}}}
    ok = {"metric": "decode_tok_s", "n_gpus": 1, "value": 128.0, "higher_is_better": True, "config": {"model": "m"}, "clocks": {"reasons": ["sw_power_cap"]}}
    assert perf.check_perf(ok, base) == []
    assert "tolerance" in perf.check_perf({**ok, "value": 120.0}, base)[0]
    assert "slowdown" in perf.check_perf({**ok, "clocks": {"reasons": ["hw_thermal_slowdown"]}}, base)[0]
    assert perf.check_perf({**ok, "n_gpus": 4}, base) == ["no baseline for decode_tok_s@4"]
    lat = {"metric": "ms", "n_gpus": 1, "value": 8.0, "higher_is_better": False}
    assert perf.check_perf(lat, {"ms@1": {"value": 7.5}}) != [] and perf.check_perf({**lat, "value": 7.6}, {"ms@1": {"value": 7.5}}) == []
    assert perf.expected_collectives(40) == 81 and perf.check_collectives(40, 81) == [] and perf.check_collectives(40, 86) != []
