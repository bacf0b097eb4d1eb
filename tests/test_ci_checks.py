"""The host gates' own checks: ABI argument counts, source rules, the env table (reference: ci/ of the reference and
its scripts/tests)."""
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(REPO, "ci"))


def test_native_entry_points_and_python_callers_agree_on_argument_counts():
    import check_abi
    sigs, calls = check_abi.c_signatures(), check_abi.python_calls()
    assert len(sigs) > 150 and len(calls) > 200
    assert sigs["sfb_moe_plan"][0] == 14 and sigs["sfb_spec_cost"][0] == 6
    wrong = [(n, k, f, l) for n, k, f, l in calls if n in sigs and sigs[n][0] != k]
    unknown = [(n, f, l) for n, k, f, l in calls if n not in sigs]
    assert wrong == [] and unknown == []


def test_abi_check_flags_a_wrong_call(tmp_path, monkeypatch):
    import check_abi
    monkeypatch.setattr(check_abi, "c_signatures", lambda: {"sfb_demo": (3, "demo.cu")})
    monkeypatch.setattr(check_abi, "python_calls", lambda: [("sfb_demo", 4, "x.py", 7), ("sfb_gone", 1, "y.py", 2), ("sfb_demo", 3, "z.py", 1)])
    assert check_abi.main() == 1


def test_source_rules_hold_and_catch_a_violation(tmp_path, monkeypatch):
    import check_sources
    assert check_sources.scan() == []
    bad = tmp_path / "csrc"
    bad.mkdir()
    (bad / "k_bad.cu").write_text("__global__ void k() { while (true) {} __trap(); }\n")
    monkeypatch.setattr(check_sources, "CSRC", bad)
    got = check_sources.scan()
    assert any("loop without a bound" in g for g in got) and any("device trap" in g for g in got)


def test_every_environment_variable_read_is_declared():
    import host_gates
    assert "declared overrides" in host_gates.gate_env_table()
