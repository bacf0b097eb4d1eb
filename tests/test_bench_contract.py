"""bench.py pieces that need no GPU: the reference arm's answer and the clock-sample parser."""
import json
import os
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def test_reference_arm_reports_unavailable_and_exits_zero():
    out = subprocess.run([sys.executable, os.path.join(REPO, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0
    line = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 10


def test_clock_sampler_uses_the_timed_window_and_names_throttle_reasons(tmp_path):
    import bench
    s = bench.ClockSampler(0)
    s.path = str(tmp_path / "clocks.csv")
    rows = ["0, 1200, 1965, 300.0, 0x0, Not Active, Not Active, Not Active, Not Active",      # warm-up
            "0, 1950, 1965, 900.0, 0x4, Not Active, Not Active, Not Active, Active",          # timed: power cap
            "0, 1965, 1965, 950.0, 0x4, Not Active, Not Active, Not Active, Active",
            "0, 1935, 1965, 950.0, 0x4, Not Active, Not Active, Not Active, Active"]
    open(s.path, "w").write("\n".join(rows[:1]) + "\n")

    class _Done:
        def terminate(self): pass
        def wait(self, timeout=None): return 0
        def kill(self): pass
    s.proc, s.f = _Done(), open(s.path, "a")
    s.mark()
    s.f.write("\n".join(rows[1:]) + "\n"); s.f.flush()
    got = s.stop()
    assert got["samples"] == 3 and got["sm_mhz"] == 1950.0 and got["sm_max_mhz"] == 1965.0
    assert got["reasons"] == ["sw_power_cap"] and got["window"] == "timed regions"
    # a run shorter than two sampling periods falls back to every sample taken under load, and says so
    s2 = bench.ClockSampler(0)
    s2.path = str(tmp_path / "clocks2.csv")
    open(s2.path, "w").write("\n".join(rows[:3]) + "\n")
    s2.proc, s2.f = _Done(), open(s2.path, "a")
    s2.skip = 3
    got2 = s2.stop()
    assert got2["samples"] == 3 and got2["window"] == "warm-up and timed regions"
