"""Run header, logits dump round trip and comparison (reference: run_header.rs, logits_dump.rs of the forward crate)."""
import json

import pytest
import torch

from sparkflash_b200.utils import evidence as EV


def test_run_header_names_the_build_and_the_engine():
    class Comm: name = "fused"
    class W: moe_mode = "tp"
    class Cfg: name = "tiny"
    class Eng:
        arm, world, rank, max_rows, max_lanes, comm, use_graphs, w, cfg = "tc", 4, 1, 64, 16, Comm(), True, W(), Cfg()
    h = EV.run_header(Eng(), extra={"note": "x"})
    assert len(h["build_id"]) == 16 and h["build_id"] == EV.build_id()
    assert h["engine"] == {"arm": "tc", "world": 4, "rank": 1, "max_rows": 64, "max_lanes": 16, "collective": "fused",
                           "cuda_graphs": True, "moe_mode": "tp", "model": "tiny"}
    assert h["note"] == "x" and "nccl_env" in h
    json.dumps(h)


def test_logits_dump_round_trip_and_gate_numbers(tmp_path):
    g = torch.Generator().manual_seed(0)
    rows = [torch.randn(50, generator=g) for _ in range(6)]
    a, b = str(tmp_path / "a.bin"), str(tmp_path / "b.bin")
    da, db = EV.LogitsDump(a, {"arm": "cuda"}), EV.LogitsDump(b, {"arm": "tc"})
    for i, r in enumerate(rows):
        da.add(i, 0, 10 + i, r)
        db.add(i, 0, 10 + i, r + (0.01 if i == 3 else 0.0))
    da.close(); db.close()
    hdr, recs = EV.LogitsDump.read(a)
    assert hdr == {"arm": "cuda"} and len(recs) == 6 and torch.equal(recs[2][3], rows[2]) and recs[2][:3] == (2, 0, 12)
    cmp_ = EV.compare_dumps(a, b)
    assert cmp_["records"] == 6 and cmp_["top1"] == 1.0 and cmp_["max_abs"] == pytest.approx(0.01, abs=1e-6) and cmp_["kl"] < 1e-6
    assert EV.compare_dumps(a, a)["max_abs"] == 0.0
    with pytest.raises(ValueError):
        EV.LogitsDump.read(str(tmp_path / "nope.bin")) if (tmp_path / "nope.bin").write_bytes(b"garbage!") else None
