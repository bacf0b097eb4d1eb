"""Checkpoint and rank-file IO (reference tests: crates/sparkflash-weights rank_file round trips,
crates/sparkflash-engine/tests/loader.rs, crates/sparkflash-device converted.rs)."""
import dataclasses
import os

import pytest
import torch

from sparkflash_b200.config import tiny_config
from sparkflash_b200.models.deepseek_v41 import prepare as P, weights as W
from sparkflash_b200.weights import files as F


def test_safetensors_roundtrip_and_views(tmp_path):
    ts = {"a.weight": torch.arange(24, dtype=torch.float32).reshape(2, 3, 4), "b": torch.randn(5, 7).to(torch.bfloat16),
          "q": torch.randint(0, 255, (16, 8), dtype=torch.uint8), "empty": torch.zeros(0, 4)}
    p = str(tmp_path / "m.safetensors")
    F.write_safetensors(p, ts, {"format": "pt"})
    f = F.SafeTensorsFile(p)
    assert set(f.names) == set(ts)
    for k, v in ts.items():
        assert torch.equal(f.tensor(k), v), k
    assert f.info("b") == ("BF16", [5, 7])
    # the independent implementation reads the same file
    from safetensors import safe_open
    with safe_open(p, "pt") as g:
        assert torch.equal(g.get_tensor("a.weight"), ts["a.weight"])
    f.close()
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes((10 ** 9).to_bytes(8, "little") + b"{}")
    with pytest.raises(OSError):
        F.SafeTensorsFile(str(bad))


def _raw_safetensors(path, header: dict, payload: bytes) -> str:
    import json
    h = json.dumps(header).encode()
    path.write_bytes(len(h).to_bytes(8, "little") + h + payload)
    return str(path)


def test_safetensors_rejects_crafted_offsets(tmp_path):
    """A header whose byte ranges are reversed, negative, beyond the file or at odds with shape x dtype is refused at open
    (the length b - a must never wrap into a huge unsigned value)."""
    ok = {"t": {"dtype": "U8", "shape": [16], "data_offsets": [0, 16]}}
    f = F.SafeTensorsFile(_raw_safetensors(tmp_path / "ok.safetensors", ok, bytes(16)))
    assert f.tensor("t").numel() == 16
    f.close()
    cases = {
        "reversed": {"t": {"dtype": "U8", "shape": [16], "data_offsets": [16, 0]}},
        "negative": {"t": {"dtype": "U8", "shape": [16], "data_offsets": [-16, 0]}},
        "huge": {"t": {"dtype": "U8", "shape": [16], "data_offsets": [0, 2 ** 62]}},
        "huge_begin": {"t": {"dtype": "U8", "shape": [0], "data_offsets": [2 ** 62, 2 ** 62]}},
        "beyond": {"t": {"dtype": "U8", "shape": [17], "data_offsets": [0, 17]}},
        "shape_mismatch": {"t": {"dtype": "F32", "shape": [16], "data_offsets": [0, 16]}},
        "negative_dim": {"t": {"dtype": "U8", "shape": [-16], "data_offsets": [0, 16]}},
    }
    for name, header in cases.items():
        with pytest.raises(OSError):
            F.SafeTensorsFile(_raw_safetensors(tmp_path / f"{name}.safetensors", header, bytes(16)))


def test_digest_is_stable_and_sensitive():
    t = torch.arange(1000, dtype=torch.int32)
    d = F.digest64(t)
    assert d == F.digest64(t.clone()) and d != F.digest64(t + (torch.arange(1000) == 999).int())
    assert F.digest64(torch.zeros(0)) == 0xEF46DB3751D8E999          # XXH64 of the empty input, seed 0


@pytest.mark.parametrize("world", [1, 2])
def test_rank_file_roundtrip_and_corruption(tmp_path, world):
    cfg = tiny_config()
    ck = W.synthetic_checkpoint(cfg, 0)
    for rank in range(world):
        w = P.prepare_from_checkpoint(ck, cfg, rank, world, device="cpu")
        path = str(tmp_path / f"rank{rank}.sfb")
        info = F.write_rank_file(path, w, {"source": "synthetic"})
        assert info["tensors"] > 20
        w2 = F.load_rank_file(path, device="cpu", expect_rank=rank, expect_world=world)
        assert w2.cfg == cfg and w2.rank == rank and w2.world == world and w2.il == w.il
        a, sa = F._flatten(w)
        b, sb = F._flatten(w2)
        assert a.keys() == b.keys() and sa == sb
        for k in a:
            assert a[k].dtype == b[k].dtype and torch.equal(a[k].view(torch.uint8) if a[k].dtype != torch.bool else a[k],
                                                             b[k].view(torch.uint8) if b[k].dtype != torch.bool else b[k]), k
    with pytest.raises(ValueError):
        F.load_rank_file(path, device="cpu", expect_rank=0, expect_world=4)
    # flip one payload byte: the digest check names the tensor
    size = os.path.getsize(path)
    with open(path, "r+b") as f:
        f.seek(4096 + 17); b = f.read(1); f.seek(4096 + 17); f.write(bytes([b[0] ^ 0x40]))
    with pytest.raises(OSError, match="digest mismatch"):
        F.load_rank_file(path, device="cpu")
    F.load_rank_file(path, device="cpu", verify=False)
    with open(path, "r+b") as f:
        f.truncate(size - 100)
    with pytest.raises(OSError, match="truncated|footer|table"):
        F.load_rank_file(path, device="cpu")
