"""Lazily backed lane memory on the device (reference: crates/sparkflash-kernels lane_memory tests)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_lanes_back_lazily_within_budget_and_give_chunks_back():
    from sparkflash_b200.kv.lanes import LaneBudgetExceeded, LanePool, LaneRegion
    pool = LanePool(budget_bytes=16 << 20)
    g = pool.granularity
    assert g >= 2 << 20 and g % (2 << 20) == 0
    free0 = torch.cuda.mem_get_info()[0]
    reg = LaneRegion(pool, lanes=4, rows=(1 << 20), width=256)          # 256 MiB of address space per lane, none backed
    assert reg.tensor.shape == (4, reg.rows, 256) and reg.mapped_bytes == 0 and reg.backed_rows(2) == 0
    assert free0 - torch.cuda.mem_get_info()[0] < (8 << 20)
    reg.ensure_rows(2, 100)                                             # one chunk
    assert reg.mapped_bytes == g and reg.backed_rows(2) == g // 256
    t = reg.tensor
    t[2, :100] = 7
    t[2, 99, 255] = 9
    torch.cuda.synchronize()
    assert int(t[2, :100].sum()) == 7 * 100 * 256 + 2
    reg.ensure_rows(2, 3 * g // 256)                                    # grows to three chunks; the old rows stay
    assert reg.mapped_bytes == 3 * g and int(t[2, 99, 255]) == 9
    reg.copy_prefix(2, 0, 100)                                          # prefix adoption into another lane
    torch.cuda.synchronize()
    assert torch.equal(t[0, :100], t[2, :100]) and reg.backed_rows(0) >= 100
    with pytest.raises(LaneBudgetExceeded):
        reg.ensure_rows(1, 8 * g // 256)                                # 4 mapped + 8 wanted > 8-chunk budget
    reg.release(1)
    reg.release(2, from_row=g // 256)                                   # shrink lane 2 to its first chunk
    assert reg.backed_rows(2) == g // 256 and int(t[2, 99, 255]) == 9
    st = pool.stats()
    assert st["spare"] >= 2 and st["created"] <= st["budget"] == 8
    reg.ensure_rows(3, 10)                                              # served from the spare list, no new chunk
    assert pool.stats()["created"] == st["created"]
    pool.close()


def test_engine_on_lazy_lanes_matches_the_dense_cache():
    from sparkflash_b200.config import tiny_config
    from sparkflash_b200.models.deepseek_v41 import engine as E, prepare as P, weights as W
    cfg = tiny_config()
    w = P.prepare_from_checkpoint(W.synthetic_checkpoint(cfg, 0), cfg, 0, 1)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    dense = E.Engine(w, max_lanes=2, max_context=1 << 16, max_rows=16, arm="tc")
    want = dense.generate(prompt, 8)
    lazy = E.Engine(w, max_lanes=2, max_context=1 << 16, max_rows=16, arm="tc", lane_budget_bytes=256 << 20)
    assert lazy.kv.nbytes() < dense.kv.nbytes()
    got = lazy.generate(prompt, 8)
    assert got == want
    used = lazy.kv.pool.stats()["created"]
    assert used > 0
    lazy.kv.release_lane(0)
    assert lazy.kv.pool.stats()["spare"] == used
    assert lazy.generate(prompt, 8, lane=1) == want
