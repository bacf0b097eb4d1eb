"""Second KV tier: park a lane's caches in host memory and restore them into another lane (reference tests:
crates/sparkflash-kv/tests tier / swa / cache)."""
import torch

from sparkflash_b200.config import tiny_config
from sparkflash_b200.kv.tier import KVTier
from sparkflash_b200.models.deepseek_v41.engine import KVCache


def _fill(kv, lane, seed):
    g = torch.Generator().manual_seed(seed)
    for dct in (kv.win_q, kv.win_s, kv.ckv_q, kv.ckv_s, kv.ik_q, kv.ik_s):
        for t in dct.values():
            t[lane].copy_(torch.randint(0, 200, t[lane].shape, dtype=torch.uint8, generator=g))
    for t in kv.cin.values():
        t[lane].copy_(torch.randn(t[lane].shape, generator=g))


def test_park_and_restore_move_a_sequence_between_lanes_bit_for_bit():
    cfg = tiny_config()
    kv = KVCache(cfg, lanes=3, max_context=128, max_rows=8, device="cpu")
    _fill(kv, 0, 1); _fill(kv, 2, 2)
    tier = KVTier(kv, budget_bytes=1 << 30)
    tokens = list(range(100, 160))
    P = 45
    ent = tier.park(0, tokens, P)
    assert ent.positions == P and ent.nbytes > 0 and tier.stats()["entries"] == 1
    # a new prompt that extends the parked tokens finds it; a diverging one does not
    assert tier.longest_prefix(tokens[:P] + [7, 8]) is ent
    assert tier.longest_prefix(tokens[:P - 1] + [9999, 1]) is None and tier.longest_prefix(tokens[:10]) is None
    got = tier.restore(ent, 2)
    assert got == P
    first = max(0, P - cfg.window)
    slots = [p % kv.ring for p in range(first, P)]
    for l in kv.win_q:
        assert torch.equal(kv.win_q[l][2, slots], kv.win_q[l][0, slots]) and torch.equal(kv.win_s[l][2, slots], kv.win_s[l][0, slots])
        if l in kv.cin:
            assert torch.equal(kv.cin[l][2, slots], kv.cin[l][0, slots])
        if l in kv.ckv_q:
            n = P // cfg.ratio(l) + 1
            for name in ("ckv_q", "ckv_s", "ik_q", "ik_s"):
                a = getattr(kv, name)[l]
                assert torch.equal(a[2, :n], a[0, :n])


def test_tier_evicts_least_recently_used_within_its_byte_budget():
    cfg = tiny_config()
    kv = KVCache(cfg, lanes=2, max_context=128, max_rows=8, device="cpu")
    _fill(kv, 0, 3)
    one = KVTier(kv).park(0, list(range(40)), 40).nbytes
    tier = KVTier(kv, budget_bytes=int(one * 2.5))
    a = tier.park(0, [1] * 40, 40); b = tier.park(0, [2] * 40, 40)
    tier.restore(a, 1)                       # a is now the most recently used
    tier.park(0, [3] * 40, 40)               # over budget: b goes
    assert tier.longest_prefix([2] * 41) is None and tier.longest_prefix([1] * 41) is a and tier.stats()["evicted"] == 1
