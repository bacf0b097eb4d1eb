"""Tensor-parallel plan: divisibility, per-rank shapes and bytes (reference: crates/sparkflash-device resident.rs tests,
crates/sparkflash-model tp_plan)."""
import pytest

from sparkflash_b200.config import full_config
from sparkflash_b200.models import tp_plan as TP


def test_released_model_shapes_per_rank():
    cfg = full_config()
    for W, heads, groups, inter, vocab in ((2, 32, 4, 1152, 64640), (4, 16, 2, 576, 32320), (8, 8, 1, 288, 16160)):
        p = TP.plan(cfg, W)
        assert (p.heads_per_rank, p.groups_per_rank, p.inter_per_rank, p.vocab_per_rank) == (heads, groups, inter, vocab)
        assert p.collectives_per_step() == 2 * cfg.n_layers + 1
    assert TP.plan(cfg, 1).collectives_per_step() == 0
    ep = TP.plan(cfg, 8, "ep")
    assert ep.experts_per_rank == 48 and ep.inter_per_rank == cfg.moe_inter


def test_bytes_per_rank_match_the_footprint_of_the_released_model():
    """About 307 GB resident in total (routed experts 289 GB in FP4): a quarter of the split tensors plus the replicated
    ones per rank at four ranks, and experts dominate."""
    cfg = full_config()
    one = TP.plan(cfg, 1).bytes_per_rank() / 1e9
    assert 295 < one < 325
    four = TP.plan(cfg, 4).bytes_per_rank() / 1e9
    eight = TP.plan(cfg, 8).bytes_per_rank() / 1e9
    assert one / 4 < four < one / 4 + 8 and one / 8 < eight < one / 8 + 8
    experts = sum(t.bytes_per_rank(1) for t in TP.plan(cfg, 1).layer if t.name.startswith("expert.")) * cfg.n_layers / 1e9
    assert 280 < experts < 300
    # expert parallelism keeps the shared expert whole on every rank
    assert TP.plan(cfg, 8, "ep").bytes_per_rank() > TP.plan(cfg, 8).bytes_per_rank()


def test_plans_that_do_not_divide_are_refused():
    cfg = full_config()
    with pytest.raises(ValueError):
        TP.plan(cfg, 3)
    with pytest.raises(ValueError):
        TP.plan(cfg, 16)            # 8 output groups do not divide over 16 ranks
