"""Planning layer: parts catalogue vs the built library, step plans, collective plans.
Reference tests: crates/sparkflash-ops (parts.rs asserts on the catalogue, collective.rs plan choices)."""
import pytest

from sparkflash_b200.ops import plan as P


def test_every_catalogued_entry_point_is_exported_by_the_library():
    r = P.KernelResolver()
    assert r.missing() == []
    assert r.resolve("attention", "tc") == "sfb_attn_tc"
    with pytest.raises(KeyError):
        r.resolve("attention", "nonexistent")
    with pytest.raises(KeyError):
        r.resolve("no_such_part", "x")


def test_resolver_reports_a_dropped_symbol():
    class Fake:
        def __getattr__(self, name):
            if name == "sfb_attn_tc":
                raise AttributeError(name)
            return object()
    r = P.KernelResolver(lib=Fake())
    assert ("attention", "tc", "sfb_attn_tc") in r.missing()
    with pytest.raises(LookupError):
        r.resolve("attention", "tc")


def test_step_plan_switches_variants_at_the_engine_thresholds():
    from sparkflash_b200.models.deepseek_v41.engine import Engine
    assert Engine.GROUP_MIN_ROWS == P.GROUP_MIN_ROWS and Engine.GROUP_WIDE_ROWS == P.GROUP_WIDE_ROWS
    one, few, chunk, bulk = (P.plan_step(n) for n in (1, 16, 128, 1024))
    assert (one.dense, one.attention, one.moe, one.coef, one.fold) == ("skinny", "rows", "token", "rows", "cluster")
    assert few.moe == "seg16" and few.attention == "rows"
    assert chunk.attention == "tc" and chunk.wo_a == "pair_bulk" and chunk.dense == "skinny"
    assert (bulk.dense, bulk.moe, bulk.coef, bulk.fold, bulk.gate) == ("bulk", "seg64", "gemm", "rows", "gemm")
    cuda = P.plan_step(16, arm="cuda")
    assert cuda.dense == "cuda_core" and cuda.moe == "cuda_core" and cuda.index_scores == "cuda_core"
    assert one.kernels_per_layer() < bulk.kernels_per_layer(index_layer=True, kv_source=True)


def test_collective_plan_forms_and_bytes():
    d = 5120
    assert P.plan_collective(8, d, 1).kind is P.CollectiveKind.NONE
    a = P.plan_collective(8, d, 8)
    b = P.plan_collective(1024, d, 8)
    assert a.kind is P.CollectiveKind.ONE_SHOT and b.kind is P.CollectiveKind.TWO_SHOT
    assert P.plan_collective(1024, d, 4).kind is P.CollectiveKind.ONE_SHOT                # below 8 ranks the one-shot push measured faster
    assert P.plan_collective(1024, d, 4, two_shot_world=4).kind is P.CollectiveKind.TWO_SHOT
    assert a.bytes_sent_per_rank == 8 * d * 2 * 7
    assert b.bytes_sent_per_rank == 2 * 1024 * d * 2 * 7 // 8            # 2 (W-1)/W of the message
    assert P.plan_collective(1024, d, 8, arm="nccl").kind is P.CollectiveKind.NCCL
    o = P.plan_collective(4096, d, 4, bulk_chunks=8)
    assert o.kind is P.CollectiveKind.OVERLAPPED and o.chunks_in_flight == 3
    # rows are owned in equal blocks; every row has exactly one owner
    owned = [b.rows_owned(r) for r in range(8)]
    assert owned[0] == (0, 128) and owned[-1] == (896, 1024)
    odd = P.plan_collective(1000, d, 8)
    cover = [i for r in range(8) for i in range(*odd.rows_owned(r))]
    assert cover == list(range(1000))
    assert b.link_seconds() == pytest.approx(b.bytes_sent_per_rank / 770e9)
