"""Speculative-decoding policy (host): cost model, depth allocation, draft passes, acceptance, Philox.
Reference tests: crates/sparkflash-scheduler/tests/{batching,decisions}.rs, tp4_forward/spec.rs unit tests."""
import pytest

from sparkflash_b200.sched import spec as SP


def test_step_cost_bands_and_fit():
    c = SP.StepCost(a0=5.0, b0=2.0, a1=12.0, b1=0.5, band=5)
    assert c(1) == 7.0 and c(5) == 15.0 and c(6) == 15.0 and c(16) == 20.0
    rows = [1, 2, 4, 5, 8, 16, 32, 64]
    fit = SP.StepCost.fit(rows, [c(r) for r in rows], band=5)
    for got, want in zip((fit.a0, fit.b0, fit.a1, fit.b1), (5.0, 2.0, 12.0, 0.5)):
        assert got == pytest.approx(want, abs=1e-6)
    one_band = SP.StepCost.fit([8, 16, 32], [16.0, 20.0, 28.0], band=5)        # nothing measured below the band: copied
    assert one_band.a0 == pytest.approx(one_band.a1) and one_band.b0 == pytest.approx(0.5)
    with pytest.raises(ValueError):
        SP.StepCost.fit([4], [10.0], band=5)


def test_allocation_keeps_prefixes_prefers_likely_drafts_and_stops_when_the_rate_falls():
    cost = SP.StepCost(a0=5.0, b0=2.0, a1=12.0, b1=0.5, band=5)
    pol = SP.SpecPolicy(cost, max_rows=64, max_depth=5)
    # one confident sequence, one hopeless one
    a = pol.allocate([[0.95, 0.9, 0.9, 0.85, 0.8], [0.05, 0.05, 0.05, 0.05, 0.05]])
    assert a.keep[0] >= 3 and a.keep[1] == 0
    assert a.rows == 2 + sum(a.keep) and a.cost_ms == pytest.approx(cost(a.rows))
    assert a.tokens_per_ms >= 2 / cost(2)                 # never worse than not speculating
    # a low-probability first draft blocks the (useless) deeper ones behind it
    b = pol.allocate([[0.1, 0.99, 0.99]])
    assert b.keep == [0] or b.keep == [1]
    # the row cap binds: 32 sequences in 40 rows leave 8 draft rows, given to the likeliest first drafts
    pol40 = SP.SpecPolicy(SP.StepCost(a0=10.0, b0=0.01, a1=10.0, b1=0.01, band=5), max_rows=40, max_depth=5)
    probs = [[0.9 if s < 8 else 0.5] * 3 for s in range(32)]
    c = pol40.allocate(probs)
    assert c.rows == 40 and sum(c.keep) == 8 and all(k == 1 for k in c.keep[:8])
    with pytest.raises(ValueError):
        SP.SpecPolicy(cost, max_rows=4).allocate([[0.5]] * 5)
    # steep row cost: speculation does not pay at all
    steep = SP.SpecPolicy(SP.StepCost(a0=0.1, b0=5.0, a1=0.1, b1=5.0, band=5), max_rows=64)
    assert steep.allocate([[0.6, 0.6]]).keep == [0]


def test_draft_passes_accept_rule_and_calibration():
    pol = SP.SpecPolicy(max_rows=64, passes_of=16)
    assert [list(r)[0:1] + [len(r)] for r in pol.draft_passes(40)] == [[0, 16], [16, 16], [32, 8]]
    assert pol.draft_passes(0) == []
    assert SP.accept([5, 6, 7], [5, 6, 9, 1]) == 2 and SP.accept([5], [4, 5]) == 0 and SP.accept([], [3]) == 0
    assert SP.calibrate(0.0) == 0.5 and SP.calibrate(50.0) > 0.999 and SP.calibrate(-1000.0) == 0.0


def test_philox_known_answer_and_streams():
    # Random123 known-answer vectors for philox4x32-10
    assert SP.philox4x32((0, 0, 0, 0), (0, 0)) == (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)
    assert SP.philox4x32((0xffffffff,) * 4, (0xffffffff,) * 2) == (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)
    u = [SP.philox_uniform(7, 1, i) for i in range(1000)]
    assert all(0.0 <= x < 1.0 for x in u) and 0.45 < sum(u) / len(u) < 0.55
    assert SP.philox_uniform(7, 1, 3) == u[3] and SP.philox_uniform(7, 2, 3) != u[3] and SP.philox_uniform(8, 1, 3) != u[3]
