"""Runtime bookkeeping on the host: ledger budgets, launch-list identity of captured segments, in-step agreement.
Reference tests: crates/sparkflash-deepseek-forward device_counters / tp4_graph unit tests, crates/sparkflash-runtime."""
import pytest

from sparkflash_b200.runtime import group as G, ledger as L, segments as S


def test_ledger_accepts_a_step_within_budget_and_refuses_a_stray_collective():
    b = L.Budget.for_rows_step(n_layers=40, world=8, fused=True)
    assert b.collectives == 81 and b.max_d2h == 1
    led = L.StepLedger(b)
    led.begin()
    led.count("launch", 620); led.count("collective", 81); led.count("h2d", 5); led.count("d2h"); led.count("host_sync")
    assert led.end()["problems"] == []
    led.begin()
    led.count("launch", 620); led.count("collective", 82); led.count("h2d", 5)
    with pytest.raises(L.LedgerError, match="collectives 82 != 81"):
        led.end()
    led.begin()
    led.count("collective", 81); led.count("d2h", 2); led.count("alloc")
    got = led.end(strict=False)
    assert any("d2h" in p for p in got["problems"]) and any("alloc" in p for p in got["problems"])
    assert led.snapshot()["steps"] == 3
    assert L.Budget.for_rows_step(40, 1, False).collectives == 0
    assert L.Budget.for_rows_step(40, 4, True, sampled=False).collectives == 80
    with pytest.raises(KeyError):
        led.count("nonsense")


def test_launch_log_identity_of_a_segment():
    with S.recording() as a:
        for name in ("seam_fold", "umma_dense", "attn_rows", "umma_dense"):
            S.note(name)
    cache = S.SegmentCache()
    cache.put((1, 1024), a)
    with S.recording() as same:
        for name in ("seam_fold", "umma_dense", "attn_rows", "umma_dense"):
            S.note(name)
    cache.check((1, 1024), same)
    with S.recording() as other:          # one kernel swapped for another: same count, different list
        for name in ("seam_fold", "umma_dense", "attn_tc", "umma_dense"):
            S.note(name)
    with pytest.raises(RuntimeError, match="changed since capture"):
        cache.check((1, 1024), other)
    with pytest.raises(KeyError):
        cache.check((2, 1024), same)
    S.note("outside any recording")         # a no-op without an installed log
    assert len(a) == 4


def test_native_wrappers_feed_the_launch_log():
    """A wrapper that returns success notes its name; a failing one raises before anything is noted."""
    from sparkflash_b200.ops import native as N
    with S.recording() as log:
        N._check(0, "some_kernel")
        with pytest.raises(N.NativeError):
            N._check(700, "bad_kernel")
    assert log.items == ["some_kernel"]


def test_group_lanes_detect_a_rank_that_took_another_branch():
    W = 4
    ranks = [G.GroupLanes(r, W) for r in range(W)]
    lead = ranks[0]
    for t in range(1, 4):
        for r in ranks:
            d = r.record([11, 12], [0, 1], [t, t], [5, 6])
            lead.report(r.rank, t, d)
        assert lead.in_step(t) is True
        lead.check(t)
    # rank 2 runs a different row list at tick 4
    for r in ranks:
        rows = [11, 12] if r.rank != 2 else [11, 13]
        lead.report(r.rank, 4, r.record(rows, [0, 1], [4, 4], [5, 6]))
    assert lead.in_step(4) is False
    with pytest.raises(G.GroupOutOfStep, match="tick 4"):
        lead.check(4)
    # a tick with a missing report is undecided, not wrong
    lead.report(0, 5, "x")
    assert lead.in_step(5) is None
    lead.check(5)


def test_kernel_marks_summary_separates_idle_ctas_and_old_launches():
    """Phase marks: the summary uses the CTAs of the newest launch, tells idle CTAs (no stage ever landed) from working ones
    and reports the phases in microseconds."""
    import torch
    from sparkflash_b200.utils.kernel_marks import summarize
    m = torch.zeros(6, 16, dtype=torch.int64)
    base = 1_000_000_000
    # two working CTAs of the newest launch
    for i, life in enumerate((20_000, 24_000)):
        t0 = base + i * 1000
        m[i, :8] = torch.tensor([t0, t0 + 250, t0 + 1250, t0 + 2250, t0 + 10_250, t0 + 10_300, t0 + life - 200, t0 + life])
        m[i, 8] = t0 + 10_400
    # an idle CTA of the newest launch: its "first stage landed" mark is left over from an older launch
    m[2, :8] = torch.tensor([base + 50, base + 300, base + 700, base - 500_000, base + 800, base + 900, base + 1900, base + 2000])
    # a CTA slot only an older launch touched (a second earlier)
    m[3, :8] = torch.tensor([base - 10**9 + k for k in range(8)])
    rep = summarize(m.view(-1))
    assert rep["ctas"] == 3 and rep["ctas_with_work"] == 2
    assert rep["idle_cta_us"] == pytest.approx(1.95, abs=0.01)
    assert rep["setup_us"] == pytest.approx(0.25) and rep["mainloop_us"] == pytest.approx(8.0) and rep["first_stage_latency_us"] == pytest.approx(1.0)
    assert rep["epilogue_first_read_us"] == pytest.approx(0.1)
    assert summarize(torch.zeros(32, dtype=torch.int64)) == {"ctas": 0}


def test_mark_summaries_of_the_attention_seam_and_persistent_kernels():
    """The attention kernel's phase marks, the bulk-copy seam's and the persistent MoE kernels' cycle counters are turned into
    named durations: synthetic records with known gaps come back as those gaps."""
    import torch
    from sparkflash_b200.utils import kernel_marks as KM
    buf = torch.zeros(16 * 8, dtype=torch.int64)
    m = buf.view(-1, 16)
    t0 = 1_000_000
    order = [0, 1, 2, 3, 4, 5, 6, 8, 12, 9, 10, 7]            # the slots in the order the kernel passes them
    for cta in range(3):
        for i, slot in enumerate(order):
            m[cta, slot] = t0 + cta * 100 + i * 1000           # 1 us between consecutive marks
        m[cta, 11] = m[cta, 8] + 400
    a = KM.summarize_attention(buf)
    assert a["ctas"] == 3 and a["cta_life_us"] == 11.0 and a["kernel_span_us"] == 11.2
    assert a["first_tile_decoded_us"] == 1.0 and a["epilogue_accumulator_pass_us"] == 1.0 and a["epilogue_rope_quant_pass_us"] == 1.0
    assert KM.summarize_attention(torch.zeros(32, dtype=torch.int64)) == {"ctas": 0}
    words = []
    for row in range(4):
        words += [5000 + row * 10 + k * 2000 for k in range(7)] + [0]
    s_ = KM.summarize_seam(words, 4)
    assert s_["rows"] == 4 and s_["block_life_us"] == 12.0 and s_["fold_us"] == 2.0 and s_["kernel_span_us"] == 12.0
    pc = torch.zeros(16 * 4, dtype=torch.int64)
    pv = pc.view(-1, 16)
    pv[0, :9] = torch.tensor([20, 1000, 50, 300, 900, 600, 360, 980, 420])
    pv[1, :9] = torch.tensor([22, 1200, 70, 500, 1100, 800, 396, 1180, 620])
    down = KM.summarize_persistent(pc, "down")
    assert down["ctas"] == 2 and down["tiles"] == 21.0 and down["mma_wait_scales"] == 400.0 and down["producer_wait_free"] == 520.0
    gu = KM.summarize_persistent(pc, "gate_up")
    assert gu["mma_wait_data"] == 400.0 and "ksteps" not in gu


def test_roofline_accounting_groups_launches_and_uses_the_measured_peaks(tmp_path):
    from sparkflash_b200.utils import roofline as R
    assert R.classify("umma_gate_up_grouped") == "moe_gate_up" and R.classify("umma_down_grouped") == "moe_down"
    assert R.classify("umma_bulk") == "dense" and R.classify("attn_tc") == "attention" and R.classify("seam_fold") == "seams"
    assert R.classify("index_scores_tc") == "indexer" and R.classify("something_else") == "rest"
    (tmp_path / "MEASURED_PEAKS.json").write_text('{"hbm_gbs": 5000.0, "bf16_tflops": 1500.0, "bf16_tflops_sustained": 1000.0}')
    pk = R.peaks(tmp_path)
    assert pk == {"hbm_gbs": 5000.0, "bf16_tflops_sustained": 1000.0, "source": "measured"}
    assert R.peaks(tmp_path / "nowhere")["source"] == "fallback"
    work = {"moe_gate_up": R.ClassWork(bytes=1e9, flops=1e11), "dense": R.ClassWork(bytes=1e8, flops=4e11)}
    rows = R.account([("umma_gate_up_grouped", 400.0), ("umma_bulk", 300.0), ("umma_bulk", 200.0), ("moe_plan", 30.0)], work, pk)
    by = {r["class"]: r for r in rows}
    assert by["moe_gate_up"]["roofline_us"] == 200.0 and by["moe_gate_up"]["bound"] == "memory" and by["moe_gate_up"]["fraction_of_measured"] == 0.5
    assert by["dense"]["launches"] == 2 and by["dense"]["bound"] == "compute" and by["dense"]["fraction_of_measured"] == 0.8
    assert by["moe_plan"]["fraction_of_measured"] is None
    assert rows[0]["class"] == "dense"                       # sorted by measured time
    assert "| class |" in R.format_table(rows)


def test_guard_arena_leaves_host_allocations_alone_and_restores_torch():
    import torch
    from sparkflash_b200.utils import canary
    z, e = torch.zeros, torch.empty
    with canary.guarded() as arena:
        t = torch.zeros(4, 3)                       # a host tensor: not guarded
        assert t.shape == (4, 3) and not arena.records
        with arena.active():                        # nesting keeps the outer patch
            assert torch.zeros is not z
        assert torch.zeros is not z
    assert torch.zeros is z and torch.empty is e
