"""Scheduler policy (reference: crates/sparkflash-scheduler/tests/{batching,decisions}.rs,
crates/sparkflash-serve/tests/{concurrency,prefix_cache}.rs) and KV planning structures."""
from sparkflash_b200.sched.core import PHASE_DECODE, PHASE_IDLE, PHASE_PREFILL, Pager, RadixCache, Scheduler


def _run_prefill(s, eos=1):
    phase, rows = s.tick()
    assert phase == PHASE_PREFILL
    seq = rows[0].seq
    done = s.info(seq)["computed"] + len(rows) >= len(PROMPTS[seq])
    s.commit(seq, len(rows), [100 + seq] if done else [], eos)
    return rows


PROMPTS = {}


def test_prefill_chunks_then_decode_and_finish():
    s = Scheduler(max_lanes=2, max_rows=8, prefill_chunk=4, prefill_chunk_busy=2, prefix_reuse_min=3)
    PROMPTS[1] = list(range(10, 20))
    assert s.submit(1, PROMPTS[1], 3) == 0
    seen = []
    for _ in range(3):
        rows = _run_prefill(s)
        seen += [(r.pos, r.token) for r in rows]
    assert seen == [(i, 10 + i) for i in range(10)]
    phase, rows = s.tick()
    assert phase == PHASE_DECODE and len(rows) == 1 and rows[0].pos == 10 and rows[0].token == 101 and rows[0].kind == 1
    assert s.commit(1, 1, [55], 1) == 0
    phase, rows = s.tick()
    assert rows[0].pos == 11 and rows[0].token == 55
    assert s.commit(1, 1, [1], 1) == 1  # eos
    assert s.tick()[0] == PHASE_IDLE
    assert s.info(1)["state"] == "finished"


def test_fewest_rows_left_goes_first_and_busy_chunk():
    s = Scheduler(max_lanes=4, max_rows=8, prefill_chunk=100, prefill_chunk_busy=3, prefix_reuse_min=1000)
    PROMPTS[1], PROMPTS[2] = list(range(50)), list(range(100, 105))
    s.submit(1, PROMPTS[1], 4); s.submit(2, PROMPTS[2], 4)
    phase, rows = s.tick()
    assert phase == PHASE_PREFILL and rows[0].seq == 2 and len(rows) == 5   # shorter prompt first, whole chunk
    s.commit(2, 5, [7], 1)
    # now one sequence decodes: prefill of the other runs in busy chunks and alternates with decode steps
    phases = []
    for _ in range(6):
        phase, rows = s.tick()
        phases.append((phase, len(rows)))
        if phase == PHASE_PREFILL:
            s.commit(1, len(rows), [], 1)
        elif phase == PHASE_DECODE:
            s.commit(2, 1, [9], 1)
    assert (PHASE_PREFILL, 3) in phases and any(p == PHASE_DECODE for p, _ in phases)


def test_queue_limit_and_refusal():
    s = Scheduler(max_lanes=1, queue_depth=2, max_rows=4, prefill_chunk=4)
    for i in range(1, 4):
        PROMPTS[i] = [5, 6, 7]
    assert s.submit(1, PROMPTS[1], 2) == 0
    s.tick()
    assert s.submit(2, PROMPTS[2], 2) == 0 and s.submit(3, PROMPTS[3], 2) == 0
    assert s.submit(4, [1, 2], 2) == 1            # lane busy and queue full
    assert s.stats()["rejected"] == 1
    assert s.submit(5, [], 2) == 2                # invalid


def test_prefix_reuse_from_a_freed_lane():
    s = Scheduler(max_lanes=1, max_rows=4, prefill_chunk=64, prefix_reuse_min=4)
    base = list(range(200, 216))
    PROMPTS[1] = base
    s.submit(1, base, 1)
    phase, rows = s.tick(); s.commit(1, len(rows), [1], 1)       # prefill 16 rows, sampled eos -> finished
    PROMPTS[2] = base[:12] + [9, 9, 9]
    s.submit(2, PROMPTS[2], 1)
    phase, rows = s.tick()
    assert phase == PHASE_PREFILL and rows[0].pos == 12 and len(rows) == 3   # 12 rows reused
    st = s.stats()
    assert st["prefix_hits"] == 1 and st["prefix_rows"] == 12


def test_speculative_rows_keep_prefixes_and_budget():
    s = Scheduler(max_lanes=4, max_rows=6, prefill_chunk=64, prefix_reuse_min=1000)
    for i in (1, 2):
        PROMPTS[i] = [3, 4, 5]
        s.submit(i, PROMPTS[i], 10)
    while any(s.info(i)["state"] != "decode" for i in (1, 2)):
        phase, rows = s.tick()
        if phase == PHASE_PREFILL:
            s.commit(rows[0].seq, len(rows), [40 + rows[0].seq], 1)
    s.set_drafts(1, [11, 12, 13], [0.9, 0.1, 0.05])
    s.set_drafts(2, [21, 22, 23], [0.5, 0.4, 0.3])
    phase, rows = s.tick()
    assert phase == PHASE_DECODE and len(rows) == 6
    by = {}
    for r in rows:
        by.setdefault(r.seq, []).append((r.pos, r.token, r.kind))
    assert by[1][0] == (3, 41, 1) and by[2][0] == (3, 42, 1)
    # drafts are consecutive positions after the anchor, depth-first across sequences
    assert [p for p, _, _ in by[1]] == list(range(3, 3 + len(by[1])))
    assert [p for p, _, _ in by[2]] == list(range(3, 3 + len(by[2])))
    assert len(by[1]) == 3 and len(by[2]) == 3
    # commit: sequence 1 accepted 1 draft (+ bonus), sequence 2 none
    assert s.commit(1, 2, [11, 77], 1) == 0
    assert s.commit(2, 1, [88], 1) == 0
    phase, rows = s.tick()
    anchors = {r.seq: (r.pos, r.token) for r in rows if r.kind == 1}
    assert anchors == {1: (5, 77), 2: (4, 88)}


def test_preemption_when_row_budget_is_exhausted():
    s = Scheduler(max_lanes=2, max_rows=4, prefill_chunk=8, prefix_reuse_min=1000, lane_row_budget=12)
    PROMPTS[1], PROMPTS[2] = list(range(8)), list(range(50, 58))
    s.submit(1, PROMPTS[1], 5); s.submit(2, PROMPTS[2], 5)
    phase, rows = s.tick(); s.commit(rows[0].seq, len(rows), [9], 1)
    for _ in range(3):       # second prompt needs 8 more rows than the budget allows -> newest is preempted
        phase, rows = s.tick()
        if phase == PHASE_DECODE:
            s.commit(rows[0].seq, 1, [9], 1)
    assert s.stats()["preemptions"] >= 1
    assert s.info(2)["state"] in ("waiting", "prefill")


def test_radix_cache_and_pager():
    r = RadixCache()
    a = [1, 2, 3, 4, 5, 6]
    r.insert(a)
    assert r.match([1, 2, 3, 9]) == 3 and r.match(a + [7]) == 6 and r.match([8]) == 0
    r.insert([1, 2, 3, 9, 9])
    assert r.tokens == 8 and r.match([1, 2, 3, 9, 9, 9]) == 5
    r.pin(a, 1)
    freed = r.evict(0)
    assert freed == 2 and r.match(a) == 6          # the pinned path survives
    r.pin(a, -1)
    r.evict(0)
    assert r.tokens == 0
    p = Pager(3)
    x, y, z = p.alloc(), p.alloc(), p.alloc()
    assert p.alloc() == -1 and p.share(x) == 2
    assert p.release(x) == 1 and p.release(x) == 0 and p.free == 1


def test_decoder_skip_chunks_stop_at_the_tail_and_forks_rerun_one_tail():
    s = Scheduler(max_lanes=1, max_rows=16, prefill_chunk=16, prefix_reuse_min=4)
    s.set_decoder_tail(10)
    PROMPTS[1] = list(range(100, 140))                      # 40 rows: rows 0..29 skip the upper layers, 30..39 run everything
    s.submit(1, PROMPTS[1], 1)
    kinds = []
    while True:
        phase, rows = s.tick()
        if phase != PHASE_PREFILL:
            break
        kinds.append((rows[0].pos, len(rows), rows[0].kind))
        assert len({r.kind for r in rows}) == 1             # a chunk never straddles the boundary
        done = rows[-1].pos + 1 == 40
        s.commit(1, len(rows), [1] if done else [], 1)
        if done:
            break
    assert kinds == [(0, 16, 3), (16, 14, 3), (30, 10, 0)]
    # a prompt that forks at row 20 (inside the skipped rows) re-runs from row 10 with every layer
    PROMPTS[2] = PROMPTS[1][:20] + [7] * 30
    s.submit(2, PROMPTS[2], 1)
    phase, rows = s.tick()
    assert rows[0].pos == 10 and s.stats()["prefix_rows"] == 10
    # a continuation of the whole first prompt (fork point inside the fully computed tail) keeps all of it
    s2 = Scheduler(max_lanes=1, max_rows=16, prefill_chunk=64, prefix_reuse_min=4)
    s2.set_decoder_tail(10)
    s2.submit(1, PROMPTS[1], 1)
    while s2.info(1)["state"] != "finished":
        phase, rows = s2.tick()
        s2.commit(1, len(rows), [1] if rows[-1].pos + 1 == 40 else [], 1)
    s2.submit(2, PROMPTS[1] + [5, 6, 7], 1)
    phase, rows = s2.tick()
    assert rows[0].pos == 40
