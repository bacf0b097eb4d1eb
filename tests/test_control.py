"""Control channel and failure detection on CPU ranks (processes and threads; no GPU is involved).
Reference: crates/sparkflash-comm/src/control.rs tests; fault injection on the host only."""
import multiprocessing as mp
import threading
import time

import pytest

from sparkflash_b200.parallel.control import HEARTBEAT, ChannelClosed, ControlChannel

PORT = 29711


def _follower(rank, world, port, n, q, die_after=None):
    ch = ControlChannel(rank, world, port=port, heartbeat=0.05, timeout=0.6)
    got = []
    try:
        for i in range(n):
            got.append(ch.broadcast(None))
            if die_after is not None and i + 1 == die_after:
                import os
                os._exit(1)         # the rank disappears between steps, without a goodbye
        q.put((rank, "ok", got))
        ch.close()
    except ChannelClosed as e:
        q.put((rank, "closed", str(e)))


def test_tick_broadcast_reaches_every_rank_in_order():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_follower, args=(r, 3, PORT, 5, q)) for r in (1, 2)]
    [p.start() for p in ps]
    lead = ControlChannel(0, 3, port=PORT, heartbeat=0.05, timeout=2.0)
    msgs = [{"tick": i, "subs": [("seq", [1, 2, i])], "cancels": []} for i in range(5)]
    for m in msgs:
        assert lead.broadcast(m) is m
    res = sorted(q.get(timeout=20) for _ in ps)
    assert [r[1] for r in res] == ["ok", "ok"] and res[0][2] == msgs and res[1][2] == msgs
    [p.join(5) for p in ps]
    ok, why = lead.alive()          # an orderly goodbye is still the end of the group
    assert ok or "left the group" in why
    lead.close()


def test_leader_notices_a_dead_follower_and_survivors_leave():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_follower, args=(1, 3, PORT + 1, 50, q, 2)), ctx.Process(target=_follower, args=(2, 3, PORT + 1, 50, q))]
    [p.start() for p in ps]
    lead = ControlChannel(0, 3, port=PORT + 1, heartbeat=0.05, timeout=0.6)
    t0 = time.monotonic()
    with pytest.raises(ChannelClosed):
        for i in range(50):
            lead.broadcast({"tick": i})
            time.sleep(0.05)
    assert time.monotonic() - t0 < 5 and not lead.alive()[0] and "rank 1" in lead.alive()[1]
    lead.close()          # fail-stop: the leader leaves, and the surviving follower follows it out
    rank, state, why = q.get(timeout=10)
    assert (rank, state) == (2, "closed")
    [p.join(5) for p in ps]


def test_lost_heartbeats_time_out_without_any_socket_error():
    lost = {"on": False}
    res = {}

    def follower():
        ch = ControlChannel(1, 2, port=PORT + 2, heartbeat=0.05, timeout=0.4, drop=lambda kind, d: lost["on"] and kind == HEARTBEAT and d == "out")
        try:
            while True:
                ch.broadcast(None)
        except ChannelClosed as e:
            res["why"] = str(e)
    th = threading.Thread(target=follower, daemon=True); th.start()
    lead = ControlChannel(0, 2, port=PORT + 2, heartbeat=0.05, timeout=0.4)
    lead.broadcast({"tick": 0})
    time.sleep(0.3)
    assert lead.alive()[0]
    lost["on"] = True            # the follower stays connected but falls silent (a hung rank)
    time.sleep(1.0)
    ok, why = lead.alive()
    assert not ok and "no heartbeat from rank 1" in why
    lead.close()
    th.join(5)
    assert "why" in res


def _serve_rank(rank, world, port, q):
    """One rank of a serving group on CPU: the driver over a fake rows engine, tick inputs replicated through the channel."""
    import asyncio
    from sparkflash_b200.serve.driver import DeviceDriver, FakeRowsEngine
    from sparkflash_b200.serve.engine_api import EngineRequest
    from sparkflash_b200.serve.tokenizer import ByteTokenizer
    ch = ControlChannel(rank, world, port=port, heartbeat=0.05, timeout=3.0)
    eng = FakeRowsEngine(max_rows=8)
    drv = DeviceDriver(eng, ByteTokenizer(300), channel=ch, eos_id=10 ** 9, prefix_reuse_min=1000).start()
    if rank == 0:
        async def go():
            async def one(i):
                toks = []
                async for ev in drv.generate(EngineRequest(f"r{i}", "m", list(range(40 + i, 60 + i)), max_tokens=6, temperature=0.0)):
                    if ev[0] == "token":
                        toks.append(ev[1])
                return toks
            return await asyncio.gather(*[one(i) for i in range(3)])
        out = asyncio.run(go())
        time.sleep(0.3)                       # let the followers run the last tick before the channel closes
        q.put((0, out, list(eng.steps)))
        drv.shutdown(0.5)
    else:
        while drv.failed is None and ch.alive()[0]:
            time.sleep(0.05)
        q.put((rank, None, list(eng.steps)))


def test_followers_replay_the_leaders_ticks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_serve_rank, args=(r, 2, PORT + 5, q)) for r in range(2)]
    [p.start() for p in ps]
    got = sorted([q.get(timeout=60) for _ in ps], key=lambda t: t[0])
    [p.join(10) for p in ps]
    lead_steps, foll_steps = [s for s in got[0][2]], [s for s in got[1][2]]
    assert all(len(t) == 6 for t in got[0][1])
    # the follower ran the same rows steps in the same order (it may miss only ticks after the leader's last answer)
    assert foll_steps[:len(lead_steps)] == lead_steps[:len(foll_steps)] and len(foll_steps) >= len(lead_steps) - 1 and len(foll_steps) > 5
