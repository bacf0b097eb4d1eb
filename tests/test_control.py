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


def test_wire_codec_round_trips_requests_and_refuses_unknown_types():
    import dataclasses
    import torch
    from sparkflash_b200.parallel import wire
    from sparkflash_b200.serve.engine_api import EngineRequest
    req = EngineRequest("r1", "m", [1, 2, 3], temperature=0.5, stop=["x"], seed=2 ** 70, constraint={"a": [1, None, True]})
    emb = torch.arange(12, dtype=torch.float32).reshape(3, 4).to(torch.bfloat16)
    msg = {"subs": [(7, req)], "cancels": [3, 4], "emb": emb, "blob": b"\x00\x01", "t": (1.5, "s")}
    back = wire.loads(wire.dumps(msg))
    assert dataclasses.asdict(back["subs"][0][1]) == dataclasses.asdict(req) and back["subs"][0][0] == 7
    assert torch.equal(back["emb"], emb) and back["blob"] == b"\x00\x01" and back["t"] == (1.5, "s") and back["cancels"] == [3, 4]

    class Stranger:
        pass
    with pytest.raises(wire.WireError):
        wire.dumps({"x": Stranger()})
    for bad in (b"\xff", wire.dumps([1, 2])[:-1], wire.dumps(1) + b"\x00", bytes([12, 3]) + b"Foo" + bytes(4)):
        with pytest.raises(wire.WireError):
            wire.loads(bad)


def test_leader_refuses_strangers_and_ignores_ticks_from_followers():
    """A connection without the group's token, with an out-of-range rank or with a rank already taken is turned
    away; a tick frame sent *to* the leader is dropped, never decoded."""
    import socket
    import struct
    import threading
    from sparkflash_b200.parallel import control as C
    port = PORT + 7
    box = {}
    t = threading.Thread(target=lambda: box.setdefault("lead", ControlChannel(0, 2, port=port, heartbeat=0.05, timeout=5.0, token="secret")))
    t.start()

    def knock(rank, token):
        for _ in range(200):
            try:
                s = socket.create_connection(("127.0.0.1", port), timeout=2.0)
                break
            except OSError:
                time.sleep(0.02)
        nonce = C._recv_exact(s, 16)
        s.sendall(struct.pack("<I", rank) + C._answer(token, nonce, rank))
        ok = C._recv_exact(s, 1)
        return s, ok
    s1, ok1 = knock(1, b"wrong")
    s2, ok2 = knock(5, b"secret")
    assert ok1 == b"\x00" and ok2 == b"\x00"
    good = ControlChannel(1, 2, port=port, heartbeat=0.05, timeout=5.0, token="secret")
    t.join(10)
    lead = box["lead"]
    assert lead.rejected == 2
    # a follower-originated tick never reaches the leader's queue
    C._send(good._socks[0], C.TICK, b"\x80\x04garbage-that-an-unpickler-would-run", good._locks[0])
    time.sleep(0.3)
    assert lead._ticks == [] and lead.alive()[0]
    lead.broadcast({"tick": 1})
    assert good.broadcast(None) == {"tick": 1}
    good.close(); lead.close()
    s1.close(); s2.close()
