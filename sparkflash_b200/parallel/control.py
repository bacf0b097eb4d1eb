"""Control channel between the ranks of one serving group: rank 0 broadcasts the inputs of every tick, every
rank sends heartbeats, and each side notices when the other stops.

Wire: TCP, frames of ``u32 length | u8 kind | payload`` (kind 0 tick, 1 heartbeat, 2 goodbye).  Tick payloads
are plain data in the tagged binary encoding of ``wire.py`` - nothing on this socket is ever unpickled.  The
leader keeps one socket per follower; a connection is admitted only after it answers the leader's random
challenge with an HMAC under the group's shared token and announces a rank in 1..world-1 that nobody holds
yet.  Tick frames are accepted from the leader only: the leader drops any that a follower sends.  Liveness is host-side only - a rank that stops answering is detected by a
missing heartbeat, never by waiting on the device.  Policy is fail-stop: when any rank is lost the group
stops serving and an outside supervisor restarts it.

Reference: crates/sparkflash-comm/src/control.rs (watch_workers:731, watch_leader:770, exit_now:719),
crates/sparkflash-cli/src/serve/device.rs:1085-1107,1182-1191 (DeviceLink::fail, followers leave when the
channel closes), crates/sparkflash-comm/src/tcp.rs.
"""
from __future__ import annotations

import hashlib
import hmac
import os
import socket
import struct
import threading
import time

from . import wire

TICK, HEARTBEAT, GOODBYE = 0, 1, 2


class ChannelClosed(Exception):
    pass


def _send(sock: socket.socket, kind: int, payload: bytes, lock: threading.Lock) -> None:
    with lock:
        sock.sendall(struct.pack("<IB", len(payload), kind) + payload)


def _recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = b""
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ChannelClosed("peer closed the control channel")
        buf += chunk
    return buf


MAX_FRAME = 1 << 30


def _recv(sock: socket.socket) -> tuple[int, bytes]:
    ln, kind = struct.unpack("<IB", _recv_exact(sock, 5))
    if ln > MAX_FRAME:
        raise ChannelClosed("oversized control frame")
    return kind, _recv_exact(sock, ln) if ln else b""


def _default_token() -> bytes:
    """Shared secret of the group: ``SFB_CONTROL_TOKEN`` when set (multi-node launches export the same value on
    every node), else a value derived from the rendezvous address every rank already agrees on."""
    t = os.environ.get("SFB_CONTROL_TOKEN")
    if t:
        return t.encode()
    return f"sfb:{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{os.environ.get('MASTER_PORT', '0')}".encode()


def _answer(token: bytes, nonce: bytes, rank: int) -> bytes:
    return hmac.new(token, nonce + struct.pack("<I", rank), hashlib.sha256).digest()


class ControlChannel:
    """``broadcast(msg)``: on rank 0 sends ``msg`` to every follower and returns it; on a follower ignores its
    argument and returns the leader's next message (blocking, bounded by ``timeout``)."""

    def __init__(self, rank: int, world: int, addr: str = "127.0.0.1", port: int = 29600, heartbeat: float = 0.5,
                 timeout: float = 5.0, connect_timeout: float = 60.0, drop=None, token: bytes | str | None = None):
        self.rank, self.world = rank, world
        token = _default_token() if token is None else (token.encode() if isinstance(token, str) else token)
        self.rejected = 0                      # connections the leader turned away (bad token, bad or duplicate rank)
        self.heartbeat, self.timeout = heartbeat, timeout
        self._drop = drop                      # test hook: drop(kind, direction) -> True to lose the frame
        self._lock = threading.Lock()
        self._closed = False
        self._failed: str | None = None
        self.departed: set[int] = set()      # peers that said goodbye
        self._last_seen: dict[int, float] = {}
        self._ticks: list = []
        self._cv = threading.Condition()
        self._socks: dict[int, socket.socket] = {}
        self._locks: dict[int, threading.Lock] = {}
        if world == 1:
            return
        if rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port)); srv.listen(world)
            srv.settimeout(connect_timeout)
            try:
                while len(self._socks) < world - 1:
                    s, _ = srv.accept()
                    s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                    try:
                        s.settimeout(5.0)
                        nonce = os.urandom(16)
                        s.sendall(nonce)
                        hello = _recv_exact(s, 4 + 32)
                        r = struct.unpack("<I", hello[:4])[0]
                        good = 1 <= r < world and r not in self._socks and hmac.compare_digest(hello[4:], _answer(token, nonce, r))
                        s.sendall(b"\x01" if good else b"\x00")
                        s.settimeout(None)
                    except (OSError, ChannelClosed):
                        good = False
                    if not good:
                        self.rejected += 1
                        s.close()
                        continue
                    self._socks[r], self._locks[r] = s, threading.Lock()
                    self._last_seen[r] = time.monotonic()
            finally:
                srv.close()
        else:
            t0 = time.monotonic()
            while True:
                try:
                    s = socket.create_connection((addr, port), timeout=2.0)
                    break
                except OSError:
                    if time.monotonic() - t0 > connect_timeout:
                        raise
                    time.sleep(0.05)
            s.settimeout(10.0)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            nonce = _recv_exact(s, 16)
            s.sendall(struct.pack("<I", rank) + _answer(token, nonce, rank))
            if _recv_exact(s, 1) != b"\x01":
                s.close()
                raise ChannelClosed("the leader refused this rank (token mismatch, or the rank is out of range or taken)")
            s.settimeout(None)
            self._socks[0], self._locks[0] = s, threading.Lock()
            # the leader only starts beating once every rank has joined: until its first frame arrives the silence is
            # bounded by the connect timeout, not by the heartbeat timeout
            self._last_seen[0] = time.monotonic() + connect_timeout - timeout
        for peer, s in self._socks.items():
            threading.Thread(target=self._reader, args=(peer, s), daemon=True).start()
        threading.Thread(target=self._beater, daemon=True).start()

    # ---- background -----------------------------------------------------------------------------------
    def _reader(self, peer: int, s: socket.socket) -> None:
        try:
            while not self._closed:
                kind, payload = _recv(s)
                if self._drop and self._drop(kind, "in"):
                    continue
                self._last_seen[peer] = time.monotonic()
                if kind == TICK:
                    if self.rank == 0:
                        continue                     # only the leader originates ticks
                    try:
                        msg = wire.loads(payload)
                    except (wire.WireError, struct.error, UnicodeDecodeError, TypeError) as e:
                        self._fail(f"rank {peer}: malformed tick ({e})")
                        return
                    with self._cv:
                        self._ticks.append(msg)
                        self._cv.notify_all()
                elif kind == GOODBYE:
                    self.departed.add(peer)          # an orderly leave (drain), as opposed to a silent or broken peer
                    self._fail(f"rank {peer} left the group")
                    return
        except (ChannelClosed, OSError) as e:
            if not self._closed:
                self._fail(f"rank {peer}: {e}")

    def _beater(self) -> None:
        while not self._closed and self._failed is None:
            for peer, s in list(self._socks.items()):
                try:
                    if not (self._drop and self._drop(HEARTBEAT, "out")):
                        _send(s, HEARTBEAT, b"", self._locks[peer])
                except OSError as e:
                    self._fail(f"rank {peer}: {e}")
            now = time.monotonic()
            for peer, t in list(self._last_seen.items()):
                if now - t > self.timeout:
                    self._fail(f"no heartbeat from rank {peer} for {now - t:.1f}s")
            time.sleep(self.heartbeat)

    def _fail(self, why: str) -> None:
        if self._failed is None:
            self._failed = why
        with self._cv:
            self._cv.notify_all()

    # ---- API --------------------------------------------------------------------------------------------
    def alive(self) -> tuple[bool, str]:
        return (self._failed is None, self._failed or "ok")

    def broadcast(self, msg):
        if self.world == 1:
            return msg
        if self._failed:
            raise ChannelClosed(self._failed)
        if self.rank == 0:
            payload = wire.dumps(msg)
            for peer, s in self._socks.items():
                try:
                    if not (self._drop and self._drop(TICK, "out")):
                        _send(s, TICK, payload, self._locks[peer])
                except OSError as e:
                    self._fail(f"rank {peer}: {e}")
                    raise ChannelClosed(self._failed)
            return msg
        with self._cv:
            deadline = time.monotonic() + max(self.timeout, 1.0) * 4
            while not self._ticks:
                if self._failed:
                    raise ChannelClosed(self._failed)
                left = deadline - time.monotonic()
                if left <= 0:
                    self._failed = self._failed or "no tick from the leader"
                    raise ChannelClosed(self._failed)
                self._cv.wait(min(left, 0.2))
            return self._ticks.pop(0)

    def close(self) -> None:
        if self._closed:
            return
        for peer, s in self._socks.items():
            try:
                _send(s, GOODBYE, b"", self._locks[peer])
            except OSError:
                pass
        self._closed = True
        for s in self._socks.values():
            try:
                s.shutdown(socket.SHUT_RDWR)
            except OSError:
                pass
            s.close()
