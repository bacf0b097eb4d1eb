"""Host transports for CPU ranks: all-reduce / all-gather of bf16 rows over an in-process loopback or TCP, with the
canonical rank-order fold, plus per-collective telemetry.

The device collectives (parallel/fused.py, csrc/k_comm.cu) fold the ranks' partials in rank order in fp32 and round to
bf16 once.  These transports do exactly that on the host, so a CPU-rank run (tests of the tick protocol, the oracle's
TP-seam simulation, the host serving arm) gives the bits a GPU group gives, whatever order the messages arrive in.

Reference: crates/sparkflash-comm/src/{transport,tcp,loopback}.rs (``Transport`` trait: all_reduce_bf16, all_gather_bf16),
telemetry.rs, tests reduction_bits.rs / reduce_path_bits.rs (every reduce arm gives the same bits).
"""
from __future__ import annotations

import socket
import struct
import threading
import time
from dataclasses import dataclass, field

import torch


def fold_rank_order(parts: list[torch.Tensor]) -> torch.Tensor:
    """fp32 sum of the ranks' bf16 partials in rank order 0..W-1, one bf16 rounding at the end."""
    acc = parts[0].float().clone()
    for p in parts[1:]:
        acc += p.float()
    return acc.to(torch.bfloat16)


@dataclass
class Telemetry:
    """Counts and times per collective kind (exposed through /v1/cluster/stats and the shutdown log)."""
    calls: dict = field(default_factory=dict)
    bytes: dict = field(default_factory=dict)
    seconds: dict = field(default_factory=dict)
    worst: dict = field(default_factory=dict)

    def note(self, kind: str, nbytes: int, dt: float) -> None:
        self.calls[kind] = self.calls.get(kind, 0) + 1
        self.bytes[kind] = self.bytes.get(kind, 0) + nbytes
        self.seconds[kind] = self.seconds.get(kind, 0.0) + dt
        self.worst[kind] = max(self.worst.get(kind, 0.0), dt)

    def snapshot(self) -> dict:
        return {k: {"calls": self.calls[k], "bytes": self.bytes[k], "mean_us": 1e6 * self.seconds[k] / self.calls[k],
                    "worst_us": 1e6 * self.worst[k]} for k in self.calls}


class Transport:
    """Interface: ``all_reduce_bf16(x)`` (in place, returns x), ``all_gather_bf16(x)`` -> [W, ...]."""
    rank: int
    world: int

    def __init__(self):
        self.telemetry = Telemetry()

    def exchange(self, payload: bytes) -> list[bytes]:
        raise NotImplementedError

    def all_gather_bf16(self, x: torch.Tensor) -> torch.Tensor:
        t0 = time.perf_counter()
        raw = x.contiguous().view(torch.uint8).numpy().tobytes()
        got = self.exchange(raw)
        out = torch.stack([torch.frombuffer(bytearray(b), dtype=torch.uint8).view(torch.bfloat16).reshape(x.shape) for b in got])
        self.telemetry.note("all_gather", len(raw) * (self.world - 1), time.perf_counter() - t0)
        return out

    def all_reduce_bf16(self, x: torch.Tensor) -> torch.Tensor:
        t0 = time.perf_counter()
        parts = self.all_gather_bf16(x)
        x.copy_(fold_rank_order(list(parts)))
        self.telemetry.note("all_reduce", x.numel() * 2 * (self.world - 1), time.perf_counter() - t0)
        return x

    def barrier(self) -> None:
        self.exchange(b"")

    def close(self) -> None:
        pass


class LoopbackCluster:
    """W transports inside one process (rank threads).  A rank that never joins an exchange makes the others time out."""

    def __init__(self, world: int, timeout: float = 5.0):
        self.world, self.timeout = world, timeout
        self._lock = threading.Condition()
        self._round: dict[int, dict[int, bytes]] = {}
        self._seq = [0] * world
        self.transports = [LoopbackTransport(self, r) for r in range(world)]

    def _exchange(self, rank: int, payload: bytes) -> list[bytes]:
        with self._lock:
            seq = self._seq[rank]
            self._seq[rank] += 1
            slot = self._round.setdefault(seq, {})
            slot[rank] = payload
            self._lock.notify_all()
            deadline = time.monotonic() + self.timeout
            while len(slot) < self.world:
                left = deadline - time.monotonic()
                if left <= 0:
                    missing = sorted(set(range(self.world)) - set(slot))
                    raise TimeoutError(f"exchange {seq}: ranks {missing} never arrived")
                self._lock.wait(left)
            out = [slot[r] for r in range(self.world)]
            slot.setdefault("_taken", 0)
            slot["_taken"] += 1
            if slot["_taken"] == self.world:
                del self._round[seq]
            return out


class LoopbackTransport(Transport):
    def __init__(self, cluster: LoopbackCluster, rank: int):
        super().__init__()
        self.cluster, self.rank, self.world = cluster, rank, cluster.world

    def exchange(self, payload: bytes) -> list[bytes]:
        return self.cluster._exchange(self.rank, payload)


def _recv_exact(s: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = s.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the transport")
        buf += chunk
    return bytes(buf)


class TcpTransport(Transport):
    """Star over TCP: rank 0 listens, gathers every rank's payload and sends the whole set back.  Frames are
    ``u32 length | bytes``; payloads are raw tensor bytes, nothing is deserialised into objects."""

    def __init__(self, rank: int, world: int, addr: str = "127.0.0.1", port: int = 29650, timeout: float = 10.0):
        super().__init__()
        self.rank, self.world = rank, world
        self._peers: dict[int, socket.socket] = {}
        if world == 1:
            return
        if rank == 0:
            srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port)); srv.listen(world)
            srv.settimeout(timeout)
            try:
                while len(self._peers) < world - 1:
                    s, _ = srv.accept()
                    s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
                    s.settimeout(timeout)
                    r = struct.unpack("<I", _recv_exact(s, 4))[0]
                    if not 1 <= r < world or r in self._peers:
                        s.close()
                        continue
                    self._peers[r] = s
            finally:
                srv.close()
        else:
            t0 = time.monotonic()
            while True:
                try:
                    s = socket.create_connection((addr, port), timeout=2.0)
                    break
                except OSError:
                    if time.monotonic() - t0 > timeout:
                        raise
                    time.sleep(0.02)
            s.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            s.settimeout(timeout)
            s.sendall(struct.pack("<I", rank))
            self._peers[0] = s

    def exchange(self, payload: bytes) -> list[bytes]:
        if self.world == 1:
            return [payload]
        if self.rank == 0:
            got = {0: payload}
            for r, s in self._peers.items():
                ln = struct.unpack("<I", _recv_exact(s, 4))[0]
                got[r] = _recv_exact(s, ln) if ln else b""
            frame = b"".join(struct.pack("<I", len(got[r])) + got[r] for r in range(self.world))
            for s in self._peers.values():
                s.sendall(frame)
            return [got[r] for r in range(self.world)]
        s = self._peers[0]
        s.sendall(struct.pack("<I", len(payload)) + payload)
        out = []
        for _ in range(self.world):
            ln = struct.unpack("<I", _recv_exact(s, 4))[0]
            out.append(_recv_exact(s, ln) if ln else b"")
        return out

    def close(self) -> None:
        for s in self._peers.values():
            try:
                s.close()
            except OSError:
                pass
        self._peers = {}
