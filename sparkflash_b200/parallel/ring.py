"""Latent-recurrence ring: pipeline parallelism for models that run one shared block many times (Dory family).
No rank holds a slice of a layer and nothing is reduced: rank r runs its share of the recurrent loops on the whole
hidden width and passes the latent rows on; the last rank runs the head and answers rank 0.  While one lane's step is on
rank 2, another lane's can be on rank 1: the ring is kept busy by lanes, not by splitting a step.

Messages are a fixed header (kind, lane, position, rows) followed by the latent rows, sent with point-to-point
``torch.distributed`` operations (NCCL between GPUs, gloo in the CPU tests).  Every rank handles frames in arrival order, so
answers come back in the order the steps were sent.  Reference: crates/sparkflash-model-dory/src/recurrence.rs:15-84.
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

STEP, SHUTDOWN = 1, 2
HEADER = 4


class RingStage:
    """``stage_fn(lane, pos, latent[rows, d]) -> latent`` runs this rank's loops (and keeps this rank's per-lane caches);
    ``head_fn(lane, pos, latent) -> int64 tokens [rows]`` runs on the last rank."""

    def __init__(self, stage_fn: Callable, head_fn: Callable | None, d: int, device="cpu", group=None):
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.stage_fn, self.head_fn, self.d, self.dev, self.group = stage_fn, head_fn, d, device, group
        self.nxt, self.prev = (self.rank + 1) % self.world, (self.rank - 1) % self.world

    def _send(self, dst: int, kind: int, lane: int, pos: int, payload: torch.Tensor | None) -> None:
        rows = 0 if payload is None else payload.shape[0]
        dist.send(torch.tensor([kind, lane, pos, rows], dtype=torch.int64, device=self.dev), dst, group=self.group)
        if rows:
            dist.send(payload.contiguous(), dst, group=self.group)

    def _recv(self, src: int, width: int, dtype) -> tuple[int, int, int, torch.Tensor | None]:
        h = torch.empty(HEADER, dtype=torch.int64, device=self.dev)
        dist.recv(h, src, group=self.group)
        kind, lane, pos, rows = (int(x) for x in h)
        payload = None
        if rows:
            payload = torch.empty((rows, width), dtype=dtype, device=self.dev)
            dist.recv(payload, src, group=self.group)
        return kind, lane, pos, payload

    # ---- rank 0 -------------------------------------------------------------------------------------------------
    def drive(self, steps: list[tuple[int, int, torch.Tensor]]) -> list[torch.Tensor]:
        """Rank 0: run ``steps`` = [(lane, pos, embedded rows)] through the ring, keeping up to world-1 steps in flight,
        and return each step's tokens in order."""
        assert self.rank == 0
        if self.world == 1:
            return [self.head_fn(l, p, self.stage_fn(l, p, x)) for l, p, x in steps]
        answers, sent = [], 0
        inflight = 0
        while len(answers) < len(steps):
            while sent < len(steps) and inflight < self.world - 1:
                lane, pos, x = steps[sent]
                self._send(self.nxt, STEP, lane, pos, self.stage_fn(lane, pos, x))
                sent += 1; inflight += 1
            _, _, _, toks = self._recv(self.world - 1, 1, torch.int64)       # the last rank answers rank 0 directly
            answers.append(toks.flatten())
            inflight -= 1
        return answers

    def shutdown(self) -> None:
        if self.rank == 0 and self.world > 1:
            self._send(self.nxt, SHUTDOWN, 0, 0, None)

    # ---- ranks 1..W-1 ---------------------------------------------------------------------------------------------
    def serve(self) -> int:
        """Every other rank: take frames in arrival order until the shutdown frame; returns how many steps it ran."""
        assert self.rank != 0
        n = 0
        while True:
            kind, lane, pos, x = self._recv(self.prev, self.d, torch.float32)
            if kind == SHUTDOWN:
                if self.rank != self.world - 1:
                    self._send(self.nxt, SHUTDOWN, 0, 0, None)
                return n
            y = self.stage_fn(lane, pos, x)
            n += 1
            if self.rank == self.world - 1:
                toks = self.head_fn(lane, pos, y).reshape(-1, 1).to(torch.int64)
                self._send(0, STEP, lane, pos, toks)
            else:
                self._send(self.nxt, STEP, lane, pos, y)
