"""Collectives of the tensor-parallel forward.

Two arms behind one small interface (reference: crates/sparkflash-comm/src/device_reduce.rs:587-1082
``RunReduce``; crates/sparkflash-ops/src/collective.rs:29-150 ``CollectivePlan``):

* ``NcclComm``  - the baseline arm: NCCL all-reduce / all-gather through torch.distributed.
* ``FusedComm`` - this framework's own arm: every rank's producer kernel pushes its bf16 partial into
  a slot of every peer's symmetric buffer over NVLink and raises a flag; the consumer (the mHC seam)
  folds the slots in rank order in fp32.  See parallel/symm.py and csrc/k_comm.cu.

``parts(y, n)`` returns what the next seam must fold: a list of per-rank partial buffers.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class NcclComm:
    name = "nccl"
    wait_ns = 0

    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world
        self.calls = 0

    def attach(self, engine) -> None:
        self.engine = engine

    def parts(self, y: torch.Tensor, n: int):
        dist.all_reduce(y[:n])
        self.calls += 1
        return [y]

    def gather_best(self, best_val: torch.Tensor, best_id: torch.Tensor, n: int) -> None:
        dist.all_gather_into_tensor(best_val, best_val[self.rank])
        dist.all_gather_into_tensor(best_id, best_id[self.rank])


def make_comm(kind: str, rank: int, world: int):
    if kind == "nccl":
        return NcclComm(rank, world)
    if kind == "fused":
        from .fused import FusedComm
        return FusedComm(rank, world)
    raise ValueError(f"unknown collective arm {kind!r}")
