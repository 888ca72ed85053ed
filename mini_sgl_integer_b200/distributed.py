"""Tensor-parallel plumbing: the interface of ``minisgl.distributed`` (distributed/info.py:7-28,
distributed/impl.py:25-70) over ``torch.distributed``.

One process per GPU.  The reference's default PyNCCL wrapper only maps fp16/bf16
(kernel/csrc/src/pynccl.cu:59-63), so its integer mode needs the torch path (distributed/impl.py:25-41);
this module always uses it: NCCL over NVLink on GPUs, gloo on CPU (tests).  Integer sums are exact and
order-independent, so an all-reduce of int32 partial sums gives the same bits on any rank count.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class DistributedInfo:
    """distributed/info.py:7-18."""

    rank: int
    size: int

    def __post_init__(self):
        assert 0 <= self.rank < self.size

    def is_primary(self) -> bool:
        return self.rank == 0


_TP_INFO: Optional[DistributedInfo] = None


def set_tp_info(rank: int, size: int) -> None:
    """distributed/info.py:21-25 (may be set once)."""
    global _TP_INFO
    if _TP_INFO is not None:
        raise RuntimeError("TP info has been set")
    _TP_INFO = DistributedInfo(rank, size)


def get_tp_info() -> DistributedInfo:
    """distributed/info.py:28-31."""
    if _TP_INFO is None:
        raise RuntimeError("TP info has not been set")
    return _TP_INFO


def try_get_tp_info() -> Optional[DistributedInfo]:
    return _TP_INFO


def _reset_tp_info_for_tests() -> None:
    global _TP_INFO
    _TP_INFO = None


class DistributedCommunicator:
    """distributed/impl.py:63-70: ``all_reduce`` (sum) and ``all_gather`` along dim 0, plus ``all_reduce_max``.

    With a world of one every call returns its argument unchanged, as the reference does (impl.py:27-28).
    """

    def __init__(self, group=None, single: bool = False):
        """``single``: a communicator of one rank whatever process group exists (an unsplit layer built inside a
        multi-rank job, e.g. for a parity check)."""
        self.group = group
        self.single = bool(single)

    @property
    def size(self) -> int:
        if self.single:
            return 1
        return dist.get_world_size(self.group) if dist.is_initialized() else 1

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        dist.all_reduce(x, op=dist.ReduceOp.SUM, group=self.group)
        return x

    def all_reduce_max(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        dist.all_reduce(x, op=dist.ReduceOp.MAX, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        out = torch.empty((x.shape[0] * self.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out


def shard_rows(t: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """Column-parallel weight shard: output rows [rank*N/size, (rank+1)*N/size) (models/weight.py:12-52)."""
    n = t.shape[0]
    assert n % size == 0
    return t[rank * (n // size):(rank + 1) * (n // size)].contiguous()


def shard_cols(t: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    """Row-parallel weight shard: input columns [rank*K/size, (rank+1)*K/size)."""
    k = t.shape[1]
    assert k % size == 0
    return t[:, rank * (k // size):(rank + 1) * (k // size)].contiguous()
