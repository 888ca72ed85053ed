"""A linear whose requantisation is left to the kernel that reads its output.

At decode sizes a launch costs as much as the work in it, so the split-K linear leaves its exact int32 accumulators
in a workspace and the consumer (add + RMSNorm + quant, or the q/k/v preparation) applies the fixed-point epilogue
while it loads them - the same bits as the materialised Q15.16 tensor of ``apply_weights_q15``
(layers/quantization/w8a8_int8.py:242-286), two launches fewer per linear.

The workspace protocol: a buffer is all zero whenever no linear is pending in it.  The GEMM adds its split-K parts
into it (no clearing launch), the consumer zeroes every element it reads.  Buffers are kept per (device, width)
and shared by the linears of that width; calls on one stream follow each other, so at most one linear is pending
in a buffer at a time.  Work issued to several streams that may overlap on the device takes a buffer set of its
own per stream with ``workspace_scope(tag)``.  Not for use from several host threads at once.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .._lib import call, ptr, stream

__all__ = ["PendingLinear", "zero_workspace", "workspace_scope", "reset_workspaces", "PENDING_MAX_ROWS"]

PENDING_MAX_ROWS = 256          # the GEMM splits K (and needs a zeroed buffer) up to this many token rows

_workspaces: dict = {}
_scope = [0]


class workspace_scope:
    """``with workspace_scope(tag):`` linears issued inside use the buffer set `tag` (any hashable), so that two streams
    whose kernels may run at the same time never share a workspace."""

    def __init__(self, tag):
        self.tag, self.prev = tag, None

    def __enter__(self):
        self.prev, _scope[0] = _scope[0], self.tag
        return self

    def __exit__(self, *exc):
        _scope[0] = self.prev
        return False


def zero_workspace(device: torch.device, rows: int, n: int) -> torch.Tensor:
    """An all-zero int32 [rows, n] view of the buffer kept for (device, n, scope); grows (zeroed) when rows exceed it."""
    index = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    key = (index, n, _scope[0])
    buf = _workspaces.get(key)
    if buf is None or buf.shape[0] < rows:
        cap = max(rows, PENDING_MAX_ROWS)
        buf = torch.zeros((cap, n), dtype=torch.int32, device=device)
        _workspaces[key] = buf
    return buf[:rows]


def reset_workspaces() -> None:
    """Zeroes every workspace: after an exception between a pending linear and its consumer (the one situation that
    leaves a buffer dirty), before the buffers are used again."""
    for buf in _workspaces.values():
        buf.zero_()


@dataclass
class PendingLinear:
    acc: torch.Tensor                       # int32 [rows, n]: exact accumulators, inside a zero workspace
    x_absmax: torch.Tensor                  # int32 [rows]: absmax of each token's input row
    weight_mul: torch.Tensor                # int32 [n]
    weight_shift: Optional[torch.Tensor]    # int32 [n] or None (31)

    @property
    def shape(self):
        return self.acc.shape

    @property
    def device(self):
        return self.acc.device

    def materialise(self) -> torch.Tensor:
        """The Q15.16 tensor, for a consumer without a fused form; the workspace is zero again afterwards."""
        rows, n = self.acc.shape
        out = torch.empty((rows, n), dtype=torch.int32, device=self.acc.device)
        if rows:
            from .fixed_point import absmax_to_mul_shift
            x_mul, x_shift = absmax_to_mul_shift(self.x_absmax.reshape(-1))
            call("b200_requant_q15", ptr(self.acc), ptr(x_mul), ptr(x_shift), ptr(self.weight_mul), ptr(self.weight_shift),
                 ptr(out), rows, n, stream())
            self.acc.zero_()
        return out
