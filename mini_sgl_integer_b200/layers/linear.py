"""Tensor-parallel W8A8 linear layers with Q15.16 activations: the classes of ``minisgl.layers.linear``
(layers/linear.py:24-160) for int8 checkpoints.

Same constructors and sharding.  ``forward`` takes a Q15.16 int32 activation and returns Q15.16 (the branch
``x.dtype == torch.int32`` of the reference, :42-49).  Row-split layers (O, down) keep the result independent of
the rank count: the ranks agree on the token's absmax, add the exact int32 accumulators and requantise once
(`tp_linear.row_parallel_q15`), over NCCL or, when an exchange block has been installed with
``set_tp_exchange``, over peer memory without a collective call.  Float weights are out of scope here.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..distributed import DistributedCommunicator, get_tp_info
from .base import BaseOP
from .tp_linear import TpExchange, row_parallel_q15
from .w8a8_int8 import W8A8Int8LinearMethod

_METHOD = W8A8Int8LinearMethod()
_EXCHANGE: Optional[TpExchange] = None


def set_tp_exchange(exchange: Optional[TpExchange]) -> None:
    """Install (or remove) the peer-memory exchange block that the row-split layers of this process use."""
    global _EXCHANGE
    _EXCHANGE = exchange


def div_even(a: int, b: int) -> int:
    if a % b:
        raise ValueError(f"{a} is not divisible by {b}")
    return a // b


class _LinearTPImpl(BaseOP):
    def __init__(self, full_isize: int, full_osize: int, local_isize: int, local_osize: int, has_bias: bool):
        self.full_input_size, self.full_output_size = full_isize, full_osize
        self.local_input_size, self.local_output_size = local_isize, local_osize
        self.weight = torch.empty(local_osize, local_isize)
        self.bias = torch.empty(local_osize) if has_bias else None

    def _check(self, x: torch.Tensor) -> None:
        if self.weight.dtype != torch.int8 or not hasattr(self, "weight_scale"):
            raise TypeError("this layer runs int8 checkpoints only (int8 `weight` plus `weight_scale`); "
                            "the float model is not part of the integer path")
        if x.dtype != torch.int32:
            raise TypeError(f"the activation must be Q15.16 int32, got {x.dtype}")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._check(x)
        return _METHOD.apply_weights_q15(self, x, self.bias)


class LinearReplicated(_LinearTPImpl):
    def __init__(self, input_size: int, output_size: int, has_bias: bool):
        super().__init__(input_size, output_size, input_size, output_size, has_bias)


class LinearColParallelMerged(_LinearTPImpl):
    def __init__(self, input_size: int, output_sizes: List[int], has_bias: bool):
        tp = get_tp_info().size
        super().__init__(input_size, sum(output_sizes), input_size, sum(div_even(s, tp) for s in output_sizes), has_bias)


class LinearQKVMerged(_LinearTPImpl):
    def __init__(self, hidden_size: int, head_dim: int, num_qo_heads: int, num_kv_heads: int, has_bias: bool):
        tp = get_tp_info().size
        ratio = div_even(num_qo_heads, num_kv_heads)
        local_kv = div_even(num_kv_heads, tp)
        super().__init__(hidden_size, (ratio + 2) * num_kv_heads * head_dim, hidden_size, (ratio + 2) * local_kv * head_dim, has_bias)


class _RowSplit(_LinearTPImpl):
    def __init__(self, input_size: int, output_size: int, has_bias: bool):
        tp = get_tp_info()
        self._comm = DistributedCommunicator()
        self._tp_size = tp.size
        super().__init__(input_size, output_size, div_even(input_size, tp.size), output_size, has_bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        self._check(x)
        if self._tp_size == 1:
            return _METHOD.apply_weights_q15(self, x, self.bias)
        rows = x.reshape(-1, x.shape[-1]).shape[0]
        if _EXCHANGE is not None and _EXCHANGE.fits(rows, self.local_output_size):
            y = _EXCHANGE.row_parallel_q15(_METHOD, self, x)
        else:
            y = row_parallel_q15(_METHOD, self, x, self._comm)
        if self.bias is not None:
            y = _METHOD._add_bias(y, self.bias)
        return y.reshape(*x.shape[:-1], -1)


class LinearOProj(_RowSplit):
    pass


class LinearRowParallel(_RowSplit):
    pass


__all__ = ["LinearReplicated", "LinearColParallelMerged", "LinearQKVMerged", "LinearOProj", "LinearRowParallel", "set_tp_exchange"]
