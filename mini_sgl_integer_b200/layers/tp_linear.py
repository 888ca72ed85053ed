"""Tensor-parallel W8A8 linears with Q15.16 activations.

Column-parallel (QKV, gate-up; layers/linear.py:73-105): every rank holds a block of output channels and the
whole input; no communication, and the per-token quant of the replicated input is the same on every rank.
Row-parallel (O, down; layers/linear.py:108-160): every rank holds a slice of the input features.  The
reference quantises each rank's slice with its own absmax and all-reduces the Q15.16 outputs, which makes the
result depend on the rank count.  Here the ranks first agree on the token's absmax (a [tokens] int32 max
all-reduce), quantise their slices with it, all-reduce the exact int32 accumulators and requantise once:
bit-identical to a single GPU.
"""
from __future__ import annotations

import torch

from .._lib import call, ptr, require_cuda, stream
from ..distributed import DistributedCommunicator
from ..kernel.fixed_point import absmax_to_mul_shift, assert_q15
from .w8a8_int8 import W8A8Int8LinearMethod, int8_gemm_q15


def row_absmax_q15(x_q15: torch.Tensor) -> torch.Tensor:
    """max(1, max|x|) per row as int32 [rows] (the integer absmax of per_token_quant_int8_from_q15)."""
    from ..kernel.fixed_point import per_token_quant_int8_from_q15
    _, _, absmax = per_token_quant_int8_from_q15(x_q15, return_absmax=True)
    return absmax.reshape(-1)


def quant_given_absmax(x_q15: torch.Tensor, absmax: torch.Tensor) -> torch.Tensor:
    assert_q15(x_q15, "x_q15")
    require_cuda(x_q15, absmax)
    x = x_q15.contiguous()
    k = x.shape[-1]
    rows = x.numel() // k
    codes = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    if rows:
        call("b200_quant_given_absmax_q15", ptr(x), ptr(absmax.to(torch.int32).contiguous()), ptr(codes), rows, k, stream())
    return codes


def requant_q15(acc: torch.Tensor, x_mul, x_shift, w_mul, w_shift=None) -> torch.Tensor:
    require_cuda(acc, x_mul, x_shift, w_mul, w_shift)
    acc = acc.contiguous()
    m, n = acc.shape
    out = torch.empty_like(acc)
    c = lambda t: None if t is None else t.reshape(-1).to(torch.int32).contiguous()
    if m:
        call("b200_requant_q15", ptr(acc), ptr(c(x_mul)), ptr(c(x_shift)), ptr(c(w_mul)), ptr(c(w_shift)), ptr(out), m, n, stream())
    return out


def column_parallel_q15(method: W8A8Int8LinearMethod, layer, x_q15: torch.Tensor) -> torch.Tensor:
    """``layer.weight`` is this rank's block of output channels; returns this rank's block of outputs."""
    return method.apply_weights_q15(layer, x_q15)


def row_parallel_q15(method: W8A8Int8LinearMethod, layer, x_q15_local: torch.Tensor,
                     comm: DistributedCommunicator) -> torch.Tensor:
    """``layer.weight`` is int8 [N, K/size]; ``x_q15_local`` this rank's [tokens, K/size] slice of the input.

    Returns the full Q15.16 output [tokens, N], identical on every rank and to the single-GPU result.
    """
    assert_q15(x_q15_local, "x_q15_local")
    if getattr(layer, "weight_mul", None) is None:
        method.process_weights_after_loading(layer)
    x2 = x_q15_local.reshape(-1, x_q15_local.shape[-1])
    absmax = comm.all_reduce_max(row_absmax_q15(x2))
    codes = quant_given_absmax(x2, absmax)
    acc = int8_gemm_q15(codes, None, None, layer.weight, None, want_q15=False, want_acc=True)
    acc = comm.all_reduce(acc)
    x_mul, x_shift = absmax_to_mul_shift(absmax)
    return requant_q15(acc, x_mul, x_shift, layer.weight_mul, layer.weight_shift)
