"""Tensor-parallel W8A8 linears with Q15.16 activations.

Column-parallel (QKV, gate-up; layers/linear.py:73-105): every rank holds a block of output channels and the
whole input; no communication, and the per-token quant of the replicated input is the same on every rank.
Row-parallel (O, down; layers/linear.py:108-160): every rank holds a slice of the input features.  The
reference quantises each rank's slice with its own absmax and all-reduces the Q15.16 outputs, which makes the
result depend on the rank count.  Here the ranks first agree on the token's absmax (a [tokens] int32 max
all-reduce), quantise their slices with it, all-reduce the exact int32 accumulators and requantise once:
bit-identical to a single GPU.

The sum of the accumulators comes in two forms: an NCCL all-reduce after the GEMM (`row_parallel_q15`), or, at
decode sizes, inside the GEMM kernel itself (`row_parallel_q15_fused`): every accumulator tile is added, as it
leaves tensor memory, into the accumulators of all ranks through NVLink peer memory (`PeerReduceBuffers`), so
the transfer overlaps the MMAs and no separate collective kernel runs.
"""
from __future__ import annotations

import ctypes

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


class PeerReduceBuffers:
    """int32 accumulators [2][m_max, n] in symmetric memory, one set per rank, every rank's mapped into every
    process (``torch.distributed._symmetric_memory``).  Two halves are used alternately: a half is zeroed right
    after its result has been read, and the barrier of the following call (on the other half) orders that
    zeroing before any peer adds into it again."""

    def __init__(self, comm: DistributedCommunicator, m_max: int, n: int, device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.m_max, self.n, self.size = int(m_max), int(n), comm.size
        self.buf = symm_mem.empty((2, self.m_max, self.n), dtype=torch.int32, device=device)
        self.handle = symm_mem.rendezvous(self.buf, comm.group if comm.group is not None else dist.group.WORLD)
        self.buf.zero_()
        self.handle.barrier(channel=0)
        half_bytes = self.m_max * self.n * 4
        bases = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_ptrs = [(ctypes.c_void_p * self.size)(*[b + h * half_bytes for b in bases]) for h in (0, 1)]
        self.calls = 0


def row_parallel_q15_fused(method: W8A8Int8LinearMethod, layer, x_q15_local: torch.Tensor,
                           comm: DistributedCommunicator, bufs: PeerReduceBuffers) -> torch.Tensor:
    """`row_parallel_q15` with the sum of the accumulators done by the GEMM kernel over peer memory (tokens <= 256
    and <= bufs.m_max, layer.weight.shape[0] == bufs.n); same bits."""
    assert_q15(x_q15_local, "x_q15_local")
    if getattr(layer, "weight_mul", None) is None:
        method.process_weights_after_loading(layer)
    x2 = x_q15_local.reshape(-1, x_q15_local.shape[-1])
    m, k = x2.shape
    n = layer.weight.shape[0]
    if m > min(256, bufs.m_max) or n != bufs.n:
        return row_parallel_q15(method, layer, x_q15_local, comm)
    absmax = comm.all_reduce_max(row_absmax_q15(x2))
    codes = quant_given_absmax(x2, absmax)
    half = bufs.calls & 1
    bufs.calls += 1
    if m:
        call("b200_gemm_w8a8_reduce_peers", ptr(codes), ptr(layer.weight.contiguous()), bufs.peer_ptrs[half], bufs.size,
             m, n, k, stream())
    bufs.handle.barrier(channel=half)                  # every rank's additions have landed
    acc = bufs.buf[half, :m]
    x_mul, x_shift = absmax_to_mul_shift(absmax)
    out = requant_q15(acc, x_mul, x_shift, layer.weight_mul, layer.weight_shift)
    acc.zero_()                                        # ready for its next use, two calls from now
    return out
