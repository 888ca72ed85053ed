"""Tensor-parallel W8A8 linears with Q15.16 activations.

Column-parallel (QKV, gate-up; layers/linear.py:73-105): every rank holds a block of output channels and the
whole input; no communication, and the per-token quant of the replicated input is the same on every rank.
Row-parallel (O, down; layers/linear.py:108-160): every rank holds a slice of the input features.  The
reference quantises each rank's slice with its own absmax and all-reduces the Q15.16 outputs, which makes the
result depend on the rank count.  Here the ranks first agree on the token's absmax (a [tokens] int32 max
all-reduce), quantise their slices with it, all-reduce the exact int32 accumulators and requantise once:
bit-identical to a single GPU.

The sum of the accumulators comes in three forms: an NCCL all-reduce after the GEMM (`row_parallel_q15`); at
decode sizes, inside the GEMM kernel itself (`row_parallel_q15_fused`): every accumulator tile is added, as it
leaves tensor memory, into the accumulators of all ranks through NVLink peer memory (`PeerReduceBuffers`), so
the transfer overlaps the MMAs and no separate collective kernel runs; and `TpExchange.row_parallel_q15`, where
the absmax agreement and the cross-rank ordering run over peer memory as well (signal at the end of the
producing kernel, bounded wait at the start of the consuming one), so that a tensor-parallel decode step
contains no collective call at all and can be captured in a CUDA graph on every rank.
"""
from __future__ import annotations

import ctypes
from typing import Optional

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


class _TpBlockStruct(ctypes.Structure):
    """b200_tp_block of include/b200int.h."""
    _fields_ = [("rank", ctypes.c_int), ("size", ctypes.c_int), ("m_max", ctypes.c_int), ("n", ctypes.c_int64),
                ("base", ctypes.c_void_p * 8)]


class TpExchange:
    """One rank's view of the tensor-parallel exchange blocks (see ``b200_tp_block`` in include/b200int.h).

    ``TpExchange(comm, m_max, n, device)`` allocates this rank's block in symmetric memory
    (``torch.distributed._symmetric_memory``) and maps every peer's; ``TpExchange.emulated`` builds the views of
    ``size`` ranks over blocks that all live on ONE device, for tests that run the ranks' calls one after the
    other on one stream (every wait then finds its flags already set).
    """

    def __init__(self, comm: DistributedCommunicator | None, m_max: int, n: int, device, *, _bases=None, _rank=None,
                 _keep=None):
        from .._lib import load
        self.m_max, self.n = int(m_max), int(n)
        self.nbytes = int(load().b200_tp_block_bytes(self.m_max, self.n))
        if _bases is None:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            self.size = comm.size
            self.rank = dist.get_rank(comm.group)
            self._buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
            self._handle = symm_mem.rendezvous(self._buf, comm.group if comm.group is not None else dist.group.WORLD)
            bases = [int(p) for p in self._handle.buffer_ptrs]
        else:
            self.size, self.rank, self._buf, self._handle = len(_bases), int(_rank), _keep, None
            bases = list(_bases)
        self.blk = _TpBlockStruct(self.rank, self.size, self.m_max, self.n, (ctypes.c_void_p * 8)(*(bases + [None] * (8 - len(bases)))))
        self._p = ctypes.byref(self.blk)
        if _bases is None:
            call("b200_tp_block_clear", self._p, stream())
            torch.cuda.current_stream().synchronize()
            dist.barrier(group=comm.group)                      # every rank's block is clear before anybody writes

    @classmethod
    def emulated(cls, size: int, m_max: int, n: int, device="cuda") -> list["TpExchange"]:
        from .._lib import load
        nbytes = int(load().b200_tp_block_bytes(int(m_max), int(n)))
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(size)]
        bases = [b.data_ptr() for b in bufs]
        return [cls(None, m_max, n, device, _bases=bases, _rank=r, _keep=bufs) for r in range(size)]

    # ---- the five steps of a row-split linear (separately, so that emulated ranks can be interleaved)
    def absmax_put(self, x2: torch.Tensor) -> None:
        call("b200_tp_absmax_put", self._p, ptr(x2), x2.stride(0), x2.shape[0], x2.shape[1], stream())

    def quant_wait(self, x2: torch.Tensor):
        codes = torch.empty(x2.shape, dtype=torch.int8, device=x2.device)
        absmax = torch.empty(x2.shape[0], dtype=torch.int32, device=x2.device)
        call("b200_tp_quant_wait", self._p, ptr(x2), x2.stride(0), x2.shape[0], x2.shape[1], ptr(codes), ptr(absmax), stream())
        return codes, absmax

    def absmax_quant(self, x2: torch.Tensor):
        """absmax_put + quant_wait in one launch (the ranks meet per token row)."""
        codes = torch.empty(x2.shape, dtype=torch.int8, device=x2.device)
        absmax = torch.empty(x2.shape[0], dtype=torch.int32, device=x2.device)
        call("b200_tp_absmax_quant", self._p, ptr(x2), x2.stride(0), x2.shape[0], x2.shape[1], ptr(codes), ptr(absmax), stream())
        return codes, absmax

    def gemm_add(self, codes: torch.Tensor, weight: torch.Tensor) -> None:
        m, k = codes.shape
        call("b200_gemm_w8a8_tp", self._p, ptr(codes), ptr(weight), m, weight.shape[0], k, stream())

    def requant_scatter(self, absmax: torch.Tensor, w_mul: torch.Tensor, w_shift) -> None:
        call("b200_tp_requant_scatter", self._p, ptr(absmax), ptr(w_mul), ptr(w_shift), absmax.shape[0], stream())

    def requant_direct(self, absmax: torch.Tensor, w_mul: torch.Tensor, w_shift) -> torch.Tensor:
        """One or two ranks: every rank has received all partial sums and finishes all rows itself."""
        m = absmax.shape[0]
        out = torch.empty((m, self.n), dtype=torch.int32, device=absmax.device)
        call("b200_tp_requant_direct", self._p, ptr(absmax), ptr(w_mul), ptr(w_shift), ptr(out), m, stream())
        return out

    @property
    def direct(self) -> bool:
        return self.size <= 2

    def collect(self, m: int, device) -> torch.Tensor:
        out = torch.empty((m, self.n), dtype=torch.int32, device=device)
        call("b200_tp_collect", self._p, ptr(out), m, stream())
        return out

    @staticmethod
    def _rows(x_q15_local: torch.Tensor) -> torch.Tensor:
        assert_q15(x_q15_local, "x_q15_local")
        require_cuda(x_q15_local)
        x2 = x_q15_local.reshape(-1, x_q15_local.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 4 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        return x2

    def fits(self, rows: int, n: int) -> bool:
        return 0 < rows <= min(256, self.m_max) and n == self.n

    def row_parallel_q15(self, method: W8A8Int8LinearMethod, layer, x_q15_local: torch.Tensor) -> torch.Tensor:
        """`row_parallel_q15` without a collective call: same bits."""
        if getattr(layer, "weight_mul", None) is None:
            method.process_weights_after_loading(layer)
        x2 = self._rows(x_q15_local)
        codes, absmax = self.absmax_quant(x2)
        self.gemm_add(codes, layer.weight)
        if self.direct:
            return self.requant_direct(absmax, layer.weight_mul, layer.weight_shift)
        self.requant_scatter(absmax, layer.weight_mul, layer.weight_shift)
        return self.collect(x2.shape[0], x2.device)

    # ---- the row-split linear fused with the add + RMSNorm + quant that follows it (row owners)
    def owner_norm(self, absmax: torch.Tensor, w_mul: torch.Tensor, w_shift, residual, norm_weight: torch.Tensor) -> None:
        call("b200_tp_owner_norm", self._p, ptr(absmax), ptr(w_mul), ptr(w_shift), ptr(residual), ptr(norm_weight),
             absmax.shape[0], stream())

    def collect_codes(self, m: int, device):
        codes = torch.empty((m, self.n), dtype=torch.int8, device=device)
        absmax = torch.empty(m, dtype=torch.int32, device=device)
        call("b200_tp_collect_codes", self._p, ptr(codes), ptr(absmax), m, stream())
        return codes, absmax

    def owner_rows(self, m: int) -> slice:
        """The token rows of an [m, n] matrix that this rank finishes (and whose residual it keeps)."""
        rpr = (m + self.size - 1) // self.size
        return slice(min(m, self.rank * rpr), min(m, (self.rank + 1) * rpr))

    def silu_absmax_quant(self, gate_up: torch.Tensor, fwht_block: int = 128):
        """SiLU(gate) * up -> blocked FWHT of this rank's columns -> absmax agreement -> int8 codes, one launch
        (silu_mul_fwht_q15 + absmax_quant).  Returns (codes int8 [rows, inter], agreed absmax int32 [rows])."""
        require_cuda(gate_up)
        if gate_up.dtype != torch.int32 or gate_up.ndim != 2:
            raise TypeError(f"gate_up must be int32 [tokens, 2*inter], got {gate_up.dtype} {tuple(gate_up.shape)}")
        g = gate_up.contiguous()
        rows, inter = g.shape[0], g.shape[1] // 2
        codes = torch.empty((rows, inter), dtype=torch.int8, device=g.device)
        absmax = torch.empty(rows, dtype=torch.int32, device=g.device)
        call("b200_tp_silu_absmax_quant", self._p, ptr(g), ptr(codes), ptr(absmax), rows, inter, int(fwht_block), stream())
        return codes, absmax

    def row_parallel_norm_quant(self, method: W8A8Int8LinearMethod, layer, x_q15_local: torch.Tensor,
                                residual: Optional[torch.Tensor], norm_weight: torch.Tensor, *, quantised=None):
        """Row-split linear -> (+ residual) -> RMSNorm -> per-token int8 quant without a collective call.

        ``residual`` int32 [rows, n] is updated in place for this rank's ``owner_rows`` only (the other rows go
        stale: their owners keep them).  Returns (codes int8 [rows, n], absmax int32 [rows]) of ALL rows: the bits of
        ``fused_add_rmsnorm_quant(row_parallel_q15(...), residual, norm_weight)`` computed on every rank.
        ``quantised``: the input already as (codes, agreed absmax) instead of ``x_q15_local``."""
        if getattr(layer, "weight_mul", None) is None:
            method.process_weights_after_loading(layer)
        if quantised is not None:            # (codes, agreed absmax) of the input, e.g. from silu_absmax_quant
            codes, absmax = quantised
            rows, dev = codes.shape[0], codes.device
        else:
            x2 = self._rows(x_q15_local)
            rows, dev = x2.shape[0], x2.device
            codes, absmax = self.absmax_quant(x2)
        if residual is not None and (residual.dtype != torch.int32 or not residual.is_contiguous()
                                     or tuple(residual.shape) != (rows, self.n)):
            raise ValueError("residual must be a contiguous int32 [rows, n] tensor (it is updated in place)")
        self.gemm_add(codes, layer.weight)
        self.owner_norm(absmax, layer.weight_mul, layer.weight_shift, residual, norm_weight.contiguous())
        return self.collect_codes(rows, dev)

    def all_gather(self, src: torch.Tensor) -> torch.Tensor:
        """int32 [words] from every rank -> int32 [size, words] (words <= 2 * m_max)."""
        require_cuda(src)
        s = src.reshape(-1).to(torch.int32).contiguous()
        out = torch.empty((self.size, s.numel()), dtype=torch.int32, device=s.device)
        call("b200_tp_all_gather", self._p, ptr(s), s.numel(), ptr(out), stream())
        return out

    @staticmethod
    def status(reset: bool = True) -> int:
        """0, or channel + 1 of the first wait that ran out since the last reset (synchronises)."""
        v = ctypes.c_int(0)
        call("b200_tp_status", ctypes.byref(v), int(reset))
        return int(v.value)

    @staticmethod
    def set_timeout_us(us: int) -> None:
        call("b200_tp_set_timeout_us", int(us))
