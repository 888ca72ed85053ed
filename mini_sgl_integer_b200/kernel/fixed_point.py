"""Q15.16 fixed-point kernels: the API of ``minisgl.kernel.fixed_point`` on sm_100a CUDA.

Same names, argument meaning, result shapes and ``TypeError`` / ``ValueError`` behaviour as
the reference package (kernel/fixed_point/__init__.py:6-39); every function takes CUDA
tensors and returns new CUDA tensors.  The fused entry points at the bottom have no
single counterpart in the reference: each replaces a chain of its calls.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib
from .._lib import call, ptr, require_cuda, stream

FIXED_POINT_SCALE = 1 << 16
TRIG_Q15_SCALE = 1 << 15


def assert_q15(x: torch.Tensor, name: str = "tensor") -> None:
    """kernel/fixed_point/q15_tensor.py:12-14."""
    if x.dtype != torch.int32:
        raise TypeError(f"{name} must be torch.int32 (Q15.16), got {x.dtype}")


def to_fixed(x: torch.Tensor) -> torch.Tensor:
    """kernel/fixed_point/q15_tensor.py:17-22: int32(clamp(round(fp32(x) * 2**16)))."""
    require_cuda(x)
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.int32, device=x.device)
    if x.numel() == 0:
        return out
    if x.dtype == torch.bfloat16:
        call("b200_to_fixed_bf16", ptr(x), ptr(out), x.numel(), stream())
    else:
        if x.dtype != torch.float32:
            x = x.to(torch.float32)
        call("b200_to_fixed_f32", ptr(x), ptr(out), x.numel(), stream())
    return out


def from_fixed(x: torch.Tensor, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """kernel/fixed_point/q15_tensor.py:25-27: dtype(fp32(x) / 2**16)."""
    assert_q15(x, "x")
    require_cuda(x)
    x = x.contiguous()
    if x.numel() == 0:
        return torch.empty(x.shape, dtype=dtype, device=x.device)
    if dtype == torch.bfloat16:
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
        call("b200_from_fixed_bf16", ptr(x), ptr(out), x.numel(), stream())
        return out
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    call("b200_from_fixed_f32", ptr(x), ptr(out), x.numel(), stream())
    return out if dtype == torch.float32 else out.to(dtype)


@dataclass(frozen=True)
class Q15Tensor:
    """kernel/fixed_point/q15_tensor.py:30-50."""

    data: torch.Tensor

    def __post_init__(self) -> None:
        assert_q15(self.data, "Q15Tensor.data")

    @staticmethod
    def from_float(x: torch.Tensor) -> "Q15Tensor":
        return Q15Tensor(to_fixed(x))

    def to_float(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        return from_fixed(self.data, dtype=dtype)

    @property
    def shape(self) -> torch.Size:
        return self.data.shape

    @property
    def device(self) -> torch.device:
        return self.data.device


# ----------------------------------------------------------------------------- RMSNorm
def _norm_args(x: torch.Tensor, weight: torch.Tensor):
    if x.ndim < 2:
        raise ValueError(f"x must have at least 2 dims, got shape {tuple(x.shape)}")
    if weight.ndim != 1:
        raise ValueError(f"weight must be 1D, got shape {tuple(weight.shape)}")
    hidden = int(weight.shape[0])
    last = int(x.shape[-1])
    if last != hidden and last % hidden != 0:
        raise ValueError(
            f"x last dim={last} must equal hidden_dim={hidden} or be a multiple of hidden_dim"
        )
    return hidden


def rmsnorm_int_only_v2(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """kernel/fixed_point/rmsnorm_int_only_v2.py:319-390.

    ``x`` int32 [..., H] or [..., g*H] (each H-wide group normalised alone), ``weight`` int32 [H].
    ``eps`` is accepted and ignored, as in the reference (it uses the integer 1, :369).
    """
    assert x.dtype == torch.int32, f"Expected int32 input, got {x.dtype}"
    assert weight.dtype == torch.int32, f"Expected int32 weight, got {weight.dtype}"
    hidden = _norm_args(x, weight)
    require_cuda(x, weight)
    xc = x.contiguous()
    out = torch.empty_like(xc)
    if xc.numel() == 0:
        return out
    call("b200_rmsnorm_q15", ptr(xc), None, ptr(weight.contiguous()), None, ptr(out), None, None, None,
         xc.numel() // hidden, hidden, stream())
    return out


def fused_add_rmsnorm_int_only_v2(residual: torch.Tensor, x: torch.Tensor, weight: torch.Tensor,
                                  eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor]:
    """kernel/fixed_point/rmsnorm_int_only_v2.py:393-475: returns (normalised, residual + x)."""
    assert residual.dtype == torch.int32, f"Expected int32 residual, got {residual.dtype}"
    assert x.dtype == torch.int32, f"Expected int32 x, got {x.dtype}"
    assert weight.dtype == torch.int32, f"Expected int32 weight, got {weight.dtype}"
    if x.ndim < 2:
        raise ValueError(f"x must have at least 2 dims, got shape {tuple(x.shape)}")
    if residual.shape != x.shape:
        raise ValueError(
            f"residual and x must have same shape, got {tuple(residual.shape)} vs {tuple(x.shape)}"
        )
    hidden = _norm_args(x, weight)
    require_cuda(residual, x, weight)
    xc, rc = x.contiguous(), residual.contiguous()
    out, res_out = torch.empty_like(xc), torch.empty_like(rc)
    if xc.numel() == 0:
        return out, res_out
    call("b200_rmsnorm_q15", ptr(xc), ptr(rc), ptr(weight.contiguous()), ptr(res_out), ptr(out), None, None,
         None, xc.numel() // hidden, hidden, stream())
    return out, res_out


# ----------------------------------------------------------------------------- SiLU * up
def silu_and_mul_int_only(x: torch.Tensor) -> torch.Tensor:
    """kernel/fixed_point/silu_and_mul_int_only.py:233-275: x int32 [B, 2H] (gate || up) -> [B, H]."""
    assert x.dtype == torch.int32, f"Expected int32 input, got {x.dtype}"
    batch, two_hidden = x.shape
    hidden = two_hidden // 2
    require_cuda(x)
    xc = x.contiguous()
    out = torch.empty((batch, hidden), dtype=torch.int32, device=x.device)
    if out.numel() == 0:
        return out
    call("b200_silu_mul_q15", ptr(xc), ptr(out), None, None, None, batch, hidden, 0, stream())
    return out


# ----------------------------------------------------------------------------- FWHT
def fwht_int_q15(x_q15: torch.Tensor, *, normalize: bool = True) -> torch.Tensor:
    """kernel/fixed_point/fwht_int.py:99-147: Walsh-Hadamard over the last dim (power of two)."""
    if x_q15.dtype != torch.int32:
        raise TypeError(f"x_q15 must be int32 Q15.16, got {x_q15.dtype}")
    if x_q15.ndim < 2:
        raise ValueError(f"x_q15 must have at least 2 dims, got shape {tuple(x_q15.shape)}")
    head_dim = x_q15.shape[-1]
    if head_dim <= 0 or head_dim & (head_dim - 1):
        raise ValueError(f"head_dim must be power-of-two, got {head_dim}")
    require_cuda(x_q15)
    xc = x_q15.contiguous()
    out = torch.empty_like(xc)
    if head_dim == 1 or xc.numel() == 0:
        out.copy_(xc)  # a 1-point transform is the identity (scale round(2**15) >> 15 == 1)
        return out
    call("b200_fwht_q15", ptr(xc), ptr(out), xc.numel() // head_dim, head_dim, int(bool(normalize)), stream())
    return out


def apply_blockwise_fwht_q15(x_q15: torch.Tensor, block_size: int) -> torch.Tensor:
    """models/utils_integer.py:46-60: FWHT over consecutive ``block_size`` chunks of the last dim."""
    if x_q15.dtype != torch.int32:
        raise TypeError(f"x_q15 must be int32 Q15.16, got {x_q15.dtype}")
    if block_size <= 0:
        raise ValueError(f"block_size must be > 0, got {block_size}")
    hidden = x_q15.shape[-1]
    if hidden % block_size != 0:
        raise ValueError(f"Last dim {hidden} must be divisible by hadamard block_size {block_size}")
    x_blocks = x_q15.contiguous().view(-1, hidden // block_size, block_size)
    return fwht_int_q15(x_blocks, normalize=True).view_as(x_q15)


# ----------------------------------------------------------------------------- RoPE
def _as_3d(x: torch.Tensor, head_dim: int, name: str) -> tuple[torch.Tensor, bool]:
    """kernel/fixed_point/rope_int.py:63-80."""
    if x.dtype != torch.int32:
        raise TypeError(f"{name} must be int32 Q15.16, got {x.dtype}")
    if x.ndim == 3:
        if x.shape[-1] != head_dim:
            raise ValueError(f"{name} last dim must be head_dim={head_dim}, got {x.shape[-1]}")
        return x, False
    if x.ndim == 2:
        if x.shape[-1] % head_dim != 0:
            raise ValueError(f"{name} last dim must be divisible by head_dim={head_dim}, got {x.shape[-1]}")
        return x.view(x.shape[0], -1, head_dim), True
    raise ValueError(f"{name} must be 2D or 3D, got shape {tuple(x.shape)}")


def _rope_common(positions, query_q15, key_q15, cache, with_fwht: bool, q_norm_w=None, k_norm_w=None):
    if query_q15.dtype != torch.int32:
        raise TypeError(f"query_q15 must be int32 Q15.16, got {query_q15.dtype}")
    if key_q15.dtype != torch.int32:
        raise TypeError(f"key_q15 must be int32 Q15.16, got {key_q15.dtype}")
    if cache.dtype != torch.int32:
        raise TypeError(f"cos_sin_cache_q15 must be int32 Q1.15 cache, got {cache.dtype}")
    if query_q15.ndim not in (2, 3):
        raise ValueError(f"query_q15 must be 2D or 3D, got shape {tuple(query_q15.shape)}")
    if key_q15.ndim not in (2, 3):
        raise ValueError(f"key_q15 must be 2D or 3D, got shape {tuple(key_q15.shape)}")
    # head_dim inference follows kernel/fixed_point/rope_int.py:151-167
    head_dim = query_q15.shape[-1] if query_q15.ndim == 3 else key_q15.shape[-1]
    if query_q15.ndim == 2 and key_q15.ndim == 2:
        cands = [d for d in (64, 128, 256, 512)
                 if query_q15.shape[-1] % d == 0 and key_q15.shape[-1] % d == 0]
        if not cands:
            raise ValueError(
                "Cannot infer head_dim from 2D query/key shapes; expected common divisors in "
                f"[64, 128, 256, 512], got {query_q15.shape[-1]} and {key_q15.shape[-1]}"
            )
        if len(cands) > 1 and query_q15.shape[-1] not in cands:
            raise ValueError(
                "Ambiguous head_dim for 2D query/key inputs. Please pass 3D tensors with explicit "
                f"head_dim. Candidate head_dims: {cands}"
            )
        head_dim = query_q15.shape[-1] if query_q15.shape[-1] in cands else cands[0]
    if head_dim % 2 != 0:
        raise ValueError(f"head_dim must be even, got {head_dim}")
    q3, q_was_2d = _as_3d(query_q15, head_dim, "query_q15")
    k3, k_was_2d = _as_3d(key_q15, head_dim, "key_q15")
    if q3.shape[0] != k3.shape[0]:
        raise ValueError(f"query and key batch mismatch: {q3.shape[0]} vs {k3.shape[0]}")
    tokens = q3.shape[0]
    if positions.numel() != tokens:
        raise ValueError(f"positions size mismatch: expected {tokens}, got {positions.numel()}")
    if head_dim != 128:
        raise NotImplementedError(f"the sm_100a RoPE kernel is built for head_dim 128, got {head_dim}")
    require_cuda(q3, k3, cache)
    dev = q3.device
    positions = positions.to(device=dev, dtype=torch.int32).contiguous()
    cache = cache.to(dev).contiguous()
    # q and k may be column slices of one qkv buffer: pass the row pitch instead of copying
    def rows(t3):
        if t3.stride(-1) == 1 and t3.stride(1) == head_dim and t3.stride(0) % 2 == 0 and t3.data_ptr() % 8 == 0:
            return t3, t3.stride(0)
        t3 = t3.contiguous()
        return t3, t3.stride(0)
    q3, q_pitch = rows(q3)
    k3, k_pitch = rows(k3)
    q_out = torch.empty(q3.shape, dtype=torch.int32, device=dev)
    k_out = torch.empty(k3.shape, dtype=torch.int32, device=dev)
    call("b200_qk_rope_q15", ptr(positions), ptr(q3), q_pitch, ptr(k3), k_pitch, ptr(cache), cache.shape[0],
         ptr(q_norm_w), ptr(k_norm_w), ptr(q_out), ptr(k_out), tokens, q3.shape[1], k3.shape[1],
         int(with_fwht), stream())
    if q_was_2d:
        q_out = q_out.view(query_q15.shape)
    if k_was_2d:
        k_out = k_out.view(key_q15.shape)
    return q_out, k_out


def rope_int_q15(positions, query_q15, key_q15, cos_sin_cache_q15):
    """kernel/fixed_point/rope_int.py:128-247."""
    return _rope_common(positions, query_q15, key_q15, cos_sin_cache_q15, with_fwht=False)


def rope_fwht_int_q15(positions, query_q15, key_q15, cos_sin_cache_q15):
    """kernel/fixed_point/rope_fwht_int.py:9-23: RoPE, then FWHT over every q and k head."""
    return _rope_common(positions, query_q15, key_q15, cos_sin_cache_q15, with_fwht=True)


# ----------------------------------------------------------------------------- int8 quant
def per_token_quant_int8_from_q15(x_q15: torch.Tensor, return_absmax: bool = False):
    """layers/quantization/w8a8_int8.py:104-131: (int8 codes, fp32 scales [..., 1]).

    With ``return_absmax`` the integer row absmax (int32 [..., 1]) is returned as a third
    value; the fixed-point requant multiplier is derived from it.
    """
    assert_q15(x_q15, "x_q15")
    require_cuda(x_q15)
    xc = x_q15.contiguous()
    k = xc.shape[-1]
    rows = xc.numel() // k
    codes = torch.empty(xc.shape, dtype=torch.int8, device=xc.device)
    scale = torch.empty(xc.shape[:-1] + (1,), dtype=torch.float32, device=xc.device)
    absmax = torch.empty(xc.shape[:-1] + (1,), dtype=torch.int32, device=xc.device)
    if xc.numel() > 0:
        call("b200_per_token_quant_q15", ptr(xc), ptr(codes), ptr(scale), ptr(absmax), rows, k, stream())
    return (codes, scale, absmax) if return_absmax else (codes, scale)


def absmax_to_mul_shift(absmax: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(multiplier in [2**30, 2**31), shift) with multiplier / 2**shift ~= absmax / (127 * 65536)."""
    if absmax.dtype != torch.int32:
        raise TypeError(f"absmax must be int32, got {absmax.dtype}")
    require_cuda(absmax)
    a = absmax.contiguous()
    mul, shift = torch.empty_like(a), torch.empty_like(a)
    call("b200_absmax_to_mul_shift", ptr(a), ptr(mul), ptr(shift), a.numel(), stream())
    return mul, shift


# ----------------------------------------------------------------------------- fused chains
def fused_add_rmsnorm_quant(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor,
                            want_norm: bool = False):
    """(residual + x) -> fixed-point RMSNorm -> per-token int8 quant, one pass over the row.

    Replaces fused_add_rmsnorm_int_only_v2 followed by per_token_quant_int8_from_q15.
    Returns (codes int8, scale fp32 [..., 1], absmax int32 [..., 1], residual_out or None,
    normalised Q15.16 or None).
    """
    from .pending import PendingLinear
    if isinstance(x, PendingLinear):
        return _fused_add_rmsnorm_quant_pending(x, residual, weight, want_norm)
    assert_q15(x, "x")
    assert_q15(weight, "weight")
    hidden = _norm_args(x, weight)
    if int(x.shape[-1]) != hidden:
        raise ValueError("the fused quant needs rows of exactly the weight length")
    require_cuda(x, residual, weight)
    xc = x.contiguous()
    rc = res_out = None
    if residual is not None:
        assert_q15(residual, "residual")
        if residual.shape != x.shape:
            raise ValueError("residual and x must have same shape")
        rc = residual.contiguous()
        res_out = torch.empty_like(rc)
    rows = xc.numel() // hidden
    codes = torch.empty(xc.shape, dtype=torch.int8, device=xc.device)
    scale = torch.empty(xc.shape[:-1] + (1,), dtype=torch.float32, device=xc.device)
    absmax = torch.empty(xc.shape[:-1] + (1,), dtype=torch.int32, device=xc.device)
    norm = torch.empty_like(xc) if want_norm else None
    call("b200_rmsnorm_q15", ptr(xc), ptr(rc), ptr(weight.contiguous()), ptr(res_out), ptr(norm), ptr(codes),
         ptr(scale), ptr(absmax), rows, hidden, stream())
    return codes, scale, absmax, res_out, norm


def _fused_add_rmsnorm_quant_pending(x, residual: torch.Tensor | None, weight: torch.Tensor, want_norm: bool):
    """fused_add_rmsnorm_quant on a linear whose requantisation is still pending (kernel/pending.py): the kernel
    applies the linear's fixed-point epilogue while it loads the row and zeroes the accumulators behind it."""
    assert_q15(weight, "weight")
    rows, hidden = x.acc.shape
    if weight.ndim != 1 or weight.shape[0] != hidden:
        raise ValueError(f"weight must be [{hidden}], got {tuple(weight.shape)}")
    require_cuda(x.acc, residual, weight)
    rc = res_out = None
    if residual is not None:
        assert_q15(residual, "residual")
        if tuple(residual.shape) != (rows, hidden):
            raise ValueError("residual and x must have same shape")
        rc = residual.contiguous()
        res_out = torch.empty_like(rc)
    dev = x.acc.device
    codes = torch.empty((rows, hidden), dtype=torch.int8, device=dev)
    scale = torch.empty((rows, 1), dtype=torch.float32, device=dev)
    absmax = torch.empty((rows, 1), dtype=torch.int32, device=dev)
    norm = torch.empty((rows, hidden), dtype=torch.int32, device=dev) if want_norm else None
    call("b200_rmsnorm_q15_pending", ptr(x.acc), ptr(x.x_absmax), ptr(x.weight_mul), ptr(x.weight_shift), ptr(rc),
         ptr(weight.contiguous()), ptr(res_out), ptr(norm), ptr(codes), ptr(scale), ptr(absmax), rows, hidden, stream())
    return codes, scale, absmax, res_out, norm


def silu_mul_fwht_quant(gate_up: torch.Tensor, fwht_block: int = 128, want_q15: bool = False):
    """SiLU(gate) * up -> blocked FWHT -> per-token int8 quant, one pass over the row.

    Replaces silu_and_mul_int_only + apply_blockwise_fwht_q15 + per_token_quant_int8_from_q15.
    ``fwht_block`` 0 skips the rotation.  Returns (codes, scale [..., 1], absmax [..., 1], q15 or None).
    """
    assert_q15(gate_up, "gate_up")
    if gate_up.ndim != 2:
        raise ValueError(f"gate_up must be 2D [tokens, 2*inter], got shape {tuple(gate_up.shape)}")
    require_cuda(gate_up)
    g = gate_up.contiguous()
    rows, inter = g.shape[0], g.shape[1] // 2
    codes = torch.empty((rows, inter), dtype=torch.int8, device=g.device)
    scale = torch.empty((rows, 1), dtype=torch.float32, device=g.device)
    absmax = torch.empty((rows, 1), dtype=torch.int32, device=g.device)
    q15 = torch.empty((rows, inter), dtype=torch.int32, device=g.device) if want_q15 else None
    call("b200_silu_mul_q15", ptr(g), ptr(q15), ptr(codes), ptr(scale), ptr(absmax), rows, inter,
         int(fwht_block), stream())
    return codes, scale, absmax, q15


def fwht_quant_q15(act: torch.Tensor, fwht_block: int = 128):
    """Blocked FWHT -> per-token int8 quant of an activation that already is SiLU(gate) * up (the gate_up GEMM applied
    it in its epilogue): the second half of silu_mul_fwht_quant.  Returns (codes, scale [..., 1], absmax [..., 1])."""
    assert_q15(act, "act")
    if act.ndim != 2:
        raise ValueError(f"act must be 2D [tokens, inter], got shape {tuple(act.shape)}")
    require_cuda(act)
    a = act.contiguous()
    rows, inter = a.shape
    codes = torch.empty((rows, inter), dtype=torch.int8, device=a.device)
    scale = torch.empty((rows, 1), dtype=torch.float32, device=a.device)
    absmax = torch.empty((rows, 1), dtype=torch.int32, device=a.device)
    call("b200_fwht_quant_q15", ptr(a), ptr(codes), ptr(scale), ptr(absmax), rows, inter, int(fwht_block), stream())
    return codes, scale, absmax


def silu_mul_fwht_q15(gate_up: torch.Tensor, fwht_block: int = 128) -> torch.Tensor:
    """SiLU(gate) * up -> blocked FWHT, Q15.16 out (no quant): silu_and_mul_int_only + apply_blockwise_fwht_q15."""
    assert_q15(gate_up, "gate_up")
    if gate_up.ndim != 2:
        raise ValueError(f"gate_up must be 2D [tokens, 2*inter], got shape {tuple(gate_up.shape)}")
    require_cuda(gate_up)
    g = gate_up.contiguous()
    rows, inter = g.shape[0], g.shape[1] // 2
    out = torch.empty((rows, inter), dtype=torch.int32, device=g.device)
    if out.numel():
        call("b200_silu_mul_q15", ptr(g), ptr(out), None, None, None, rows, inter, int(fwht_block), stream())
    return out


def qk_norm_rope_fwht(positions, query_q15, key_q15, cos_sin_cache_q15, q_norm_weight, k_norm_weight):
    """Per-head RMSNorm of q and k, RoPE and FWHT in one kernel.

    Replaces q_norm.forward_q15 / k_norm.forward_q15 (models/utils_integer.py:214-218) followed by
    rotary.forward_q15 (layers/rotary_integer.py:70-149).  Norm weights are int32 [128] (Q15.16).
    """
    for w, n in ((q_norm_weight, "q_norm_weight"), (k_norm_weight, "k_norm_weight")):
        if w is not None:
            assert_q15(w, n)
            require_cuda(w)
    return _rope_common(positions, query_q15, key_q15, cos_sin_cache_q15, with_fwht=True,
                        q_norm_w=None if q_norm_weight is None else q_norm_weight.contiguous(),
                        k_norm_w=None if k_norm_weight is None else k_norm_weight.contiguous())


__all__ = [
    "FIXED_POINT_SCALE", "Q15Tensor", "assert_q15", "to_fixed", "from_fixed", "TRIG_Q15_SCALE",
    "rope_int_q15", "fwht_int_q15", "rope_fwht_int_q15", "rmsnorm_int_only_v2",
    "fused_add_rmsnorm_int_only_v2", "silu_and_mul_int_only", "apply_blockwise_fwht_q15",
    "per_token_quant_int8_from_q15", "absmax_to_mul_shift", "fused_add_rmsnorm_quant",
    "silu_mul_fwht_quant", "silu_mul_fwht_q15", "fwht_quant_q15", "qk_norm_rope_fwht",
]
