"""W8A8 int8 linear with Q15.16 input/output: the interface of
``minisgl.layers.quantization.w8a8_int8`` (layers/quantization/w8a8_int8.py) on sm_100a.

The reference quantises the Q15.16 activation per token with fp32 arithmetic, calls a
third-party int8 GEMM with a float epilogue and converts the bf16 result back to Q15.16
(:242-286).  Here the per-token quant keeps the reference's bit-exact codes, the GEMM runs
on the tcgen05 tensor cores with exact int32 accumulators, and the epilogue is fixed-point:

    out = sat32(mul_shift(acc, (x_mul * w_mul) >> 32, x_shift + w_shift - 48))

with (x_mul, x_shift) derived from the token's integer absmax and (w_mul, w_shift) from the
checkpoint's fp32 ``weight_scale`` per output channel (fp32_to_multiplier_shift of
kernel/fixed_point/attention_prototype.py:100-112).
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import torch

from .._lib import call, ptr, require_cuda, stream
from ..kernel.fixed_point import absmax_to_mul_shift, assert_q15, per_token_quant_int8_from_q15
from ..kernel.pending import PENDING_MAX_ROWS, PendingLinear, zero_workspace

__all__ = ["W8A8Int8LinearMethod", "int8_gemm_q15", "weight_scale_to_mul_shift", "per_token_quant_int8_from_q15",
           "per_tensor_quant_int8_static_from_q15"]


def per_tensor_quant_int8_static_from_q15(x_q15: torch.Tensor, input_scale: torch.Tensor | float) -> torch.Tensor:
    """int8 codes of a Q15.16 tensor under a checkpoint-provided per-tensor ``input_scale``: what
    per_tensor_quant_int8_static gives on from_fixed(x) (layers/quantization/w8a8_int8.py:75-92, :251-254);
    a multi-element scale is reduced to its maximum like the reference (:82-83)."""
    assert_q15(x_q15, "x_q15")
    require_cuda(x_q15)
    scale = float(input_scale.max()) if isinstance(input_scale, torch.Tensor) else float(input_scale)
    if not scale > 0:
        raise ValueError(f"input_scale must be positive, got {scale}")
    x = x_q15.contiguous()
    if x.numel() % 4:
        raise ValueError("the number of elements must be a multiple of 4")
    codes = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    if x.numel():
        call("b200_static_quant_q15", ptr(x), scale, ptr(codes), x.numel(), stream())
    return codes


def weight_scale_to_mul_shift(weight_scale: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-channel fp32 scale -> (multiplier in [2**30, 2**31), shift), both int32 [N], on the scale's device.

    Follows fp32_to_multiplier_shift (attention_prototype.py:100-112) in double precision on the host:
    e = floor(log2 v); shift = 30 - e; multiplier = min(round(v * 2**shift), 2**31 - 1).
    """
    s = weight_scale.detach().reshape(-1).to("cpu", torch.float64).tolist()
    mul, sh = [], []
    for v in s:
        if not v > 0:
            raise ValueError(f"weight_scale must be positive, got {v}")
        e = math.floor(math.log2(v + 1e-38))
        shift = 30 - e
        mul.append(min(round(v * (2.0 ** shift)), (1 << 31) - 1))
        sh.append(shift)
    dev = weight_scale.device
    return (torch.tensor(mul, dtype=torch.int32, device=dev), torch.tensor(sh, dtype=torch.int32, device=dev))


def int8_gemm_q15(x8: torch.Tensor, x_mul: Optional[torch.Tensor], x_shift: Optional[torch.Tensor], w8: torch.Tensor,
                  w_mul: torch.Tensor, w_shift: Optional[torch.Tensor] = None, *, want_q15: bool = True,
                  want_acc: bool = False, x_absmax: Optional[torch.Tensor] = None):
    """x8 int8 [M, K] @ w8 int8 [N, K]^T with the fixed-point epilogue.

    The per-token scale is (x_mul, x_shift), or ``x_absmax`` int32 [M] from which the kernel derives them
    (same values as absmax_to_mul_shift).  Returns the Q15.16 result int32 [M, N], the exact int32
    accumulators, or both (q15, acc).
    """
    if x8.dtype != torch.int8 or w8.dtype != torch.int8:
        raise TypeError(f"x8 and w8 must be int8, got {x8.dtype} and {w8.dtype}")
    if x8.ndim != 2 or w8.ndim != 2 or x8.shape[1] != w8.shape[1]:
        raise ValueError(f"shape mismatch: x8 {tuple(x8.shape)} vs w8 {tuple(w8.shape)}")
    require_cuda(x8, w8, x_mul, x_shift, w_mul, w_shift, x_absmax)
    m, k = x8.shape
    n = w8.shape[0]
    x8, w8 = x8.contiguous(), w8.contiguous()
    c = lambda t: None if t is None else t.reshape(-1).to(torch.int32).contiguous()
    x_mul, x_shift, w_mul, w_shift = c(x_mul), c(x_shift), c(w_mul), c(w_shift)
    out = torch.empty((m, n), dtype=torch.int32, device=x8.device) if want_q15 else None
    acc = torch.empty((m, n), dtype=torch.int32, device=x8.device) if want_acc else None
    if m > 0 and x_absmax is not None:
        call("b200_gemm_w8a8_absmax", ptr(x8), ptr(w8), ptr(c(x_absmax)), ptr(w_mul), ptr(w_shift), ptr(out), ptr(acc),
             m, n, k, stream())
    elif m > 0:
        call("b200_gemm_w8a8", ptr(x8), ptr(w8), ptr(x_mul), ptr(x_shift), ptr(w_mul), ptr(w_shift), ptr(out),
             ptr(acc), m, n, k, stream())
    if want_q15 and want_acc:
        return out, acc
    return out if want_q15 else acc


class W8A8Int8LinearMethod:
    """Same role and method names as the reference class (layers/quantization/w8a8_int8.py:134-286)."""

    def create_weights(self, layer: torch.nn.Module, output_partition_sizes: list[int],
                       input_size_per_partition: int, params_dtype: torch.dtype, weight_loader: Callable):
        """int8 ``weight`` [out, in] and fp32 ``weight_scale`` [out, 1] (:145-180)."""
        out = sum(output_partition_sizes)
        layer.logical_widths = output_partition_sizes
        layer.register_parameter("weight", torch.nn.Parameter(
            torch.empty(out, input_size_per_partition, dtype=torch.int8), requires_grad=False))
        layer.register_parameter("weight_scale", torch.nn.Parameter(
            torch.empty((out, 1), dtype=torch.float32), requires_grad=False))

    def process_weights_after_loading(self, layer) -> None:
        """Derive the fixed-point channel scales once (the reference does nothing here, :182-188)."""
        layer.weight_mul, layer.weight_shift = weight_scale_to_mul_shift(layer.weight_scale)

    def apply_weights_q15(self, layer, x_q15: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Q15.16 int32 [..., K] -> Q15.16 int32 [..., N] (:242-286)."""
        assert_q15(x_q15, "x_q15")
        if getattr(layer, "weight_mul", None) is None:
            self.process_weights_after_loading(layer)
        lead = x_q15.shape[:-1]
        x2 = x_q15.reshape(-1, x_q15.shape[-1])
        static = getattr(layer, "input_scale", None)
        if isinstance(static, torch.Tensor) and static.numel() > 0:
            # static per-tensor activation scale (:95-101, :251-254): same codes as the reference, and the
            # scale enters the fixed-point epilogue as one (multiplier, shift) for every token
            if getattr(layer, "input_mul", None) is None:
                layer.input_mul, layer.input_shift = weight_scale_to_mul_shift(static.max().reshape(1).to(torch.float32))
            codes = per_tensor_quant_int8_static_from_q15(x2, static)
            rows = x2.shape[0]
            out = int8_gemm_q15(codes, layer.input_mul.expand(rows), layer.input_shift.expand(rows), layer.weight,
                                layer.weight_mul, layer.weight_shift)
            if bias is not None:
                out = self._add_bias(out, bias)
            return out.reshape(*lead, -1)
        codes, _scale, absmax = per_token_quant_int8_from_q15(x2, return_absmax=True)
        return self.apply_quantised(layer, codes, absmax, bias).reshape(*lead, -1)

    def apply_quantised(self, layer, codes: torch.Tensor, absmax: torch.Tensor,
                        bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The GEMM half of apply_weights_q15 for activations already quantised by a fused row kernel."""
        if getattr(layer, "weight_mul", None) is None:
            self.process_weights_after_loading(layer)
        x8 = codes.reshape(-1, codes.shape[-1])
        m, n = x8.shape[0], layer.weight.shape[0]
        if 0 < m <= PENDING_MAX_ROWS and x8.is_contiguous() and layer.weight.is_contiguous() and layer.weight_shift is not None:
            # decode sizes: split-K parts go into a workspace that is kept zero, which saves the clearing launch
            out = torch.empty((m, n), dtype=torch.int32, device=x8.device)
            require_cuda(x8, layer.weight, absmax, layer.weight_mul, layer.weight_shift)
            call("b200_gemm_w8a8_absmax_ws", ptr(x8), ptr(layer.weight), ptr(absmax.reshape(-1).to(torch.int32).contiguous()), ptr(layer.weight_mul),
                 ptr(layer.weight_shift), ptr(out), ptr(zero_workspace(x8.device, m, n)), m, n, x8.shape[1], stream())
        else:
            out = int8_gemm_q15(x8, None, None, layer.weight, layer.weight_mul, layer.weight_shift, x_absmax=absmax.reshape(-1))
        if bias is not None:
            out = self._add_bias(out, bias)
        return out

    @staticmethod
    def can_fuse_gate_up_silu(layer, rows: int) -> bool:
        """Whether ``apply_gate_up_silu`` takes this merged gate_up layer and batch: decode sizes, 128 activation
        channels per CTA pair, per-channel shifts present."""
        w = layer.weight
        return (0 < rows <= PENDING_MAX_ROWS and w.shape[0] % 256 == 0 and w.shape[1] % 16 == 0 and w.is_contiguous()
                and getattr(layer, "weight_shift", None) is not None and getattr(layer, "input_scale", None) is None)

    def apply_gate_up_silu(self, layer, codes: torch.Tensor, absmax: torch.Tensor) -> torch.Tensor:
        """The merged gate_up projection with SiLU(gate) * up applied in the GEMM's epilogue: int8 codes [rows, k] ->
        Q15.16 int32 [rows, inter], the bits of silu_and_mul_q15(apply_quantised(layer, codes, absmax))."""
        if getattr(layer, "weight_mul", None) is None:
            self.process_weights_after_loading(layer)
        x8 = codes.reshape(-1, codes.shape[-1]).contiguous()
        require_cuda(x8, layer.weight, absmax, layer.weight_mul, layer.weight_shift)
        m, n2 = x8.shape[0], layer.weight.shape[0]
        out = torch.empty((m, n2 // 2), dtype=torch.int32, device=x8.device)
        if m:
            call("b200_gemm_gate_up_silu", ptr(x8), ptr(layer.weight), ptr(absmax.reshape(-1).to(torch.int32).contiguous()),
                 ptr(layer.weight_mul), ptr(layer.weight_shift), ptr(out), ptr(zero_workspace(x8.device, m, n2)), m, n2,
                 x8.shape[1], stream())
        return out

    def apply_pending(self, layer, codes: torch.Tensor, absmax: torch.Tensor) -> PendingLinear:
        """apply_quantised without the requantisation: the exact accumulators stay in a zero workspace and the next
        row kernel (fused_add_rmsnorm_quant, qkv_rope_quant_store) finishes the linear while it loads them."""
        if getattr(layer, "weight_mul", None) is None:
            self.process_weights_after_loading(layer)
        x8 = codes.reshape(-1, codes.shape[-1]).contiguous()
        require_cuda(x8, layer.weight, absmax, layer.weight_mul, layer.weight_shift)
        m, n = x8.shape[0], layer.weight.shape[0]
        ws = zero_workspace(x8.device, m, n)
        if m:
            call("b200_gemm_w8a8_acc_ws", ptr(x8), ptr(layer.weight.contiguous()), ptr(ws), m, n, x8.shape[1], stream())
        return PendingLinear(ws, absmax.reshape(-1).to(torch.int32).contiguous(), layer.weight_mul, layer.weight_shift)

    @staticmethod
    def _add_bias(out: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
        b = bias if bias.dtype == torch.int32 else torch.clamp(
            torch.round(bias.to(torch.float32) * 65536.0), -(2 ** 31), 2 ** 31 - 1).to(torch.int32)
        return torch.clamp(out.to(torch.int64) + b.to(torch.int64), -(2 ** 31), 2 ** 31 - 1).to(torch.int32)
