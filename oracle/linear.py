"""numpy restatement of the W8A8 linear (TEST INFRASTRUCTURE ONLY).

The reference (layers/quantization/w8a8_int8.py:242-286) quantises the Q15.16
activation per token (pinned: ``fixed_point.per_token_quant_from_q15``), calls a
third-party int8 GEMM whose epilogue is float (``sgl_kernel.int8_scaled_mm``,
sgl_kernel >= 0.3.17.post1 per pyproject.toml:28, not vendored), and converts the
bf16 result back to Q15.16.  Only the int32 accumulators are exact across
implementations; the integer requant below is the build's definition (parity
unpinned) and follows the reference's multiplier/shift convention
(kernel/fixed_point/attention_prototype.py:100-118,
kernel/triton/int8_attention_kernels.py:278-285):

  acc[t,n]  = sum_k x8[t,k] * w8[n,k]                                   (int32, exact)
  cm[t,n]   = (x_mul[t] * w_mul[n]) >> 32
  out[t,n]  = sat32(mul_shift(acc[t,n], cm[t,n], x_shift[t] + w_shift[n] - 48))   (Q15.16)

where x_mul/x_shift = ``attention.absmax_to_mul_shift`` of the token's absmax and
(w_mul[n], w_shift[n]) is the fixed-point form of the checkpoint's fp32
``weight_scale[n]`` (``weight_scale_to_mul_shift``).
"""
from __future__ import annotations

import math

import numpy as np

from .attention import mul_shift
from .fixed_point import sat32


def int32_accumulate(x8: np.ndarray, w8: np.ndarray) -> np.ndarray:
    """x8 int8 [T, K], w8 int8 [N, K] -> int32 [T, N]; exact (|acc| <= K * 2**14)."""
    a = x8.astype(np.float64) @ w8.astype(np.float64).T
    return np.rint(a).astype(np.int64).astype(np.int32)


def weight_scale_to_mul_shift(scale: np.ndarray):
    """fp32_to_multiplier_shift (attention_prototype.py:100-112) applied per channel.

    e = floor(log2 v); shift = 30 - e; mul = min(round(v * 2**shift), 2**31 - 1).
    """
    s = np.asarray(scale, dtype=np.float64).reshape(-1)
    mul = np.empty(s.shape, dtype=np.int32)
    sh = np.empty(s.shape, dtype=np.int32)
    for i, v in enumerate(s):
        assert v > 0
        e = math.floor(math.log2(v + 1e-38))
        shift = 30 - e
        mul[i] = min(round(v * (2.0**shift)), (1 << 31) - 1)
        sh[i] = shift
    return mul, sh


def requant_q15(acc, x_mul, x_shift, w_mul, w_shift) -> np.ndarray:
    """The fixed-point epilogue defined in the module docstring. acc int32 [T, N]."""
    acc = np.asarray(acc, dtype=np.int64)
    cm = (np.asarray(x_mul, dtype=np.int64).reshape(-1, 1) * np.asarray(w_mul, dtype=np.int64).reshape(1, -1)) >> 32
    sh = np.asarray(x_shift, dtype=np.int64).reshape(-1, 1) + np.asarray(w_shift, dtype=np.int64).reshape(1, -1) - 48
    return sat32(mul_shift(acc, cm, sh))


def linear_q15_float_reference(x8, x_scale, w8, w_scale) -> np.ndarray:
    """The reference's fallback branch (w8a8_int8.py:280-284) in fp32, then to_fixed.

    Used only to show that the integer epilogue stays within the reference's own
    tolerance (cosine > 0.999, tests/kernel/test_q15_layer_flow.py:123-143).
    """
    from .fixed_point import to_fixed

    wf = w8.astype(np.float32) * np.asarray(w_scale, dtype=np.float32).reshape(-1, 1)
    xf = x8.astype(np.float32) * np.asarray(x_scale, dtype=np.float32).reshape(-1, 1)
    return to_fixed(xf @ wf.T)
