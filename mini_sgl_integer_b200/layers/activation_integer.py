"""``silu_and_mul_q15`` / ``silu_and_mul_fixed`` of ``minisgl.layers.activation_integer``
(layers/activation_integer.py:12-49) on the sm_100a kernel."""
from __future__ import annotations

from typing import Optional

import torch

from ..kernel import fixed_point as fp


def silu_and_mul_q15(x_q15: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """SiLU(gate) * up for x = gate || up, Q15.16 int32 in and out."""
    fp.assert_q15(x_q15, "x_q15")
    result = fp.silu_and_mul_int_only(x_q15)
    if out is not None:
        fp.assert_q15(out, "out")
        out.copy_(result)
        return out
    return result


def silu_and_mul_fixed(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The float bridge: to_fixed, the integer kernel, from_fixed in the input's dtype."""
    res = fp.from_fixed(silu_and_mul_q15(fp.to_fixed(x)), x.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


__all__ = ["silu_and_mul_q15", "silu_and_mul_fixed"]
