"""Integer RMSNorm layers: the classes of ``minisgl.layers.norm_integer`` (layers/norm_integer.py:17-83) on the
sm_100a kernels.  ``weight`` is the checkpoint's float tensor; its Q15.16 form is ``to_fixed(weight)`` as in the
reference (:29, :60), converted once per weight tensor instead of on every call."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ..kernel import fixed_point as fp
from .base import BaseOP


class _FixedWeight:
    """to_fixed(weight), recomputed only when the tensor is replaced (load_state_dict) or modified in place
    (fuse_attn_scale_into_qnorm multiplies q_norm.weight)."""

    def __init__(self):
        self._key, self._q15 = None, None

    def get(self, weight: torch.Tensor) -> torch.Tensor:
        key = (weight.data_ptr(), weight._version, weight.device, weight.dtype)
        if key != self._key:
            self._q15 = weight if weight.dtype == torch.int32 else fp.to_fixed(weight)
            self._key = key
        return self._q15


class RMSNormInteger(BaseOP):
    def __init__(self, size: int, eps: float) -> None:
        self.eps = eps
        self.weight = torch.empty(size)
        self._fixed = _FixedWeight()

    def weight_q15(self) -> torch.Tensor:
        return self._fixed.get(self.weight)

    def forward_q15(self, x_q15: torch.Tensor) -> torch.Tensor:
        fp.assert_q15(x_q15, "x_q15")
        return fp.rmsnorm_int_only_v2(x_q15, self.weight_q15(), self.eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return fp.from_fixed(self.forward_q15(fp.to_fixed(x)), x.dtype)


class RMSNormFusedInteger(BaseOP):
    def __init__(self, size: int, eps: float) -> None:
        self.eps = eps
        self.weight = torch.empty(size)
        self._fixed = _FixedWeight()

    def weight_q15(self) -> torch.Tensor:
        return self._fixed.get(self.weight)

    def forward_q15(self, x_q15: torch.Tensor, residual_q15: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        fp.assert_q15(x_q15, "x_q15")
        if residual_q15 is None:
            return fp.rmsnorm_int_only_v2(x_q15, self.weight_q15(), self.eps), x_q15
        fp.assert_q15(residual_q15, "residual_q15")
        return fp.fused_add_rmsnorm_int_only_v2(residual_q15, x_q15, self.weight_q15(), self.eps)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None):
        out, res = self.forward_q15(fp.to_fixed(x), None if residual is None else fp.to_fixed(residual))
        return fp.from_fixed(out, x.dtype), fp.from_fixed(res, x.dtype)


__all__ = ["RMSNormInteger", "RMSNormFusedInteger"]
