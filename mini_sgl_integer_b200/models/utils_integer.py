"""Attention and MLP blocks of the integer model as layer classes: ``GatedMLPInteger``, ``AttentionLayerInteger``,
``RopeAttnInteger`` and ``apply_blockwise_fwht_q15`` of ``minisgl.models.utils_integer``
(models/utils_integer.py:46-301), same constructors, attribute names (so the checkpoint keys match) and
``forward_q15`` signatures.

Differences that the integer path allows: attention receives Q15.16 q / k / v (no bf16 bridge, :222-227), and when
the active backend offers ``forward_qkv_q15`` (the backend of this package) everything between the qkv projection
and the attention kernel runs in one launch.  Float checkpoints are not handled here.
"""
from __future__ import annotations

import fnmatch
from typing import Optional

import torch

from ..core import get_global_ctx
from ..distributed import get_tp_info
from ..kernel import fixed_point as fp
from ..layers.activation_integer import silu_and_mul_q15
from ..layers.base import BaseOP, StateLessOP
from ..layers.linear import LinearColParallelMerged, LinearOProj, LinearQKVMerged, LinearRowParallel, div_even
from ..layers.norm_integer import RMSNormInteger
from ..layers.rotary_integer import get_rope_integer

apply_blockwise_fwht_q15 = fp.apply_blockwise_fwht_q15


def _hadamard_targets(layer_name: str, targets) -> bool:
    """A target names a layer exactly, by its last component ("down_proj"), or as a glob / "re:" pattern."""
    import re
    for t in targets:
        if t.startswith("re:"):
            if re.search(t[3:], layer_name):
                return True
        elif t == layer_name or layer_name.endswith("." + t) or fnmatch.fnmatch(layer_name, t):
            return True
    return False


class GatedMLPInteger(BaseOP):
    def __init__(self, config, layer_id: Optional[int] = None):
        self.gate_up_proj = LinearColParallelMerged(config.hidden_size, [config.intermediate_size, config.intermediate_size], has_bias=False)
        self.down_proj = LinearRowParallel(config.intermediate_size, config.hidden_size, has_bias=False)
        name = f"model.layers.{layer_id}.mlp.down_proj" if layer_id is not None else "mlp.down_proj"
        ht = getattr(config, "hadamard_transform", None)
        self._hadamard_block_size = int(getattr(ht, "block_size", 0) or 0)
        self._apply_hadamard = bool(ht is not None and ht.enabled and self._hadamard_block_size > 0 and _hadamard_targets(name, ht.targets))

    def forward_q15(self, x_q15: torch.Tensor) -> torch.Tensor:
        if x_q15.dtype != torch.int32:
            raise TypeError(f"x_q15 must be int32 Q15.16, got {x_q15.dtype}")
        gate_up = self.gate_up_proj.forward(x_q15)
        if self._apply_hadamard and self._hadamard_block_size == 128 and self.down_proj._tp_size == 1:
            # SiLU * up, the rotation and the per-token quant of down_proj in one pass over gate || up
            from ..layers.linear import _METHOD
            codes, _, absmax, _ = fp.silu_mul_fwht_quant(gate_up.reshape(-1, gate_up.shape[-1]), 128)
            self.down_proj._check(gate_up)
            return _METHOD.apply_quantised(self.down_proj, codes, absmax).reshape(*gate_up.shape[:-1], -1)
        y = silu_and_mul_q15(gate_up)
        if self._apply_hadamard:
            y = apply_blockwise_fwht_q15(y, self._hadamard_block_size)
        return self.down_proj.forward(y)

    forward = forward_q15


class AttentionLayerInteger(StateLessOP):
    attn_scale_fused: bool = False

    def __init__(self, layer_id: int, num_qo_heads: int, num_kv_heads: int, head_dim: int, rotary_config,
                 q_norm: Optional[BaseOP] = None, k_norm: Optional[BaseOP] = None):
        if num_qo_heads % num_kv_heads:
            raise ValueError("num_qo_heads must be a multiple of num_kv_heads")
        tp = get_tp_info().size
        self.layer_id, self.head_dim = layer_id, head_dim
        self.num_qo_heads, self.num_kv_heads = div_even(num_qo_heads, tp), div_even(num_kv_heads, tp)
        self.qo_attn_dim, self.kv_attn_dim = self.num_qo_heads * head_dim, self.num_kv_heads * head_dim
        self.rotary = get_rope_integer(head_dim=head_dim, rotary_dim=rotary_config.rotary_dim, max_position=rotary_config.max_position,
                                       base=rotary_config.base,
                                       rope_scaling=tuple(rotary_config.scaling.items()) if rotary_config.scaling else None)
        self.q_norm, self.k_norm = q_norm, k_norm
        self.attn_scale_fused = False

    def fuse_attn_scale_into_qnorm(self) -> None:
        """q_norm.weight *= head_dim ** -0.5, once, in the weight's own dtype (:171-183): the integer attention then
        needs no softmax scale."""
        if self.attn_scale_fused or self.q_norm is None:
            return
        self.q_norm.weight.data.mul_(self.head_dim ** -0.5)
        self.attn_scale_fused = True

    def forward_q15(self, qkv_q15: torch.Tensor) -> torch.Tensor:
        if qkv_q15.dtype != torch.int32:
            raise TypeError(f"qkv_q15 must be int32 Q15.16, got {qkv_q15.dtype}")
        ctx = get_global_ctx()
        backend = ctx.attn_backend
        if getattr(backend, "requires_q_scale_fusion", False) and not self.attn_scale_fused:
            self.fuse_attn_scale_into_qnorm()
        batch = ctx.batch
        if hasattr(backend, "forward_qkv_q15"):
            return backend.forward_qkv_q15(qkv_q15, self.layer_id, batch, self.rotary.cache_q15(qkv_q15.device),
                                           None if self.q_norm is None else self.q_norm.weight_q15(),
                                           None if self.k_norm is None else self.k_norm.weight_q15())
        q, k, v = qkv_q15.split([self.qo_attn_dim, self.kv_attn_dim, self.kv_attn_dim], dim=-1)
        if self.q_norm is not None:
            q = self.q_norm.forward_q15(q)
        if self.k_norm is not None:
            k = self.k_norm.forward_q15(k)
        q, k = self.rotary.forward_q15(batch.positions, q, k)
        return backend.forward(q, k, v, self.layer_id, batch).view(-1, self.qo_attn_dim)

    forward = forward_q15


class RopeAttnInteger(BaseOP):
    def __init__(self, config, layer_id: int, *, has_attn_bias: bool = False, has_qk_norm: bool = False):
        self.qkv_proj = LinearQKVMerged(hidden_size=config.hidden_size, head_dim=config.head_dim, num_qo_heads=config.num_qo_heads,
                                        num_kv_heads=config.num_kv_heads, has_bias=has_attn_bias)
        self.has_qk_norm = has_qk_norm
        self.q_norm = RMSNormInteger(config.head_dim, eps=config.rms_norm_eps) if has_qk_norm else None
        self.k_norm = RMSNormInteger(config.head_dim, eps=config.rms_norm_eps) if has_qk_norm else None
        self.attn = AttentionLayerInteger(layer_id=layer_id, head_dim=config.head_dim, num_qo_heads=config.num_qo_heads,
                                          num_kv_heads=config.num_kv_heads, rotary_config=config.rotary_config,
                                          q_norm=self.q_norm, k_norm=self.k_norm)
        self.o_proj = LinearOProj(config.head_dim * config.num_qo_heads, config.hidden_size, has_bias=False)

    def forward_q15(self, x_q15: torch.Tensor) -> torch.Tensor:
        if x_q15.dtype != torch.int32:
            raise TypeError(f"x_q15 must be int32 Q15.16, got {x_q15.dtype}")
        return self.o_proj.forward(self.attn.forward_q15(self.qkv_proj.forward(x_q15)))

    forward = forward_q15


__all__ = ["apply_blockwise_fwht_q15", "GatedMLPInteger", "AttentionLayerInteger", "RopeAttnInteger"]
