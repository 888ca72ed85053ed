"""Integer rotary embedding: ``RotaryEmbeddingInteger`` / ``get_rope_integer`` of
``minisgl.layers.rotary_integer`` (layers/rotary_integer.py:13-212).  The cos | sin table is built in fp32 on the
host exactly as the reference builds it (:25-38) and rounded to Q1.15; ``forward_q15`` applies RoPE and then the
Hadamard rotation of every head (rope_fwht_int_q15)."""
from __future__ import annotations

import functools
import math
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from ..kernel import fixed_point as fp
from .base import StateLessOP

TRIG_Q15_SCALE = 1 << 15


class RotaryEmbeddingInteger(StateLessOP):
    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: float,
                 post_process: Optional[Callable[[torch.Tensor], torch.Tensor]] = None) -> None:
        if rotary_dim != head_size:
            raise ValueError(f"rotary_dim ({rotary_dim}) must equal head_size ({head_size})")
        if head_size != 128:
            raise NotImplementedError(f"the rotary kernels are built for head_size 128, got {head_size}")
        self.head_size = head_size
        inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float, device="cpu") / rotary_dim))
        if post_process is not None:
            inv_freq = post_process(inv_freq)
        freqs = torch.einsum("i,j -> ij", torch.arange(max_position_embeddings, dtype=torch.float, device="cpu"), inv_freq)
        self._cos_sin_cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1)
        self._cos_sin_cache_q15 = torch.clamp(torch.round(self._cos_sin_cache * TRIG_Q15_SCALE), -(1 << 15), (1 << 15) - 1).to(torch.int32)

    def cache_q15(self, device) -> torch.Tensor:
        if self._cos_sin_cache_q15.device != torch.device(device):
            self._cos_sin_cache_q15 = self._cos_sin_cache_q15.to(device)
        return self._cos_sin_cache_q15

    def forward_q15(self, positions: torch.Tensor, query_q15: torch.Tensor, key_q15: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """query [T, Hq*128] or [T, Hq, 128], key likewise, Q15.16 int32 -> (query [T, Hq, 128], key in its input
        rank), as the reference (:70-149)."""
        for name, t in (("query_q15", query_q15), ("key_q15", key_q15)):
            if t.dtype != torch.int32:
                raise TypeError(f"{name} must be int32 Q15.16, got {t.dtype}")
        batch = query_q15.shape[0]
        if key_q15.shape[0] != batch:
            raise ValueError(f"query/key batch mismatch: {batch} vs {key_q15.shape[0]}")

        def heads(t, name):
            if t.ndim == 2:
                if t.shape[1] % self.head_size:
                    raise ValueError(f"{name} last dim must be divisible by head_size={self.head_size}, got {t.shape[1]}")
                return t.reshape(batch, t.shape[1] // self.head_size, self.head_size)
            if t.ndim == 3:
                if t.shape[2] != self.head_size:
                    raise ValueError(f"{name} last dim must equal head_size={self.head_size}, got {t.shape[2]}")
                return t
            raise ValueError(f"{name} must be 2D or 3D, got shape {tuple(t.shape)}")
        q3, k3 = heads(query_q15, "query"), heads(key_q15, "key")
        q_out, k_out = fp.rope_fwht_int_q15(positions.to(q3.device), q3, k3, self.cache_q15(q3.device))
        if key_q15.ndim == 2:
            k_out = k_out.reshape(batch, -1)
        return q_out, k_out

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        q_out, k_out = self.forward_q15(positions, fp.to_fixed(query), fp.to_fixed(key))
        key.copy_(fp.from_fixed(k_out, key.dtype))
        return fp.from_fixed(q_out, query.dtype), key


def _llama3_post_process(scaling: Dict[str, Any]) -> Callable[[torch.Tensor], torch.Tensor]:
    """Frequency re-scaling of the "llama3" rope type (:152-187): long wavelengths are divided by ``factor``, short
    ones kept, with a linear blend between original_max_position / low_freq_factor and / high_freq_factor."""
    factor, low, high = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = int(scaling["original_max_position_embeddings"])

    def post_process(inv_freq: torch.Tensor) -> torch.Tensor:
        wave_len = 2 * math.pi / inv_freq
        if low == high:
            return torch.where(wave_len < original / high, inv_freq, inv_freq / factor)
        blend = torch.clamp((original / wave_len - low) / (high - low), 0, 1)
        return ((1 - blend) / factor + blend) * inv_freq
    return post_process


@functools.cache
def get_rope_integer(head_dim: int, rotary_dim: int, max_position: int, base: float,
                     rope_scaling: Optional[Tuple[Tuple[str, Any], ...]] = None) -> RotaryEmbeddingInteger:
    """One table per configuration (:195-212); ``rope_scaling`` as a tuple of items so that it can be a cache key."""
    if rope_scaling is None:
        return RotaryEmbeddingInteger(head_dim, rotary_dim, max_position, base)
    scaling = dict(rope_scaling)
    if scaling.get("rope_type") == "llama3":
        return RotaryEmbeddingInteger(head_dim, rotary_dim, max_position, base, _llama3_post_process(scaling))
    raise ValueError(f"Unsupported rope_scaling = {scaling}")


__all__ = ["get_rope_integer", "RotaryEmbeddingInteger"]
