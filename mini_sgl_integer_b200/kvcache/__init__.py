"""KV pool interface: ``BaseKVCache`` of ``minisgl.kvcache.base`` (kvcache/base.py:10-38) and the int8 paged pool
that implements it (see attention/kv_pool.py)."""
from __future__ import annotations

from abc import ABC, abstractmethod

import torch


class BaseKVCache(ABC):
    @abstractmethod
    def k_cache(self, index: int) -> torch.Tensor: ...

    @abstractmethod
    def v_cache(self, index: int) -> torch.Tensor: ...

    @abstractmethod
    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer_id: int) -> None: ...

    @property
    @abstractmethod
    def device(self) -> torch.device: ...

    @property
    @abstractmethod
    def dtype(self) -> torch.dtype: ...

    @property
    @abstractmethod
    def num_layers(self) -> int: ...


def __getattr__(name):
    if name == "Int8PagedKVCache":
        from ..attention.kv_pool import Int8PagedKVCache
        return Int8PagedKVCache
    raise AttributeError(name)


__all__ = ["BaseKVCache", "Int8PagedKVCache"]
