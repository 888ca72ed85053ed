"""int8 paged KV pool: the ``BaseKVCache`` interface of the reference over int8 pages.

Mirrors ``MHAKVCache`` (kvcache/mha_pool.py:11-72) behind the same methods
(``k_cache(i)``, ``v_cache(i)``, ``store_kv(k, v, out_loc, layer_id)``, ``device``,
``dtype``, ``num_layers``), but a page holds 16 tokens of int8 codes plus one
(multiplier, shift) per token and KV head:

    k_codes int8  [layers, pages, kv_heads, 16, 128]
    v_codes int8  [layers, pages, kv_heads, 2048]      (the page's 16 x 128 bytes in the operand
                                                        order of the integer MMA; see b200int.h)
    meta    int32 [layers, pages, kv_heads, 40]

A token location is ``page * 16 + offset`` (the reference's page table holds token
locations with page size 1, core.py:103; here they address 16-token pages).
"""
from __future__ import annotations

import torch

from .._lib import call, ptr, require_cuda, stream
from ..kvcache import BaseKVCache

PAGE_SIZE = 16
HEAD_DIM = 128
META_WORDS = 40


class Int8PagedKVCache(BaseKVCache):
    def __init__(self, num_kv_heads: int, num_layers: int, head_dim: int, num_pages: int,
                 device: torch.device | str | torch.dtype = "cuda", tp_size: int | torch.device | str | None = None) -> None:
        """``Int8PagedKVCache(num_kv_heads, num_layers, head_dim, num_pages, device, tp_size)``, or the argument order
        of the reference's pool, ``(num_kv_heads, num_layers, head_dim, num_pages, dtype, device)``
        (kvcache/mha_pool.py:17-25): the dtype must then be torch.int8 and the rank count comes from the
        process's tensor-parallel info, as there (:26-28).  ``num_pages`` counts 16-token pages."""
        if isinstance(device, torch.dtype):
            if device != torch.int8:
                raise TypeError(f"the int8 pool stores int8 codes, got dtype {device}")
            from ..distributed import try_get_tp_info
            info = try_get_tp_info()
            device, tp_size = tp_size if tp_size is not None else "cuda", (info.size if info is not None else 1)
        tp_size = 1 if tp_size is None else int(tp_size)
        if head_dim != HEAD_DIM:
            raise NotImplementedError(f"the int8 pool is built for head_dim {HEAD_DIM}, got {head_dim}")
        if num_kv_heads % tp_size != 0:
            raise ValueError(f"num_kv_heads={num_kv_heads} not divisible by tp_size={tp_size}")
        self._device = torch.device(device)
        if self._device.type != "cuda":
            raise RuntimeError("the int8 KV pool lives in GPU memory; there is no CPU fallback")
        self._num_layers = num_layers
        self.num_pages = num_pages
        self.kv_heads = num_kv_heads // tp_size
        shape = (num_layers, num_pages, self.kv_heads)
        self._k = torch.zeros(shape + (PAGE_SIZE, HEAD_DIM), dtype=torch.int8, device=self._device)
        self._v = torch.zeros(shape + (HEAD_DIM * PAGE_SIZE,), dtype=torch.int8, device=self._device)
        self._meta = torch.zeros(shape + (META_WORDS,), dtype=torch.int32, device=self._device)

    def k_cache(self, index: int) -> torch.Tensor:
        return self._k[index]

    def v_cache(self, index: int) -> torch.Tensor:
        return self._v[index]

    def meta(self, index: int) -> torch.Tensor:
        return self._meta[index]

    def store_kv(self, k: torch.Tensor, v: torch.Tensor, out_loc: torch.Tensor, layer_id: int) -> None:
        """Quantise Q15.16 K/V rows per token and KV head and scatter them to ``out_loc``.

        ``k``, ``v``: int32 [tokens, kv_heads*128] (column slices of a qkv buffer are fine).
        """
        if k.dtype != torch.int32 or v.dtype != torch.int32:
            raise TypeError(f"k and v must be int32 Q15.16, got {k.dtype} and {v.dtype}")
        require_cuda(k, v, out_loc)
        tokens = k.shape[0]
        k2 = k.reshape(tokens, -1)
        v2 = v.reshape(tokens, -1)
        if k2.stride(1) != 1 or k2.stride(0) % 4 or k2.data_ptr() % 16:
            k2 = k2.contiguous()
        if v2.stride(1) != 1 or v2.stride(0) % 4 or v2.data_ptr() % 16:
            v2 = v2.contiguous()
        loc = out_loc.to(torch.int32).contiguous()
        call("b200_kv_store_q15", ptr(k2), k2.stride(0), ptr(v2), v2.stride(0), ptr(loc),
             ptr(self._k[layer_id]), ptr(self._v[layer_id]), ptr(self._meta[layer_id]),
             tokens, self.kv_heads, self.num_pages, stream())

    def store_codes(self, k8, v8, k_mul, k_shift, v_mul, v_shift, out_loc, layer_id: int) -> None:
        """Scatter already-quantised tokens: codes int8 [tokens, kv_heads, 128], scales int32 [tokens, kv_heads]."""
        require_cuda(k8, v8, k_mul, k_shift, v_mul, v_shift, out_loc)
        tokens = k8.shape[0]
        c = lambda t, dt: t.to(dt).contiguous()
        loc = c(out_loc, torch.int32)
        call("b200_kv_store_codes", ptr(c(k8, torch.int8)), ptr(c(v8, torch.int8)), ptr(c(k_mul, torch.int32)),
             ptr(c(k_shift, torch.int32)), ptr(c(v_mul, torch.int32)), ptr(c(v_shift, torch.int32)), ptr(loc),
             ptr(self._k[layer_id]), ptr(self._v[layer_id]), ptr(self._meta[layer_id]),
             tokens, self.kv_heads, self.num_pages, stream())

    @property
    def device(self) -> torch.device:
        return self._device

    @property
    def dtype(self) -> torch.dtype:
        return torch.int8

    @property
    def num_layers(self) -> int:
        return self._num_layers
