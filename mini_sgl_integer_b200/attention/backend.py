"""Attention plug-in over the int8 paged pool: the ``BaseAttnBackend`` interface of the reference.

Same methods and call order as ``Int8Backend`` (attention/triton_int8.py:67-296, interface attention/base.py:18-35):
``prepare_metadata(batch)`` before a forward, ``forward(q, k, v, layer_id, batch)`` inside every layer,
``init_capture_graph / prepare_for_capture / prepare_for_replay`` around CUDA-graph decode
(engine/graph.py:49-158), ``batch.attn_metadata.get_last_indices(bs)`` for the lm_head.  Differences that the
integer path brings:

* q, k, v arrive as Q15.16 int32 (after q/k-norm, RoPE and the Hadamard rotation), not bf16; K and V are
  quantised per token and KV head on their way into the pool, q per token and head, and both prefill and
  decode run the integer kernel (the reference decodes in bf16, :155-176).
* The page table holds ids of 16-token pages, ``[max_requests, max_pages]`` int32; the kernels gather pages
  themselves, so there is no ``kv_indices`` list and no per-request ``torch.cat`` (:229-230): the metadata of a
  batch is one small pinned host array copied to the device plus a row gather of the table.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..kernel import fixed_point as fp
from .kv_pool import PAGE_SIZE, Int8PagedKVCache
from .ops import decode_attention_int8_paged, extend_attention_int8_paged, prefill_attention_int8_paged, qkv_rope_quant_store


class BaseAttnMetadata:
    """attention/base.py:12-15."""

    def get_last_indices(self, bs: int) -> torch.Tensor:
        raise NotImplementedError


class BaseAttnBackend:
    """The plug-in interface of the reference (attention/base.py:18-35)."""

    def forward(self, q, k, v, layer_id: int, batch) -> torch.Tensor:
        raise NotImplementedError

    def prepare_metadata(self, batch) -> None:
        raise NotImplementedError

    def init_capture_graph(self, max_seq_len: int, bs_list: List[int]) -> None:
        raise NotImplementedError

    def prepare_for_capture(self, batch) -> None:
        raise NotImplementedError

    def prepare_for_replay(self, batch) -> None:
        raise NotImplementedError


@dataclass
class Int8Metadata(BaseAttnMetadata):
    """What a forward needs besides q/k/v (the reference's Int8Metadata, attention/triton_int8.py:50-64)."""

    page_table: torch.Tensor          # int32 [bs, pitch] page ids of the batch's requests
    kv_lens: torch.Tensor             # int32 [bs] keys per request including the new tokens
    q_lens: Optional[torch.Tensor]    # int32 [bs] new tokens per request; None in decode
    qo_indptr: Optional[torch.Tensor]  # int32 [bs + 1] (prefill only)
    max_seqlen_q: int
    max_seqlen_k: int
    causal: bool = True
    row_order: Optional[torch.Tensor] = None   # int32 [bs] requests by descending kv length (decode only)

    def get_last_indices(self, bs: int) -> torch.Tensor:
        if self.qo_indptr is not None:
            return self.qo_indptr[1: 1 + bs] - 1
        return torch.arange(bs, device=self.kv_lens.device)


def token_locations(page_table_rows: torch.Tensor, positions: torch.Tensor, row_of_token: torch.Tensor) -> torch.Tensor:
    """KV slot of each new token: page_table[row, pos // 16] * 16 + pos % 16 (what the scheduler writes to
    ``batch.out_loc`` with 16-token pages)."""
    pos = positions.to(torch.int64)
    page = page_table_rows[row_of_token.to(torch.int64), pos // PAGE_SIZE].to(torch.int64)
    return (page * PAGE_SIZE + pos % PAGE_SIZE).to(torch.int32)


class B200Int8Backend(BaseAttnBackend):
    requires_q_scale_fusion = True     # read by the integer attention layer (models/utils_integer.py:198-208)

    def __init__(self, config, kvcache: Int8PagedKVCache, page_table: Optional[torch.Tensor] = None,
                 tp_size: Optional[int] = None) -> None:
        """``B200Int8Backend(config, kvcache)`` as the reference constructs its backends (attention/__init__.py:33-37,
        attention/triton_int8.py:74): ``config`` carries ``num_qo_heads``, ``num_kv_heads`` and ``head_dim`` (a
        ModelConfig), the rank count comes from the process's tensor-parallel info.

        ``page_table``: int32 [max_requests, max_pages] of PAGE ids (16-token pages); when omitted it is read from
        the global context at ``prepare_metadata`` time (the reference keeps its table there, engine/engine.py:66-73).
        Rows are addressed by ``req.table_idx``."""
        if tp_size is None:
            from ..distributed import try_get_tp_info
            info = try_get_tp_info()
            tp_size = info.size if info is not None else 1
        num_qo_heads, num_kv_heads = int(config.num_qo_heads), int(config.num_kv_heads)
        head_dim = int(getattr(config, "head_dim", 128))
        if num_qo_heads % tp_size or num_kv_heads % tp_size:
            raise ValueError("head counts must be divisible by tp_size")
        self.config = config
        self.kvcache = kvcache
        self.device = kvcache.device
        self._page_table = page_table
        self.qo_head_local = num_qo_heads // tp_size
        self.kv_head_local = num_kv_heads // tp_size
        self.head_dim = head_dim
        self.capture_bs: List[int] = []
        self.max_graph_bs = 0
        self.max_seq_len = 0
        self._cap_table: Optional[torch.Tensor] = None
        self._cap_kv_lens: Optional[torch.Tensor] = None
        self._cap_order: Optional[torch.Tensor] = None

    @classmethod
    def from_heads(cls, num_qo_heads: int, num_kv_heads: int, kvcache: Int8PagedKVCache, page_table: torch.Tensor,
                   tp_size: int = 1, head_dim: int = 128) -> "B200Int8Backend":
        """The same backend from bare head counts and an explicit page table."""
        from types import SimpleNamespace
        return cls(SimpleNamespace(num_qo_heads=num_qo_heads, num_kv_heads=num_kv_heads, head_dim=head_dim), kvcache,
                   page_table=page_table, tp_size=tp_size)

    @property
    def page_table(self) -> torch.Tensor:
        if self._page_table is not None:
            return self._page_table
        from ..core import get_global_ctx
        table = get_global_ctx().page_table
        if table is None:
            raise RuntimeError("no page table: pass one to the backend or set it on the global context")
        return table

    # ------------------------------------------------------------------ forward
    def forward_qkv_q15(self, qkv_q15: torch.Tensor, layer_id: int, batch, cos_sin_cache_q15: torch.Tensor,
                        q_norm_weight_q15: Optional[torch.Tensor], k_norm_weight_q15: Optional[torch.Tensor]) -> torch.Tensor:
        """The whole attention block on the qkv projection's Q15.16 output [T, (Hq + 2 Hk) * 128] in two launches:
        q/k-norm + RoPE + Hadamard rotation + KV store + q quantisation, then the attention kernel.  Same bits as
        the norms, ``rotary.forward_q15`` and ``forward`` one after the other."""
        md = batch.attn_metadata
        if not isinstance(md, Int8Metadata):
            raise TypeError("batch.attn_metadata was not prepared by this backend")
        tokens = qkv_q15.shape[0]
        q8, q_mul, q_shift = qkv_rope_quant_store(batch.positions, qkv_q15, self.qo_head_local, self.kvcache, layer_id,
                                                  batch.out_loc, cos_sin_cache_q15, q_norm_weight_q15, k_norm_weight_q15)
        if md.q_lens is None:
            out = decode_attention_int8_paged(q8, q_mul, q_shift, self.kvcache, layer_id, md.page_table, md.kv_lens,
                                              md.max_seqlen_k, row_order=md.row_order)
        else:
            out = prefill_attention_int8_paged(q8, q_mul, q_shift, self.kvcache, layer_id, md.page_table, md.kv_lens,
                                               md.q_lens, md.max_seqlen_k, md.max_seqlen_q,
                                               q_start=None if md.qo_indptr is None else md.qo_indptr[:-1])
        return out.view(tokens, self.qo_head_local * self.head_dim)

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, layer_id: int, batch) -> torch.Tensor:
        """q int32 [T, Hq*128] or [T, Hq, 128], k / v int32 [T, Hk*128] (Q15.16).  Returns Q15.16 [T, Hq*128]."""
        md = batch.attn_metadata
        if not isinstance(md, Int8Metadata):
            raise TypeError("batch.attn_metadata was not prepared by this backend")
        tokens = q.shape[0]
        self.kvcache.store_kv(k, v, batch.out_loc, layer_id)
        q8, _, q_absmax = fp.per_token_quant_int8_from_q15(q.reshape(tokens * self.qo_head_local, self.head_dim),
                                                           return_absmax=True)
        q_mul, q_shift = fp.absmax_to_mul_shift(q_absmax)
        q8 = q8.view(tokens, self.qo_head_local, self.head_dim)
        q_mul, q_shift = q_mul.view(tokens, -1), q_shift.view(tokens, -1)
        if md.q_lens is None:
            out = decode_attention_int8_paged(q8, q_mul, q_shift, self.kvcache, layer_id, md.page_table, md.kv_lens,
                                              md.max_seqlen_k, row_order=md.row_order)
        else:
            out = prefill_attention_int8_paged(q8, q_mul, q_shift, self.kvcache, layer_id, md.page_table, md.kv_lens,
                                               md.q_lens, md.max_seqlen_k, md.max_seqlen_q,
                                               q_start=None if md.qo_indptr is None else md.qo_indptr[:-1])
        return out.view(tokens, self.qo_head_local * self.head_dim)

    # ------------------------------------------------------------------ metadata
    def prepare_metadata(self, batch) -> None:
        """Build the batch's metadata from ``batch.padded_reqs`` (``table_idx``, ``cached_len``, ``device_len``)."""
        reqs = batch.padded_reqs
        lens = [r.device_len for r in reqs]
        order = sorted(range(len(reqs)), key=lambda i: -lens[i])
        host = torch.tensor([[r.table_idx for r in reqs], lens, [r.device_len - r.cached_len for r in reqs], order],
                            dtype=torch.int32)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        max_q, max_k = int(host[2].max()), int(host[1].max())
        table = self.page_table.index_select(0, dev[0].to(torch.int64))
        kv_lens = dev[1].contiguous()
        if batch.is_prefill:
            q_lens = dev[2].contiguous()
            qo_indptr = torch.zeros(len(reqs) + 1, dtype=torch.int32)
            qo_indptr[1:] = host[2].cumsum(0)
            qo_indptr = qo_indptr.to(self.device, non_blocking=True)
        else:
            q_lens, qo_indptr = None, None
        batch.attn_metadata = Int8Metadata(table, kv_lens, q_lens, qo_indptr, max_q, max_k,
                                           row_order=None if batch.is_prefill else dev[3].contiguous())

    # ------------------------------------------------------------------ CUDA graphs (decode only)
    def init_capture_graph(self, max_seq_len: int, bs_list: List[int]) -> None:
        if self._cap_table is not None:
            raise RuntimeError("capture buffers already initialised")
        self.max_seq_len = int(max_seq_len)
        self.capture_bs = sorted(bs_list)
        self.max_graph_bs = max(bs_list)
        pitch = (self.max_seq_len + PAGE_SIZE - 1) // PAGE_SIZE
        self._cap_table = torch.zeros((self.max_graph_bs, pitch), dtype=torch.int32, device=self.device)
        self._cap_kv_lens = torch.ones(self.max_graph_bs, dtype=torch.int32, device=self.device)
        self._cap_order = torch.arange(self.max_graph_bs, dtype=torch.int32, device=self.device)

    def prepare_for_capture(self, batch) -> None:
        bs = batch.size
        if bs not in self.capture_bs or self._cap_table is None:
            raise RuntimeError(f"batch size {bs} was not registered with init_capture_graph")
        if not batch.is_decode:
            raise RuntimeError("CUDA graph capture only supports decode")
        batch.attn_metadata = Int8Metadata(self._cap_table[:bs], self._cap_kv_lens[:bs], None, None, 1, self.max_seq_len,
                                           row_order=self._cap_order[:bs])

    def prepare_for_replay(self, batch) -> None:
        md = batch.attn_metadata
        bs = batch.padded_size
        if not isinstance(md, Int8Metadata) or self._cap_table is None or bs not in self.capture_bs:
            raise RuntimeError("prepare_metadata must run first, for a registered batch size")
        pitch = min(md.page_table.shape[1], self._cap_table.shape[1])
        self._cap_table[:bs, :pitch].copy_(md.page_table[:, :pitch])
        self._cap_kv_lens[:bs].copy_(md.kv_lens)
        if md.row_order is not None:
            self._cap_order[:bs].copy_(md.row_order)
