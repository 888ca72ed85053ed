"""The two ends of the integer model as layer classes: ``VocabParallelEmbedding`` / ``ParallelLMHead`` of
``minisgl.layers.embedding`` (layers/embedding.py:14-110).

The embedding keeps the reference's bf16 table and returns the rows already converted with ``to_fixed`` (what
Qwen3ModelInteger.forward does right after it, models/integer/qwen3_integer.py:115-117).  The lm_head here is an
integer layer - int8 ``weight`` [vocab / tp, hidden] with ``weight_scale`` - because a bf16 matmul's summation
order is not reproducible; it returns Q15.16 logits.
"""
from __future__ import annotations

import torch

from ..core import get_global_ctx
from ..distributed import DistributedCommunicator, get_tp_info
from .base import BaseOP
from .w8a8_int8 import W8A8Int8LinearMethod


def _div_ceil(a: int, b: int) -> int:
    return (a + b - 1) // b


class VocabParallelEmbedding(BaseOP):
    def __init__(self, num_embeddings: int, embedding_dim: int):
        tp = get_tp_info()
        self.tp_size = tp.size
        self.num_embeddings = num_embeddings
        self.num_embeddings_tp = _div_ceil(num_embeddings, tp.size)
        start = self.num_embeddings_tp * tp.rank
        self.vocab_range = (start, min(start + self.num_embeddings_tp, num_embeddings) - start)
        self.weight = torch.empty(self.num_embeddings_tp, embedding_dim)
        self._comm = DistributedCommunicator()

    def forward_q15(self, input_ids: torch.Tensor) -> torch.Tensor:
        """to_fixed(embedding rows), Q15.16 int32 [tokens, hidden]; ids of other ranks' rows give zeros and the sum
        over ranks restores the row."""
        from ..models.qwen3_integer import embedding_to_fixed
        table = self.weight[: self.vocab_range[1]] if self.weight.shape[0] != self.vocab_range[1] else self.weight
        y = embedding_to_fixed(table, input_ids, self.vocab_range[0])
        return self._comm.all_reduce(y) if self.tp_size > 1 else y

    forward = forward_q15


class ParallelLMHead(BaseOP):
    """Integer lm_head: Q15.16 hidden states -> Q15.16 logits of this rank's vocabulary rows (all ranks' rows,
    gathered, when ``gather`` is set).  ``greedy`` merges the ranks' arg-max instead of gathering the logits."""

    def __init__(self, num_embeddings: int, embedding_dim: int, bias: bool = False, tie_word_embeddings: bool = False,
                 tied_embedding=None):
        if tie_word_embeddings or tied_embedding is not None:
            raise NotImplementedError("the integer lm_head has its own int8 weight; tied embeddings are not supported")
        tp = get_tp_info()
        self.tp_size, self.tp_rank = tp.size, tp.rank
        self.num_embeddings = num_embeddings
        self.num_embeddings_tp = _div_ceil(num_embeddings, tp.size)
        self.weight = torch.empty(self.num_embeddings_tp, embedding_dim)
        self.bias = torch.empty(self.num_embeddings_tp) if bias else None
        self._comm = DistributedCommunicator()
        self._method = W8A8Int8LinearMethod()

    def _last_tokens(self, x_q15: torch.Tensor) -> torch.Tensor:
        batch = get_global_ctx().batch
        if batch.is_prefill:
            idx = batch.attn_metadata.get_last_indices(batch.size)
            x_q15 = x_q15.index_select(0, idx.to(torch.int64))
        return x_q15

    def forward(self, x_q15: torch.Tensor) -> torch.Tensor:
        if self.weight.dtype != torch.int8 or not hasattr(self, "weight_scale"):
            raise TypeError("the integer lm_head needs an int8 `weight` and its `weight_scale`")
        logits = self._method.apply_weights_q15(self, self._last_tokens(x_q15), self.bias)
        if self.tp_size == 1:
            return logits
        gathered = self._comm.all_gather(logits.unsqueeze(0))                     # [tp, rows, vocab / tp]
        return gathered.movedim(0, 1).reshape(logits.shape[0], -1)[:, : self.num_embeddings]

    def greedy(self, x_q15: torch.Tensor) -> torch.Tensor:
        from ..models.qwen3_integer import argmax_int32, merge_sharded_argmax
        logits = self._method.apply_weights_q15(self, self._last_tokens(x_q15), self.bias)
        if self.tp_size == 1:
            return argmax_int32(logits)
        idx, val = argmax_int32(logits, index_offset=self.tp_rank * self.num_embeddings_tp, return_values=True)
        both = self._comm.all_gather(torch.stack((val, idx)).reshape(1, 2, -1))
        return merge_sharded_argmax(both[:, 0], both[:, 1])


__all__ = ["VocabParallelEmbedding", "ParallelLMHead"]
