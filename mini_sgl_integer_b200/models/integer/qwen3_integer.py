"""The integer Qwen3 model as layer classes with the reference's constructors, attribute names and state-dict keys:
``Qwen3DecoderLayerInteger(config, layer_id)``, ``Qwen3ModelInteger(config)``, ``Qwen3ForCausalLMInteger(config)``
of ``minisgl.models.integer.qwen3_integer`` (models/integer/qwen3_integer.py:43-143).

Build on any device, ``load_state_dict`` an int8 checkpoint (``weight`` int8 + ``weight_scale`` per linear, float
norm weights, bf16 embedding table), set the global context (page table, attention backend) and call
``forward()`` inside ``ctx.forward_batch(batch)`` as the reference's engine does (engine/engine.py:207-222).
The lm_head is the integer one of this package (int8 weight): ``forward`` returns Q15.16 logits and
``greedy_tokens`` the arg-max token ids.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ...core import get_global_ctx
from ...layers.base import BaseOP, OPList
from ...layers.embedding import ParallelLMHead, VocabParallelEmbedding
from ...layers.norm_integer import RMSNormFusedInteger
from ..utils_integer import GatedMLPInteger, RopeAttnInteger


class Qwen3DecoderLayerInteger(BaseOP):
    def __init__(self, config, layer_id: int):
        self.mlp = GatedMLPInteger(config, layer_id=layer_id)
        self.self_attn = RopeAttnInteger(config, layer_id, has_qk_norm=True)
        self.input_layernorm = RMSNormFusedInteger(size=config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNormFusedInteger(size=config.hidden_size, eps=config.rms_norm_eps)
        self._layer_id = layer_id

    def forward_q15(self, x_q15: torch.Tensor, residual_q15: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        if x_q15.dtype != torch.int32:
            raise TypeError(f"x_q15 must be int32 Q15.16, got {x_q15.dtype}")
        if residual_q15 is not None and residual_q15.dtype != torch.int32:
            raise TypeError(f"residual_q15 must be int32 Q15.16, got {residual_q15.dtype}")
        x_q15, residual_q15 = self.input_layernorm.forward_q15(x_q15, residual_q15)
        x_q15 = self.self_attn.forward_q15(x_q15)
        x_q15, residual_q15 = self.post_attention_layernorm.forward_q15(x_q15, residual_q15)
        return self.mlp.forward_q15(x_q15), residual_q15


class Qwen3ModelInteger(BaseOP):
    def __init__(self, config):
        self.embed_tokens = VocabParallelEmbedding(num_embeddings=config.vocab_size, embedding_dim=config.hidden_size)
        self.layers = OPList([Qwen3DecoderLayerInteger(config, i) for i in range(config.num_layers)])
        self.norm = RMSNormFusedInteger(size=config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Q15.16 hidden states after the final norm, int32 [tokens, hidden]."""
        x = self.embed_tokens.forward_q15(input_ids)
        residual = None
        for layer in self.layers.op_list:
            x, residual = layer.forward_q15(x, residual)
        x, _ = self.norm.forward_q15(x, residual)
        return x


class Qwen3ForCausalLMInteger(BaseOP):
    def __init__(self, config):
        self.model = Qwen3ModelInteger(config)
        self.lm_head = ParallelLMHead(num_embeddings=config.vocab_size, embedding_dim=config.hidden_size)

    def forward(self) -> torch.Tensor:
        """Q15.16 logits int32 [batch, vocab] of the batch in the global context."""
        return self.lm_head.forward(self.model.forward(get_global_ctx().batch.input_ids))

    def greedy_tokens(self) -> torch.Tensor:
        """Next token ids int32 [batch]: integer arg-max, the lowest index wins ties."""
        return self.lm_head.greedy(self.model.forward(get_global_ctx().batch.input_ids))


__all__ = ["Qwen3DecoderLayerInteger", "Qwen3ModelInteger", "Qwen3ForCausalLMInteger"]
