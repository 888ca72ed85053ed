"""One integer-only decoder layer on the sm_100a kernels.

Follows the data flow of ``Qwen3DecoderLayerInteger.forward_q15`` (models/integer/qwen3_integer.py:62-80),
``RopeAttnInteger.forward_q15`` / ``AttentionLayerInteger.forward_q15`` (models/utils_integer.py:192-301) and
``GatedMLPInteger.forward_q15`` (models/utils_integer.py:99-121), with two differences that the integer
path makes possible: activations travel between a norm / activation and the following linear as int8 codes
(never as Q15.16 through HBM), and attention runs on int8 q/k/v against the int8 paged pool instead of the
reference's bf16 bridge (models/utils_integer.py:222-227).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from ..attention import Int8PagedKVCache, decode_attention_int8_paged, extend_attention_int8_paged, qkv_rope_quant_store
from ..kernel import fixed_point as fp
from ..kernel.pending import PENDING_MAX_ROWS, PendingLinear
from ..distributed import DistributedCommunicator
from .tp_linear import PeerReduceBuffers, TpExchange, row_parallel_q15, row_parallel_q15_fused
from .w8a8_int8 import W8A8Int8LinearMethod


_PENDING_ON = os.environ.get("B200_PENDING", "1") != "0"       # "0": every linear materialises its Q15.16 output
# "1": SiLU * up in the gate_up GEMM's epilogue at decode sizes.  Off by default: bit-identical, but measured slower on
# the 8B shape at batch 256 (the GEMM 33.5 + 6.2 -> 56.6 + 8.1 us for a row kernel that drops from 19.1 to 11.1 us:
# a CTA pair has 1.3 tiles, so the heavier epilogue is on its critical path instead of under the next tile's MMAs).
_GATE_UP_SILU_ON = os.environ.get("B200_GATE_UP_SILU", "0") == "1"


@dataclass
class AttnBatch:
    """What the reference keeps in ``Batch`` + attention metadata (core.py:72-97, attention/triton_int8.py:50-64)."""

    positions: torch.Tensor      # int32 [tokens]
    out_loc: torch.Tensor        # int32 [tokens]  token locations (page*16 + offset) of the new tokens
    page_table: torch.Tensor     # int32 [batch, pitch] page ids
    kv_lens: torch.Tensor        # int32 [batch]  keys per sequence including the new tokens
    q_lens: Optional[torch.Tensor]  # int32 [batch] new tokens per sequence; None = decode (one each)
    max_kv_len: int
    row_order: Optional[torch.Tensor] = None   # int32 [batch] rows by descending kv length (decode scheduling hint)


class _Linear(torch.nn.Module):
    """Holder of ``weight`` int8 [out, in] and ``weight_scale`` fp32 [out, 1] (or fixed-point scales directly)."""

    def __init__(self, weight: torch.Tensor, weight_scale: Optional[torch.Tensor] = None,
                 weight_mul: Optional[torch.Tensor] = None, weight_shift: Optional[torch.Tensor] = None):
        super().__init__()
        self.weight = weight
        if weight_scale is not None:
            self.weight_scale = weight_scale
        self.weight_mul, self.weight_shift = weight_mul, weight_shift


class Qwen3DecoderLayerInteger:
    def __init__(self, layer_id: int, num_qo_heads: int, num_kv_heads: int, hidden: int, inter: int,
                 weights: dict, cos_sin_cache_q15: torch.Tensor, pool: Int8PagedKVCache,
                 hadamard_block: int = 128, comm: Optional[DistributedCommunicator] = None,
                 peer_buffers: Optional[PeerReduceBuffers] = None, exchange: Optional[TpExchange] = None):
        """``weights``: qkv/o/gate_up/down -> _Linear; input_norm/post_norm int32 [hidden];
        q_norm/k_norm int32 [128] or None (Q15.16; q_norm already carries head_dim**-0.5).

        Under tensor parallelism (``comm`` with more than one rank) ``num_qo_heads``, ``num_kv_heads`` and
        ``inter`` are this rank's share, qkv / gate_up hold this rank's output channels (q | k | v and
        gate | up blocks of the local heads / columns), o / down this rank's input features, as the
        reference shards them (models/weight.py:12-52, layers/linear.py:73-160)."""
        self.comm = comm if comm is not None else DistributedCommunicator()
        self.layer_id, self.hq, self.hk, self.hidden, self.inter = layer_id, num_qo_heads, num_kv_heads, hidden, inter
        self.w = weights
        self.cache = cos_sin_cache_q15
        self.pool = pool
        self.hadamard_block = hadamard_block
        self.method = W8A8Int8LinearMethod()
        # tensor parallel: with peer buffers the o / down GEMMs add their partial sums into every rank's
        # accumulator themselves (decode sizes); without, an NCCL all-reduce follows the GEMM
        self.peer_buffers = peer_buffers
        # with an exchange block the absmax agreement and the ordering between the ranks run over peer memory too:
        # no collective call in the layer (decode sizes; larger batches fall back to NCCL)
        self.exchange = exchange

    def forward_codes(self, codes: torch.Tensor, absmax: torch.Tensor, residual: torch.Tensor, batch: AttnBatch,
                      next_norm_weight: torch.Tensor):
        """The layer between two norms, for tensor-parallel steps on an exchange block: takes the int8 codes and
        absmax of ITS input norm (all token rows) and returns those of the NEXT norm (``next_norm_weight``: the next
        layer's input_layernorm or the model's final norm).  Each row-split linear is finished, added to the
        residual, normalised and quantised by the rank that owns the token row (``exchange.owner_rows``);
        ``residual`` int32 [tokens, hidden] is updated in place for the own rows only.  Same bits as forward_q15
        followed by the next layer's fused add + RMSNorm + quant."""
        w, m, T = self.w, self.method, codes.shape[0]
        qkv = m.apply_pending(w["qkv"], codes, absmax) if T <= PENDING_MAX_ROWS and _PENDING_ON else m.apply_quantised(w["qkv"], codes, absmax)
        q8, q_mul, q_shift = qkv_rope_quant_store(batch.positions, qkv, self.hq, self.pool, self.layer_id, batch.out_loc,
                                                  self.cache, w.get("q_norm"), w.get("k_norm"))
        if batch.q_lens is None:
            attn = decode_attention_int8_paged(q8, q_mul, q_shift, self.pool, self.layer_id, batch.page_table,
                                               batch.kv_lens, batch.max_kv_len, row_order=batch.row_order)
        else:
            attn = extend_attention_int8_paged(q8, q_mul, q_shift, self.pool, self.layer_id, batch.page_table,
                                               batch.kv_lens, batch.q_lens, batch.max_kv_len)
        codes, absmax = self.exchange.row_parallel_norm_quant(m, w["o"], attn.view(T, self.hq * 128), residual, w["post_norm"])
        gate_up = m.apply_quantised(w["gate_up"], codes, absmax)
        if self.inter % 128 == 0 and T <= 256 and self.hadamard_block in (0, 128):
            # SiLU * up, rotation, the ranks' absmax agreement and the quantisation in one launch
            q = self.exchange.silu_absmax_quant(gate_up, self.hadamard_block)
            return self.exchange.row_parallel_norm_quant(m, w["down"], None, residual, next_norm_weight, quantised=q)
        act = fp.silu_mul_fwht_q15(gate_up, self.hadamard_block)
        return self.exchange.row_parallel_norm_quant(m, w["down"], act, residual, next_norm_weight)

    def forward_q15(self, x_q15, residual_q15: Optional[torch.Tensor], batch: AttnBatch,
                    trace: Optional[dict] = None, defer_down: bool = False):
        """Returns (x_out, residual_out), both Q15.16 int32 [tokens, hidden].

        At decode sizes on one GPU the qkv and o projections are left pending (kernel/pending.py) and finished by
        the kernels that read them; with ``defer_down`` the down projection is returned pending too, for the next
        layer's (or the final) add + RMSNorm + quant, and ``x_q15`` may be such a pending linear."""
        pending_in = isinstance(x_q15, PendingLinear)
        if not pending_in:
            fp.assert_q15(x_q15, "x_q15")
        t = trace if trace is not None else {}
        w, m = self.w, self.method
        T = x_q15.shape[0]
        tp = self.comm.size > 1 or (self.exchange is not None and self.exchange.size > 1)
        defer = trace is None and not tp and 0 < T <= PENDING_MAX_ROWS and _PENDING_ON
        # input_layernorm (+ residual add) -> int8 codes for qkv_proj
        codes, _, absmax, res, _ = fp.fused_add_rmsnorm_quant(x_q15, residual_q15, w["input_norm"])
        residual = res if residual_q15 is not None else x_q15
        t["ln1_codes"], t["ln1_absmax"] = codes, absmax
        qkv = m.apply_pending(w["qkv"], codes, absmax) if defer else m.apply_quantised(w["qkv"], codes, absmax)
        t["qkv"] = qkv
        qd, kd = self.hq * 128, self.hk * 128
        if trace is None:
            # one launch: q/k-norm, RoPE, rotation, K/V into the pool, q quantised
            q8, q_mul, q_shift = qkv_rope_quant_store(batch.positions, qkv, self.hq, self.pool, self.layer_id, batch.out_loc,
                                                      self.cache, w.get("q_norm"), w.get("k_norm"))
        else:
            # the same step by step, keeping the intermediates
            q, k, v = qkv[:, :qd].view(T, self.hq, 128), qkv[:, qd:qd + kd], qkv[:, qd + kd:]
            q, k = fp.qk_norm_rope_fwht(batch.positions, q, k, self.cache, w.get("q_norm"), w.get("k_norm"))
            t["q_rot"], t["k_rot"] = q, k
            self.pool.store_kv(k, v, batch.out_loc, self.layer_id)
            q8, _, q_absmax = fp.per_token_quant_int8_from_q15(q.reshape(T * self.hq, 128), return_absmax=True)
            q_mul, q_shift = fp.absmax_to_mul_shift(q_absmax)
            q8, q_mul, q_shift = q8.view(T, self.hq, 128), q_mul.view(T, self.hq), q_shift.view(T, self.hq)
        t["q8"] = q8
        if batch.q_lens is None:
            attn = decode_attention_int8_paged(q8, q_mul, q_shift, self.pool, self.layer_id, batch.page_table,
                                               batch.kv_lens, batch.max_kv_len, row_order=batch.row_order)
        else:
            attn = extend_attention_int8_paged(q8, q_mul, q_shift, self.pool, self.layer_id, batch.page_table,
                                               batch.kv_lens, batch.q_lens, batch.max_kv_len)
        t["attn"] = attn
        if self.exchange is not None and self.exchange.fits(T, self.hidden):
            rowp = lambda l, x: self.exchange.row_parallel_q15(m, l, x)
        elif self.peer_buffers is not None:
            rowp = lambda l, x: row_parallel_q15_fused(m, l, x, self.comm, self.peer_buffers)
        else:
            rowp = lambda l, x: row_parallel_q15(m, l, x, self.comm)
        if tp:
            o = rowp(w["o"], attn.view(T, qd))
        elif defer and getattr(w["o"], "input_scale", None) is None:
            a_codes, _, a_absmax = fp.per_token_quant_int8_from_q15(attn.view(T, qd), return_absmax=True)
            o = m.apply_pending(w["o"], a_codes, a_absmax)
        else:
            o = m.apply_weights_q15(w["o"], attn.view(T, qd))
        t["o"] = o
        # post_attention_layernorm (+ residual add) -> codes for gate_up_proj
        codes, _, absmax, residual, _ = fp.fused_add_rmsnorm_quant(o, residual, w["post_norm"])
        t["ln2_codes"], t["res2"] = codes, residual
        if defer and _GATE_UP_SILU_ON and self.hadamard_block in (0, 128) and m.can_fuse_gate_up_silu(w["gate_up"], T):
            # decode sizes on one GPU: SiLU(gate) * up in the gate_up GEMM's epilogue, then rotation + quant
            act = m.apply_gate_up_silu(w["gate_up"], codes, absmax)
            codes, _, absmax = fp.fwht_quant_q15(act, self.hadamard_block)
            down = (m.apply_pending if defer_down else m.apply_quantised)(w["down"], codes, absmax)
            return down, residual
        gate_up = m.apply_quantised(w["gate_up"], codes, absmax)
        t["gate_up"] = gate_up
        if tp:   # the token's absmax spans all ranks' columns: rotate locally, agree on the scale, then quantise
            down = rowp(w["down"], fp.silu_mul_fwht_q15(gate_up, self.hadamard_block))
        else:
            codes, _, absmax, _ = fp.silu_mul_fwht_quant(gate_up, self.hadamard_block)
            t["act_codes"], t["act_absmax"] = codes, absmax
            down = (m.apply_pending if defer and defer_down else m.apply_quantised)(w["down"], codes, absmax)
        t["down"] = down
        return down, residual
