"""numpy composition of the integer-only model around oracle.layer (TEST INFRASTRUCTURE ONLY).

Embedding + to_fixed, the decoder layers, the final fused add + RMSNorm, an integer lm_head (int8 weights, exact
int32 accumulators, the fixed-point epilogue of oracle.linear) and an integer arg-max with the lowest index on
ties.  Follows Qwen3ModelInteger.forward / Qwen3ForCausalLMInteger.forward (models/integer/qwen3_integer.py:115-143)
up to the final norm; the integer lm_head and arg-max replace the reference's bf16 F.linear + float arg-max
(layers/embedding.py:98, engine/sample.py:74), whose summation order is not reproducible - parity unpinned there.
"""
from __future__ import annotations

import numpy as np

from . import fixed_point as ofp
from . import layer as olayer


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def embedding_to_fixed(table_bits: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """to_fixed(embedding(ids)) for a bf16 table given as its uint16 bit patterns [vocab, hidden]."""
    return ofp.to_fixed(bf16_bits_to_f32(table_bits[np.asarray(ids, dtype=np.int64)]))


def argmax_lowest(logits: np.ndarray) -> np.ndarray:
    return np.argmax(logits, axis=-1).astype(np.int32)          # numpy returns the first maximum


def model_forward(ids, w, cache, pools, positions, out_loc, tables, kv_lens, q_lens, hq, hk, block=128):
    """``w``: "embed" uint16 bits, "layers" list of oracle.layer weight dicts, "final_norm"; ``pools``: one
    oracle PagedKV per layer.  Returns (codes int8 [T, hidden], absmax int32 [T, 1])."""
    x = embedding_to_fixed(w["embed"], ids)
    residual = None
    for i, lw in enumerate(w["layers"]):
        x, residual, _ = olayer.decoder_layer(x, residual, lw, cache, pools[i], positions, out_loc, tables, kv_lens, q_lens, hq, hk, block)
    norm, _ = ofp.fused_add_rmsnorm_v2(residual, x, w["final_norm"])
    codes, _, absmax = ofp.per_token_quant_from_q15(norm)
    return codes, absmax


def logits_q15(codes, absmax, lm_head, rows=None):
    if rows is not None:
        codes, absmax = codes[rows], absmax[rows]
    out, _ = olayer.linear(codes, absmax, *lm_head)
    return out


def greedy(ids, w, cache, pools, positions, out_loc, tables, kv_lens, q_lens, hq, hk, last_rows, block=128):
    codes, absmax = model_forward(ids, w, cache, pools, positions, out_loc, tables, kv_lens, q_lens, hq, hk, block)
    logits = logits_q15(codes, absmax, w["lm_head"], last_rows)
    return argmax_lowest(logits), logits
