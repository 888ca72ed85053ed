"""numpy composition of one integer-only decoder layer (TEST INFRASTRUCTURE ONLY).

Same data flow as ``mini_sgl_integer_b200.layers.decoder_layer`` built from the oracle's ops; it follows
Qwen3DecoderLayerInteger.forward_q15 (models/integer/qwen3_integer.py:62-80) with int8 hand-offs between a
norm / activation and the next linear and integer attention on the int8 paged pool (parity unpinned as a
whole: the reference bridges attention through bf16).
"""
from __future__ import annotations

import numpy as np

from . import attention as oattn
from . import fixed_point as ofp
from . import linear as olin


def linear(codes, absmax, w8, w_mul, w_shift):
    x_mul, x_shift = oattn.absmax_to_mul_shift(absmax.reshape(-1))
    acc = olin.int32_accumulate(codes, w8)
    return olin.requant_q15(acc, x_mul, x_shift, w_mul, w_shift), acc


def decoder_layer(x, residual, w, cache, pool, positions, out_loc, tables, kv_lens, q_lens, hq, hk, block=128):
    t = {}
    T = x.shape[0]
    if residual is None:
        norm, res = ofp.rmsnorm_v2(x, w["input_norm"]), x
    else:
        norm, res = ofp.fused_add_rmsnorm_v2(residual, x, w["input_norm"])
    codes, _, absmax = ofp.per_token_quant_from_q15(norm)
    t["ln1_codes"], t["ln1_absmax"] = codes, absmax
    qkv, t["qkv_acc"] = linear(codes, absmax, *w["qkv"])
    t["qkv"] = qkv
    qd, kd = hq * 128, hk * 128
    q, k, v = qkv[:, :qd], qkv[:, qd:qd + kd], qkv[:, qd + kd:]
    if w.get("q_norm") is not None:
        q = ofp.rmsnorm_v2(np.ascontiguousarray(q), w["q_norm"])
    if w.get("k_norm") is not None:
        k = ofp.rmsnorm_v2(np.ascontiguousarray(k), w["k_norm"])
    q, k = ofp.rope_fwht_q15(positions, q.reshape(T, hq, 128), k.reshape(T, hk, 128), cache)
    t["q_rot"], t["k_rot"] = q, k.reshape(T, kd)
    pool.store_q15(out_loc, k.reshape(T, kd), v)
    q8, _, qm = ofp.per_token_quant_from_q15(q)
    q_mul, q_shift = oattn.absmax_to_mul_shift(qm[..., 0])
    t["q8"] = q8
    attn = oattn.paged_attention(q8, q_mul, q_shift, pool, tables, kv_lens, q_lens)
    t["attn"] = attn
    codes, _, absmax = ofp.per_token_quant_from_q15(attn.reshape(T, qd))
    o, t["o_acc"] = linear(codes, absmax, *w["o"])
    t["o"] = o
    norm, res = ofp.fused_add_rmsnorm_v2(res, o, w["post_norm"])
    codes, _, absmax = ofp.per_token_quant_from_q15(norm)
    t["ln2_codes"], t["res2"] = codes, res
    gate_up, t["gate_up_acc"] = linear(codes, absmax, *w["gate_up"])
    t["gate_up"] = gate_up
    act = ofp.blockwise_fwht_q15(ofp.silu_and_mul(gate_up), block)
    codes, _, absmax = ofp.per_token_quant_from_q15(act)
    t["act_codes"], t["act_absmax"] = codes, absmax
    down, t["down_acc"] = linear(codes, absmax, *w["down"])
    t["down"] = down
    return down, res, t
