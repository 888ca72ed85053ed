"""The integer model built from the reference-form classes (constructors from a ModelConfig, an int8 checkpoint
loaded with ``load_state_dict``, the backend created through the registry, the batch and page table in the global
context) must give the oracle's logits and greedy tokens: a prefill of ragged prompts, then decode steps."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import fixed_point as ofp
from oracle import linear as olin
from oracle import model as omodel

pytestmark = pytest.mark.gpu

L, HID, HQ, HK, INTER, VOCAB = 2, 256, 4, 2, 512, 1000


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _checkpoint(rng):
    """An int8 checkpoint under the reference's key names, and the same weights in the oracle's form."""
    sd, layers = {}, []

    def lin(key, n, k):
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        scale = (rng.uniform(0.25, 0.5, n) * 2.0 ** rng.integers(-3, 0, n)).astype(np.float32)
        sd[key + ".weight"] = d(w); sd[key + ".weight_scale"] = d(scale.reshape(n, 1))
        mul, sh = olin.weight_scale_to_mul_shift(scale)
        return (w, mul, sh)

    def norm(key, n, lo, hi, fuse=False):
        w = (rng.integers(lo, hi, n) / 65536.0).astype(np.float32)                 # to_fixed(w) is the integer drawn
        sd[key + ".weight"] = d(w)
        if fuse:                                                                   # q_norm absorbs head_dim ** -0.5 in fp32
            w = (w * np.float32(128 ** -0.5)).astype(np.float32)
        return ofp.to_fixed(w)
    for i in range(L):
        p = f"model.layers.{i}."
        layers.append({"qkv": lin(p + "self_attn.qkv_proj", (HQ + 2 * HK) * 128, HID), "o": lin(p + "self_attn.o_proj", HID, HQ * 128),
                       "gate_up": lin(p + "mlp.gate_up_proj", 2 * INTER, HID), "down": lin(p + "mlp.down_proj", HID, INTER),
                       "input_norm": norm(p + "input_layernorm", HID, 2**5, 2**7), "post_norm": norm(p + "post_attention_layernorm", HID, 2**5, 2**7),
                       "q_norm": norm(p + "self_attn.q_norm", 128, 2**14, 2**16, fuse=True), "k_norm": norm(p + "self_attn.k_norm", 128, 2**12, 2**14)})
        sd[p + "mlp.down_proj.R4_input.weight"] = torch.zeros(128, 128, device="cuda")   # compressed-tensors leftovers are dropped
    embed = (torch.randn((VOCAB, HID), generator=torch.Generator().manual_seed(3)) * 0.5).to(torch.bfloat16)
    sd["model.embed_tokens.weight"] = embed.cuda()
    final = norm("model.norm", HID, 2**5, 2**7)
    head = lin("lm_head", VOCAB, HID)
    host = {"embed": embed.view(torch.int16).numpy().view(np.uint16), "layers": layers, "final_norm": final, "lm_head": head}
    return sd, host


def test_reference_form_model_matches_oracle():
    from mini_sgl_integer_b200 import core
    from mini_sgl_integer_b200 import distributed as tpd
    from mini_sgl_integer_b200.attention import create_attention_backend
    from mini_sgl_integer_b200.attention.backend import token_locations
    from mini_sgl_integer_b200.kvcache import Int8PagedKVCache
    from mini_sgl_integer_b200.models.config import HadamardTransformConfig, ModelConfig, RotaryConfig
    from mini_sgl_integer_b200.models.integer import Qwen3ForCausalLMInteger
    tpd._reset_tp_info_for_tests()
    tpd.set_tp_info(0, 1)
    try:
        cfg = ModelConfig(L, HQ, HK, 128, HID, VOCAB, INTER, 1e-6, RotaryConfig(128, 128, 128, 1000000.0),
                          hadamard_transform=HadamardTransformConfig(True, 128, ("down_proj",)))
        rng = np.random.default_rng(12)
        sd, host = _checkpoint(rng)
        model = Qwen3ForCausalLMInteger(cfg)
        model.load_state_dict(sd)
        assert model.model.layers.op_list[0].mlp._apply_hadamard

        P, max_len = 16, 64
        prompt_lens = [5, 17, 32]
        B = len(prompt_lens)
        table = rng.permutation(P)[: B * (max_len // 16)].reshape(B, max_len // 16).astype(np.int32)
        pool = Int8PagedKVCache(HK, L, 128, P, torch.int8, "cuda")                  # the reference's argument order
        ctx = core.Context(page_size=16, page_table=d(table))
        core.set_global_ctx(ctx, replace=True)
        ctx.attn_backend = create_attention_backend("b200_int8", cfg, pool)
        cache = model.model.layers.op_list[0].self_attn.attn.rotary._cos_sin_cache_q15.cpu().numpy()

        ids = rng.integers(0, VOCAB, sum(prompt_lens)).astype(np.int32)
        pools = [oattn.PagedKV(P, HK, 128) for _ in range(L)]
        tables = [table[b] for b in range(B)]
        positions = np.concatenate([np.arange(n) for n in prompt_lens]).astype(np.int32)
        out_loc = np.concatenate([table[b][np.arange(n) // 16] * 16 + np.arange(n) % 16 for b, n in enumerate(prompt_lens)]).astype(np.int32)
        want_tok, want_logits = omodel.greedy(ids, host, cache, pools, positions, out_loc, tables, prompt_lens, prompt_lens, HQ, HK,
                                              np.cumsum(prompt_lens) - 1)

        def run(phase, reqs, input_ids):
            batch = core.Batch(reqs=reqs, phase=phase)
            batch.input_ids = d(input_ids)
            pos = np.concatenate([np.arange(r.cached_len, r.device_len) for r in reqs]).astype(np.int32)
            rows = np.concatenate([np.full(r.extend_len, i) for i, r in enumerate(reqs)])
            batch.positions = d(pos)
            batch.out_loc = token_locations(ctx.page_table[[r.table_idx for r in reqs]], batch.positions, d(rows))
            ctx.attn_backend.prepare_metadata(batch)
            with ctx.forward_batch(batch):
                logits = model.forward()
            with ctx.forward_batch(batch):                                         # the same step again: idempotent on the pool
                tokens = model.greedy_tokens()
            return logits.cpu().numpy(), tokens.cpu().numpy()

        reqs = [core.Req(b, 0, n) for b, n in enumerate(prompt_lens)]
        logits, tokens = run("prefill", reqs, ids)
        np.testing.assert_array_equal(logits, want_logits)
        np.testing.assert_array_equal(tokens, want_tok)
        lens = np.asarray(prompt_lens)
        for step in range(3):
            pos = lens.astype(np.int32)
            loc = np.asarray([table[b][pos[b] // 16] * 16 + pos[b] % 16 for b in range(B)], dtype=np.int32)
            lens = lens + 1
            want_tok2, want_logits2 = omodel.greedy(want_tok, host, cache, pools, pos, loc, tables, list(lens), [1] * B, HQ, HK, None)
            reqs = [core.Req(b, int(lens[b]) - 1, int(lens[b])) for b in range(B)]
            logits, tokens = run("decode", reqs, want_tok)
            np.testing.assert_array_equal(logits, want_logits2, err_msg=f"decode step {step}")
            np.testing.assert_array_equal(tokens, want_tok2)
            want_tok = want_tok2
        for i in range(L):
            np.testing.assert_array_equal(pool.k_cache(i).cpu().numpy(), pools[i].k_codes)
    finally:
        core.set_global_ctx(None)
        tpd._reset_tp_info_for_tests()
