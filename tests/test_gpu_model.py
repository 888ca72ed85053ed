"""A small integer-only Qwen3-shaped model end to end on the CUDA kernels vs the oracle composition:
prefill of ragged prompts, then greedy decode steps whose bookkeeping runs on the device; token ids and
Q15.16 logits must be identical at every step, also when the step is replayed from a CUDA graph."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import model as omodel

pytestmark = pytest.mark.gpu

L, HID, HQ, HK, INTER, VOCAB = 2, 256, 4, 2, 512, 1000


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host_weights(w):
    """torch weights of random_weights -> the oracle's numpy form."""
    lin = lambda l: (l.weight.cpu().numpy(), l.weight_mul.cpu().numpy(), l.weight_shift.cpu().numpy())
    n = lambda t: None if t is None else t.cpu().numpy()
    layers = [{"qkv": lin(x["qkv"]), "o": lin(x["o"]), "gate_up": lin(x["gate_up"]), "down": lin(x["down"]),
               "input_norm": n(x["input_norm"]), "post_norm": n(x["post_norm"]), "q_norm": n(x["q_norm"]), "k_norm": n(x["k_norm"])}
              for x in w["layers"]]
    return {"embed": w["embed"].view(torch.int16).cpu().numpy().view(np.uint16), "layers": layers,
            "final_norm": n(w["final_norm"]), "lm_head": lin(w["lm_head"])}


def test_embedding_and_argmax_match_oracle():
    from mini_sgl_integer_b200.models import argmax_int32, embedding_to_fixed
    g = torch.Generator().manual_seed(3)
    table = (torch.randn((300, 64), generator=g) * 3).to(torch.bfloat16)
    table[5, 7] = 40000.0                                   # saturates the Q15.16 range
    ids = torch.tensor([0, 299, 5, 5, 17, 1000, -1], dtype=torch.int32)
    got = embedding_to_fixed(table.cuda(), ids.cuda()).cpu().numpy()
    bits = table.view(torch.int16).numpy().view(np.uint16)
    want = omodel.embedding_to_fixed(bits, np.clip(ids.numpy(), 0, 299))
    want[5:] = 0                                            # ids outside the table give zero rows
    np.testing.assert_array_equal(got, want)
    assert got[2, 7] == 2**31 - 1
    # shard starting at row 100: lower ids are someone else's
    got = embedding_to_fixed(table[100:].cuda(), ids.cuda(), vocab_start=100).cpu().numpy()
    assert not got[0].any() and not got[2].any()
    np.testing.assert_array_equal(got[1], want[1])

    rng = np.random.default_rng(4)
    logits = rng.integers(-2**31, 2**31, (9, 1003), dtype=np.int64).astype(np.int32)
    logits[0, :] = 7                                        # all equal: index 0
    logits[1, 500] = logits[1, 900] = 2**31 - 1             # tie: the lower index
    logits[2, :] = -2**31
    logits[2, 1002] = -2**31 + 1                            # maximum in the ragged tail
    buf = torch.zeros((9, 1004), dtype=torch.int32)
    buf[:, :1003] = torch.from_numpy(logits)
    idx, val = argmax_int32(buf.cuda()[:, :1003], return_values=True)
    np.testing.assert_array_equal(idx.cpu().numpy(), omodel.argmax_lowest(logits))
    np.testing.assert_array_equal(val.cpu().numpy(), logits.max(axis=1))
    assert argmax_int32(buf.cuda()[:, :1003], index_offset=5000).cpu().numpy()[1] == 5500


def test_decode_prepare_advances_on_device():
    from mini_sgl_integer_b200.models import DecodeBatch
    table = torch.tensor([[7, 3, 9, 0], [5, 1, 2, 4]], dtype=torch.int32).cuda()
    st = DecodeBatch(table, torch.tensor([15, 63], dtype=torch.int32).cuda(), 64)
    b = st.advance()
    assert b.positions.tolist() == [15, 63] and b.out_loc.tolist() == [7 * 16 + 15, 4 * 16 + 15] and b.kv_lens.tolist() == [16, 64]
    b = st.advance()                                        # sequence 1 is full: it stays on its last slot
    assert b.positions.tolist() == [16, 63] and b.out_loc.tolist() == [3 * 16, 4 * 16 + 15] and b.kv_lens.tolist() == [17, 64]


@pytest.mark.parametrize("use_graph", [False, True])
def test_prefill_then_greedy_decode_matches_oracle(use_graph):
    _prefill_then_decode(use_graph, (L, HID, HQ, HK, INTER, VOCAB), [5, 17, 32], 4, wide=False)


def test_prefill_then_greedy_decode_8b_shaped_layers():
    """Two layers of the Qwen3-8B shape (hidden 4096, 32 q / 8 kv heads, intermediate 12288) under a small vocabulary:
    prefill of three short prompts and two greedy decode steps, token ids, logits and pools against the oracle."""
    _prefill_then_decode(False, (2, 4096, 32, 8, 12288, 2048), [3, 9, 5], 2, wide=True)


def _prefill_then_decode(use_graph, shape, prompt_lens, steps, wide):
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch
    from mini_sgl_integer_b200.models import DecodeBatch, Qwen3ForCausalLMInteger, Qwen3IntegerConfig, random_weights, rope_cache_q15
    L, HID, HQ, HK, INTER, VOCAB = shape
    cfg = Qwen3IntegerConfig(L, HID, HQ, HK, INTER, VOCAB, max_pos=128)
    w = random_weights(cfg, seed=11)
    if wide:       # channel shifts that keep the activations of a hidden size of several thousand inside Q15.16
        for lw in w["layers"]:
            lw["qkv"].weight_shift += 1; lw["o"].weight_shift += 1
            lw["gate_up"].weight_shift += 2; lw["down"].weight_shift += 2
    hw = host_weights(w)
    rng = np.random.default_rng(5)
    P, max_len = 16, 64
    B = len(prompt_lens)
    perm = rng.permutation(P)
    pitch = max_len // 16
    table = perm[: B * pitch].reshape(B, pitch).astype(np.int32)
    tables = [table[b] for b in range(B)]
    ids = rng.integers(0, VOCAB, sum(prompt_lens)).astype(np.int32)
    positions = np.concatenate([np.arange(n) for n in prompt_lens]).astype(np.int32)
    out_loc = np.concatenate([table[b][np.arange(n) // 16] * 16 + np.arange(n) % 16 for b, n in enumerate(prompt_lens)]).astype(np.int32)
    last_rows = np.cumsum(prompt_lens) - 1
    cache = rope_cache_q15(cfg.max_pos).numpy()

    # ---- oracle: prefill, then `steps` decode steps
    pools = [oattn.PagedKV(P, HK, 128) for _ in range(L)]
    want_tokens, want_logits = [], []
    tok, lg = omodel.greedy(ids, hw, cache, pools, positions, out_loc, tables, prompt_lens, prompt_lens, HQ, HK, last_rows)
    want_tokens.append(tok); want_logits.append(lg)
    lens = np.asarray(prompt_lens)
    for _ in range(steps):
        pos = lens.astype(np.int32)
        loc = np.asarray([table[b][pos[b] // 16] * 16 + pos[b] % 16 for b in range(B)], dtype=np.int32)
        lens = lens + 1
        tok, lg = omodel.greedy(tok, hw, cache, pools, pos, loc, tables, list(lens), [1] * B, HQ, HK, None)
        want_tokens.append(tok); want_logits.append(lg)

    # ---- CUDA
    pool = Int8PagedKVCache(HK, L, 128, P, "cuda")
    lm = Qwen3ForCausalLMInteger(cfg, w, pool)
    pre = AttnBatch(d(positions), d(out_loc), d(table), d(np.asarray(prompt_lens, np.int32)), d(np.asarray(prompt_lens, np.int32)), max_len)
    logits = lm.forward(d(ids), pre, d(last_rows.astype(np.int32)))
    np.testing.assert_array_equal(logits.cpu().numpy(), want_logits[0])
    from mini_sgl_integer_b200.models import argmax_int32
    tokens = argmax_int32(logits)
    np.testing.assert_array_equal(tokens.cpu().numpy(), want_tokens[0])

    state = DecodeBatch(d(table), d(np.asarray(prompt_lens, np.int32)), max_len)
    cur = tokens.clone()
    out_logits = torch.empty((B, VOCAB), dtype=torch.int32, device="cuda")

    def step():
        lg_ = lm.forward(cur, state.advance())
        out_logits.copy_(lg_)
        cur.copy_(argmax_int32(lg_))

    if use_graph:
        # warm-up outside the capture on a scratch copy of the state, then restore it
        snap = (state.seq_lens.clone(), cur.clone(), [pool.k_cache(i).clone() for i in range(L)],
                [pool.v_cache(i).clone() for i in range(L)], [pool.meta(i).clone() for i in range(L)])
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            step()
        torch.cuda.current_stream().wait_stream(s)
        state.seq_lens.copy_(snap[0]); cur.copy_(snap[1])
        for i in range(L):
            pool.k_cache(i).copy_(snap[2][i]); pool.v_cache(i).copy_(snap[3][i]); pool.meta(i).copy_(snap[4][i])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        state.seq_lens.copy_(snap[0]); cur.copy_(snap[1])
        for i in range(L):
            pool.k_cache(i).copy_(snap[2][i]); pool.v_cache(i).copy_(snap[3][i]); pool.meta(i).copy_(snap[4][i])
    for i in range(steps):
        graph.replay() if use_graph else step()
        np.testing.assert_array_equal(out_logits.cpu().numpy(), want_logits[i + 1], err_msg=f"logits of step {i}")
        np.testing.assert_array_equal(cur.cpu().numpy(), want_tokens[i + 1], err_msg=f"tokens of step {i}")
    for i in range(L):
        np.testing.assert_array_equal(pool.k_cache(i).cpu().numpy(), pools[i].k_codes)
        np.testing.assert_array_equal(pool.meta(i).cpu().numpy(), pools[i].meta)
    assert 0 < np.abs(want_logits[-1]).max() < 2**31 - 1          # the case exercises the arithmetic, not the rails
