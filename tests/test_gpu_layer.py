"""One Qwen3-0.6B-shaped integer decoder layer on the CUDA kernels vs the oracle composition, bit-exact at
every hand-off (int8 codes, Q15.16 tensors, and the pool contents): hidden 1024, 16 q / 8 kv heads, head_dim 128,
intermediate 3072, 64 new tokens = 16 per sequence over cached prefixes so that the sequences reach
16 / 32 / 64 / 128 keys, page size 16, seed 0."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import layer as olayer

pytestmark = pytest.mark.gpu

HQ, HK, HID, INTER = 16, 8, 1024, 3072


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rope_cache(max_pos=256, base=1000000.0):
    inv = 1.0 / (base ** (torch.arange(0, 128, 2, dtype=torch.float) / 128))
    fr = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv)
    c = torch.cat((fr.cos(), fr.sin()), dim=-1)
    return torch.clamp(torch.round(c * 32768), -32768, 32767).to(torch.int32).numpy()


def make_weights(rng):
    def lin(n, k):
        return (rng.integers(-127, 128, (n, k), dtype=np.int8), rng.integers(2**29, 2**30, n).astype(np.int32),
                np.full(n, 31, dtype=np.int32))
    # multipliers in [2^29, 2^30) with shift 31 are scales in [0.25, 0.5): far larger than trained ones, so the
    # norm weights are kept small to hold the activations inside Q15.16
    return {
        "qkv": lin((HQ + 2 * HK) * 128, HID), "o": lin(HID, HQ * 128), "gate_up": lin(2 * INTER, HID), "down": lin(HID, INTER),
        "input_norm": rng.integers(2**5, 2**7, HID).astype(np.int32), "post_norm": rng.integers(2**5, 2**7, HID).astype(np.int32),
        "q_norm": rng.integers(2**11, 2**13, 128).astype(np.int32), "k_norm": rng.integers(2**12, 2**14, 128).astype(np.int32),
    }


def build(rng, kv_lens, q_lens, num_pages):
    B = len(kv_lens)
    prefix = [L - n for L, n in zip(kv_lens, q_lens)]
    perm = rng.permutation(num_pages)
    tables, off = [], 0
    for L in kv_lens:
        n = (L + 15) // 16
        tables.append(perm[off:off + n].astype(np.int32)); off += n
    loc = lambda b, a, e: np.concatenate([tables[b][i // 16] * 16 + (i % 16) for i in [np.arange(a, e)]]) if e > a else np.zeros(0, np.int64)
    ref_pool = oattn.PagedKV(num_pages, HK, 128)
    # cached prefix: random codes and scales
    pre = {}
    for b in range(B):
        p = prefix[b]
        if p:
            k8 = rng.integers(-127, 128, (p, HK, 128), dtype=np.int8); v8 = rng.integers(-127, 128, (p, HK, 128), dtype=np.int8)
            km = rng.integers(2**30, 2**31, (p, HK)); ks = rng.integers(33, 37, (p, HK))
            vm = rng.integers(2**30, 2**31, (p, HK)); vs = rng.integers(39, 43, (p, HK))
            l = loc(b, 0, p)
            ref_pool.store_codes(l, k8, v8, km, ks, vm, vs)
            pre[b] = (k8, v8, km.astype(np.int32), ks.astype(np.int32), vm.astype(np.int32), vs.astype(np.int32), l.astype(np.int32))
    positions = np.concatenate([np.arange(prefix[b], kv_lens[b]) for b in range(B)]).astype(np.int32)
    out_loc = np.concatenate([loc(b, prefix[b], kv_lens[b]) for b in range(B)]).astype(np.int32)
    pitch = max(len(t) for t in tables)
    table = np.zeros((B, pitch), dtype=np.int32)
    for b, t in enumerate(tables):
        table[b, : len(t)] = t
    return ref_pool, pre, tables, table, positions, out_loc


@pytest.mark.parametrize("mode", ["extend", "decode"])
def test_decoder_layer_bit_exact(mode):
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger, _Linear
    rng = np.random.default_rng(0)
    kv_lens = [16, 32, 64, 128]
    q_lens = [16, 16, 16, 16] if mode == "extend" else [1, 1, 1, 1]
    T = sum(q_lens)
    P = 32
    w = make_weights(rng)
    cache = rope_cache()
    ref_pool, pre, tables, table, positions, out_loc = build(rng, kv_lens, q_lens, P)
    x = np.clip(np.rint(rng.normal(0, 2**15, (T, HID))), -(2**23), 2**23).astype(np.int32)
    res = np.clip(np.rint(rng.normal(0, 2**15, (T, HID))), -(2**23), 2**23).astype(np.int32)

    want_x, want_res, wt = olayer.decoder_layer(x, res, w, cache, ref_pool, positions, out_loc, tables, kv_lens, q_lens, HQ, HK)

    pool = Int8PagedKVCache(HK, 2, 128, P, "cuda")
    for b, (k8, v8, km, ks, vm, vs, l) in pre.items():
        pool.store_codes(d(k8), d(v8), d(km), d(ks), d(vm), d(vs), d(l), 1)
    lin = lambda t: _Linear(d(t[0]), weight_mul=d(t[1]), weight_shift=d(t[2]))
    weights = {"qkv": lin(w["qkv"]), "o": lin(w["o"]), "gate_up": lin(w["gate_up"]), "down": lin(w["down"]),
               "input_norm": d(w["input_norm"]), "post_norm": d(w["post_norm"]), "q_norm": d(w["q_norm"]), "k_norm": d(w["k_norm"])}
    layer = Qwen3DecoderLayerInteger(1, HQ, HK, HID, INTER, weights, d(cache), pool)
    batch = AttnBatch(d(positions), d(out_loc), d(table), d(np.asarray(kv_lens, np.int32)),
                      d(np.asarray(q_lens, np.int32)) if mode == "extend" else None, 128)
    trace = {}
    got_x, got_res = layer.forward_q15(d(x), d(res), batch, trace)

    def same(name, got, want):
        g = got.cpu().numpy().reshape(want.shape)
        assert g.dtype == want.dtype, (name, g.dtype, want.dtype)
        if not np.array_equal(g, want):
            bad = np.argwhere(g != want)
            raise AssertionError(f"{name}: {len(bad)} of {g.size} differ, first {bad[0]}: {g[tuple(bad[0])]} vs {want[tuple(bad[0])]}")

    for name in ("ln1_codes", "qkv", "q_rot", "k_rot", "q8", "attn", "o", "ln2_codes", "res2", "gate_up", "act_codes", "down"):
        same(name, trace[name], wt[name])
    same("pool.k", pool.k_cache(1), ref_pool.k_codes); same("pool.v", pool.v_cache(1), ref_pool.v_codes)
    same("pool.meta", pool.meta(1), ref_pool.meta)
    same("x_out", got_x, want_x); same("residual_out", got_res, want_res)
    assert np.abs(want_x).max() > 0 and np.abs(wt["attn"]).max() > 0
    assert np.abs(want_x).max() < 2**31 - 1           # the case exercises the arithmetic, not the saturation rails
