"""Shared builders for the decoder-layer tests: seeded weights, the Q1.15 rotary table and a paged pool with a
cached prefix, on the host (oracle layout).  Shapes default to the Qwen3-0.6B-shaped layer."""
from __future__ import annotations

import numpy as np
import torch

from oracle import attention as oattn

HQ, HK, HID, INTER = 16, 8, 1024, 3072


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rope_cache(max_pos=256, base=1000000.0):
    inv = 1.0 / (base ** (torch.arange(0, 128, 2, dtype=torch.float) / 128))
    fr = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv)
    c = torch.cat((fr.cos(), fr.sin()), dim=-1)
    return torch.clamp(torch.round(c * 32768), -32768, 32767).to(torch.int32).numpy()


def make_weights(rng, hq=HQ, hk=HK, hid=HID, inter=INTER, wide=False):
    """``wide``: channel shifts of 32 (qkv, o) and 33 (gate_up, down) instead of 31, which keeps the activations of
    layers with a hidden size of several thousand inside Q15.16."""
    def lin(n, k, extra=0):
        return (rng.integers(-127, 128, (n, k), dtype=np.int8), rng.integers(2**29, 2**30, n).astype(np.int32),
                np.full(n, 31 + (extra if wide else 0), dtype=np.int32))
    # multipliers in [2^29, 2^30) with shift 31 are scales in [0.25, 0.5): far larger than trained ones, so the
    # norm weights are kept small to hold the activations inside Q15.16
    return {
        "qkv": lin((hq + 2 * hk) * 128, hid, 1), "o": lin(hid, hq * 128, 1), "gate_up": lin(2 * inter, hid, 2),
        "down": lin(hid, inter, 2),
        "input_norm": rng.integers(2**5, 2**7, hid).astype(np.int32), "post_norm": rng.integers(2**5, 2**7, hid).astype(np.int32),
        "q_norm": rng.integers(2**11, 2**13, 128).astype(np.int32), "k_norm": rng.integers(2**12, 2**14, 128).astype(np.int32),
    }


def build(rng, kv_lens, q_lens, num_pages, hk=HK):
    B = len(kv_lens)
    prefix = [L - n for L, n in zip(kv_lens, q_lens)]
    perm = rng.permutation(num_pages)
    tables, off = [], 0
    for L in kv_lens:
        n = (L + 15) // 16
        tables.append(perm[off:off + n].astype(np.int32)); off += n
    loc = lambda b, a, e: np.concatenate([tables[b][i // 16] * 16 + (i % 16) for i in [np.arange(a, e)]]) if e > a else np.zeros(0, np.int64)
    ref_pool = oattn.PagedKV(num_pages, hk, 128)
    # cached prefix: random codes and scales
    pre = {}
    for b in range(B):
        p = prefix[b]
        if p:
            k8 = rng.integers(-127, 128, (p, hk, 128), dtype=np.int8); v8 = rng.integers(-127, 128, (p, hk, 128), dtype=np.int8)
            km = rng.integers(2**30, 2**31, (p, hk)); ks = rng.integers(33, 37, (p, hk))
            vm = rng.integers(2**30, 2**31, (p, hk)); vs = rng.integers(39, 43, (p, hk))
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


def device_layer_weights(w):
    """Host weight dict of make_weights -> the device form Qwen3DecoderLayerInteger takes."""
    from mini_sgl_integer_b200.layers.decoder_layer import _Linear
    lin = lambda t: _Linear(d(t[0]), weight_mul=d(t[1]), weight_shift=d(t[2]))
    return {"qkv": lin(w["qkv"]), "o": lin(w["o"]), "gate_up": lin(w["gate_up"]), "down": lin(w["down"]),
            "input_norm": d(w["input_norm"]), "post_norm": d(w["post_norm"]), "q_norm": d(w["q_norm"]), "k_norm": d(w["k_norm"])}


def shard_layer_weights(w, rank, world, hq=HQ, hk=HK, inter=INTER):
    """Rank `rank`'s shard of a layer's host weights, on the device: q | k | v and gate | up output channels of
    the local heads / columns, input features of o / down (models/weight.py:12-52)."""
    from mini_sgl_integer_b200.layers.decoder_layer import _Linear
    hq_l, hk_l, inter_l = hq // world, hk // world, inter // world

    def rows(t, idx):
        wq, wm, ws = t
        return _Linear(d(wq[idx]), weight_mul=d(wm[idx]), weight_shift=d(ws[idx]))

    def cols(t, per):
        wq, wm, ws = t
        return _Linear(d(wq[:, rank * per:(rank + 1) * per]), weight_mul=d(wm), weight_shift=d(ws))
    q0, k0, v0 = 0, hq * 128, (hq + hk) * 128
    qkv_idx = np.concatenate([np.arange(q0 + rank * hq_l * 128, q0 + (rank + 1) * hq_l * 128),
                              np.arange(k0 + rank * hk_l * 128, k0 + (rank + 1) * hk_l * 128),
                              np.arange(v0 + rank * hk_l * 128, v0 + (rank + 1) * hk_l * 128)])
    gu_idx = np.concatenate([np.arange(rank * inter_l, (rank + 1) * inter_l), inter + np.arange(rank * inter_l, (rank + 1) * inter_l)])
    return {"qkv": rows(w["qkv"], qkv_idx), "o": cols(w["o"], hq_l * 128), "gate_up": rows(w["gate_up"], gu_idx),
            "down": cols(w["down"], inter_l), "input_norm": d(w["input_norm"]), "post_norm": d(w["post_norm"]),
            "q_norm": d(w["q_norm"]), "k_norm": d(w["k_norm"])}
