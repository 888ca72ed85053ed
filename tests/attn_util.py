"""Shared builders for the attention tests: a seeded paged pool on host (oracle layout) and device."""
from __future__ import annotations

import numpy as np
import torch

from oracle import attention as oattn


def make_case(seed, kv_lens, q_heads, kv_heads, num_pages, uniform=False, shift_spread=True):
    """Random int8 K/V with per-token-per-head (mul, shift) for a batch of sequences.

    Page tables are disjoint slices of a random permutation of the pool's pages.
    Returns a dict of host arrays plus the oracle-side pool.
    """
    rng = np.random.default_rng(seed)
    B = len(kv_lens)
    n_pg = [(int(l) + 15) // 16 for l in kv_lens]
    assert sum(n_pg) <= num_pages
    perm = rng.permutation(num_pages)
    tables, locs, off = [], [], 0
    for b in range(B):
        pg = perm[off:off + n_pg[b]]
        off += n_pg[b]
        tables.append(pg.astype(np.int32))
        locs.append((pg[:, None] * 16 + np.arange(16)[None, :]).reshape(-1)[: kv_lens[b]])
    T = int(sum(kv_lens))
    k8 = rng.integers(-127, 128, (T, kv_heads, 128), dtype=np.int8)
    v8 = rng.integers(-127, 128, (T, kv_heads, 128), dtype=np.int8)
    if uniform:
        km = np.full((T, kv_heads), 2062117504, dtype=np.int64); ks = np.full((T, kv_heads), 36, dtype=np.int64)
        vm = np.full((T, kv_heads), 1224789248, dtype=np.int64); vs = np.full((T, kv_heads), 35, dtype=np.int64)
    else:
        km = rng.integers(2**30, 2**31, (T, kv_heads)); vm = rng.integers(2**30, 2**31, (T, kv_heads))
        ks = rng.integers(35, 39 if shift_spread else 36, (T, kv_heads))
        vs = rng.integers(33, 38 if shift_spread else 34, (T, kv_heads))
    q8 = rng.integers(-127, 128, (B, q_heads, 128), dtype=np.int8)
    qm = rng.integers(2**30, 2**31, (B, q_heads)); qs = rng.integers(43, 46, (B, q_heads))
    pool = oattn.PagedKV(num_pages, kv_heads, 128)
    loc = np.concatenate(locs) if locs else np.zeros(0, dtype=np.int64)
    pool.store_codes(loc, k8, v8, km, ks, vm, vs)
    pitch = max(n_pg) if n_pg else 1
    table = np.zeros((B, max(pitch, 1)), dtype=np.int32)
    for b in range(B):
        table[b, : n_pg[b]] = tables[b]
    return dict(q8=q8, qm=qm.astype(np.int32), qs=qs.astype(np.int32), k8=k8, v8=v8, km=km.astype(np.int32),
                ks=ks.astype(np.int32), vm=vm.astype(np.int32), vs=vs.astype(np.int32), loc=loc.astype(np.int32),
                table=table, tables=tables, kv_lens=np.asarray(kv_lens, dtype=np.int32), pool=pool)


def device_pool(case, num_pages, kv_heads):
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    pool = Int8PagedKVCache(kv_heads, 1, 128, num_pages, "cuda")
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    if len(case["loc"]):
        pool.store_codes(d(case["k8"]), d(case["v8"]), d(case["km"]), d(case["ks"]), d(case["vm"]), d(case["vs"]),
                         d(case["loc"]), 0)
    return pool
