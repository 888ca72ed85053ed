"""int8 paged KV store + decode attention on CUDA vs the CPU oracle (bit-exact)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import fixed_point as ofp
from tests.attn_util import device_pool, make_case

pytestmark = pytest.mark.gpu


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def eq(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError(f"{len(bad)} mismatches of {a.size}, first at {bad[0]}: {a[tuple(bad[0])]} vs {b[tuple(bad[0])]}")


IMPLS = ["split", "cluster"]


def run_decode(case, pool, max_kv_len, cluster=0, **kw):
    from mini_sgl_integer_b200.attention import decode_attention_int8_paged
    need = (max_kv_len + 15) // 16
    table = case["table"]
    if table.shape[1] < need:
        table = np.pad(table, ((0, 0), (0, need - table.shape[1])))
    return decode_attention_int8_paged(d(case["q8"]), d(case["qm"]), d(case["qs"]), pool, 0, d(table),
                                       d(case["kv_lens"]), max_kv_len, cluster=cluster, **kw)


def oracle_decode(case):
    B = len(case["kv_lens"])
    return oattn.paged_attention(case["q8"], case["qm"], case["qs"], case["pool"], case["tables"],
                                 case["kv_lens"], [1] * B)


def test_store_codes_layout_matches_oracle_pool():
    case = make_case(1, [5, 16, 17, 40], 8, 2, 32)
    pool = device_pool(case, 32, 2)
    eq(pool.k_cache(0).cpu().numpy(), case["pool"].k_codes)
    eq(pool.v_cache(0).cpu().numpy(), case["pool"].v_codes)
    eq(pool.meta(0).cpu().numpy(), case["pool"].meta)


def test_store_q15_quantises_like_oracle():
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    rng = np.random.default_rng(4)
    T, H, P = 37, 4, 8
    qkv = rng.integers(-(2**21), 2**21, (T, (8 + 2 * H) * 128)).astype(np.int32)
    qkv[3, 8 * 128: 9 * 128] = 0                                   # an all-zero K head row
    k, v = qkv[:, 8 * 128:(8 + H) * 128], qkv[:, (8 + H) * 128:]
    loc = rng.permutation(P * 16)[:T].astype(np.int32)
    ref = oattn.PagedKV(P, H, 128)
    ref.store_q15(loc, k, v)
    pool = Int8PagedKVCache(H, 2, 128, P, "cuda")
    dq = d(qkv)
    pool.store_kv(dq[:, 8 * 128:(8 + H) * 128], dq[:, (8 + H) * 128:], d(loc), 1)   # strided views, layer 1
    eq(pool.k_cache(1).cpu().numpy(), ref.k_codes)
    eq(pool.v_cache(1).cpu().numpy(), ref.v_codes)
    eq(pool.meta(1).cpu().numpy(), ref.meta)
    assert int(pool.k_cache(0).abs().max()) == 0                  # the other layer is untouched


@pytest.mark.parametrize("q_heads,kv_heads", [(2, 2), (4, 2), (8, 2), (16, 2), (32, 8)])
def test_decode_split_vs_oracle(q_heads, kv_heads):
    lens = [1, 15, 16, 17, 31, 33, 64, 100, 255, 256, 257, 640, 1000]
    case = make_case(q_heads * 10 + 3, lens, q_heads, kv_heads, 256)
    pool = device_pool(case, 256, kv_heads)
    want = oracle_decode(case)
    got, codes, absmax = run_decode(case, pool, 1000, impl="split", out_q15=True, out_int8=True)
    eq(got.cpu().numpy(), want)
    wc, wm = oattn.quant_heads_int8(want)
    eq(codes.cpu().numpy(), wc); eq(absmax.cpu().numpy(), wm)
    got2 = run_decode(case, pool, 1000, impl="split")            # the workspace is reused: results must not depend on its contents
    eq(got2.cpu().numpy(), want)


@pytest.mark.parametrize("q_heads,kv_heads", [(2, 2), (4, 2), (8, 2), (16, 2), (32, 8)])
@pytest.mark.parametrize("cluster", [1, 2, 4, 8])
def test_decode_vs_oracle(q_heads, kv_heads, cluster):
    lens = [1, 15, 16, 17, 31, 33, 64, 100, 257, 640]
    case = make_case(q_heads * 10 + cluster, lens, q_heads, kv_heads, 128)
    pool = device_pool(case, 128, kv_heads)
    want = oracle_decode(case)
    got, codes, absmax = run_decode(case, pool, 640, cluster, impl="cluster", out_q15=True, out_int8=True)
    eq(got.cpu().numpy(), want)
    wc, wm = oattn.quant_heads_int8(want)
    eq(codes.cpu().numpy(), wc); eq(absmax.cpu().numpy(), wm)
    assert np.abs(want).max() > 0


def test_decode_auto_cluster_long_context_and_clamp():
    lens = [4096, 3000, 2049, 512, 7]
    case = make_case(77, lens, 8, 2, 640)
    pool = device_pool(case, 640, 2)
    want = oracle_decode(case)
    eq(run_decode(case, pool, 4096, impl="cluster").cpu().numpy(), want)
    eq(run_decode(case, pool, 8192, cluster=8, impl="cluster").cpu().numpy(), want)   # larger bound, same result
    eq(run_decode(case, pool, 4096, impl="split").cpu().numpy(), want)
    eq(run_decode(case, pool, 8192, impl="split").cpu().numpy(), want)
    codes, absmax = run_decode(case, pool, 4096, out_q15=False, out_int8=True)
    wc, wm = oattn.quant_heads_int8(want)
    eq(codes.cpu().numpy(), wc); eq(absmax.cpu().numpy(), wm)


def test_decode_zero_length_sequences_give_zero():
    case = make_case(9, [0, 20, 0], 4, 2, 8)
    pool = device_pool(case, 8, 2)
    got = run_decode(case, pool, 32, cluster=2, impl="cluster").cpu().numpy()
    eq(got, oracle_decode(case))
    eq(run_decode(case, pool, 32, impl="split").cpu().numpy(), got)
    assert not got[0].any() and not got[2].any() and got[1].any()


def test_decode_wide_shift_spread_and_uniform_scales():
    rng = np.random.default_rng(5)
    case = make_case(21, [200, 90], 8, 2, 32)
    # push a few V shifts far away from the reference scale (relative scale underflows to 0)
    case["vs"][rng.integers(0, 290, 40)] += 20
    case["pool"].store_codes(case["loc"], case["k8"], case["v8"], case["km"], case["ks"], case["vm"], case["vs"])
    pool = device_pool(case, 32, 2)
    eq(run_decode(case, pool, 256, cluster=2, impl="cluster").cpu().numpy(), oracle_decode(case))
    eq(run_decode(case, pool, 256, impl="split").cpu().numpy(), oracle_decode(case))
    uni = make_case(22, [48, 200], 4, 2, 32, uniform=True)
    pool = device_pool(uni, 32, 2)
    eq(run_decode(uni, pool, 256, cluster=1, impl="cluster").cpu().numpy(), oracle_decode(uni))
    eq(run_decode(uni, pool, 256, impl="split").cpu().numpy(), oracle_decode(uni))


def test_decode_reduces_to_reference_prefill_row(golden):
    """Uniform scales: decode over L keys == row L-1 of int8_context_attention_fwd (reference golden)."""
    ms = golden["attn_ms"]
    q, k, v = golden["attn_q"], golden["attn_k"], golden["attn_v"]
    ref = oattn.context_attention(q, k, v, ms[0], ms[1], ms[2], [0, 16], [16, 32], True)
    assert np.array_equal(oattn.q15_to_bf16_bits(ref), golden["attn_out_bf16_bits"])
    from mini_sgl_integer_b200.attention import Int8PagedKVCache, decode_attention_int8_paged
    pool = Int8PagedKVCache(2, 1, 128, 8, "cuda")
    pages = {0: [5], 1: [7, 2]}
    table = np.zeros((2, 2), dtype=np.int32)
    for b, (st, L) in enumerate(((0, 16), (16, 32))):
        table[b, : len(pages[b])] = pages[b]
        loc = np.concatenate([np.arange(16) + 16 * p for p in pages[b]])[:L].astype(np.int32)
        full = lambda val: torch.full((L, 2), int(val), dtype=torch.int32, device="cuda")
        pool.store_codes(d(k[st:st + L]), d(v[st:st + L]), full(ms[1][0]), full(ms[1][1]), full(ms[2][0]),
                         full(ms[2][1]), d(loc), 0)
    q_last = np.stack([q[15], q[47]])
    qm = np.full((2, 4), ms[0][0], dtype=np.int32); qs = np.full((2, 4), ms[0][1], dtype=np.int32)
    got = decode_attention_int8_paged(d(q_last), d(qm), d(qs), pool, 0, d(table),
                                      d(np.array([16, 32], dtype=np.int32)), 32, cluster=2).cpu().numpy()
    eq(got.astype(np.int64), np.stack([ref[15], ref[47]]))
    bits = oattn.q15_to_bf16_bits(got.astype(np.int64))
    eq(bits, np.stack([golden["attn_out_bf16_bits"][15], golden["attn_out_bf16_bits"][47]]))


def test_decode_headline_shape_sample_and_invariants():
    """Batch 64, 32/8 heads, contexts U[512,4096], 200k-page pool: oracle on a sample of sequences,
    and page-permutation invariance (a size-independent property) on all of them."""
    rng = np.random.default_rng(0)
    lens = rng.integers(512, 4097, 64).tolist()
    P = 200_000
    case = make_case(0, lens, 32, 8, P)
    pool = device_pool(case, P, 8)
    got = run_decode(case, pool, 4096).cpu().numpy()
    sample = [0, 7, 13, 21, 34, 42, 55, 63]
    sub = oattn.paged_attention(case["q8"][sample], case["qm"][sample], case["qs"][sample], case["pool"],
                                [case["tables"][i] for i in sample], case["kv_lens"][sample], [1] * len(sample))
    eq(got[sample], sub)
    # same tokens placed on other pages of the pool: identical output
    case2 = make_case(0, lens, 32, 8, P)
    perm = np.random.default_rng(123).permutation(P)
    t2 = [perm[t] for t in case2["tables"]]
    loc2 = np.concatenate([(pg[:, None] * 16 + np.arange(16)[None, :]).reshape(-1)[:l] for pg, l in zip(t2, lens)])
    case2["loc"] = loc2.astype(np.int32)
    table2 = np.zeros_like(case2["table"])
    for b, pg in enumerate(t2):
        table2[b, : len(pg)] = pg
    case2["table"] = table2
    pool2 = device_pool(case2, P, 8)
    got2 = run_decode(case2, pool2, 4096, cluster=8, impl="cluster").cpu().numpy()
    eq(got2, got)


def _extend_case(seed, kv_lens, q_lens, q_heads, kv_heads, num_pages, uniform=False):
    case = make_case(seed, kv_lens, q_heads, kv_heads, num_pages, uniform=uniform)
    rng = np.random.default_rng(seed + 99)
    T = int(sum(q_lens))
    case["q8"] = rng.integers(-127, 128, (T, q_heads, 128), dtype=np.int8)
    case["qm"] = rng.integers(2**30, 2**31, (T, q_heads)).astype(np.int32)
    case["qs"] = rng.integers(43, 46, (T, q_heads)).astype(np.int32)
    case["q_lens"] = np.asarray(q_lens, dtype=np.int32)
    return case


def run_extend(case, pool, max_kv_len, cluster=0, **kw):
    from mini_sgl_integer_b200.attention import extend_attention_int8_paged
    need = (max_kv_len + 15) // 16
    table = case["table"]
    if table.shape[1] < need:
        table = np.pad(table, ((0, 0), (0, need - table.shape[1])))
    return extend_attention_int8_paged(d(case["q8"]), d(case["qm"]), d(case["qs"]), pool, 0, d(table),
                                       d(case["kv_lens"]), d(case["q_lens"]), max_kv_len, cluster=cluster, **kw)


@pytest.mark.parametrize("cluster", [0, 1, 2, 4])
def test_extend_over_prefix_vs_oracle(cluster):
    """New tokens attend the cached prefix and, causally, themselves (the layer case: 16 new tokens over
    prefixes 0, 16, 48, 112, plus ragged ones)."""
    kv_lens = [16, 32, 64, 128, 37, 5, 200]
    q_lens = [16, 16, 16, 16, 9, 5, 1]
    case = _extend_case(40 + cluster, kv_lens, q_lens, 16, 8, 64)
    pool = device_pool(case, 64, 8)
    want = oattn.paged_attention(case["q8"], case["qm"], case["qs"], case["pool"], case["tables"], kv_lens, q_lens)
    got, codes, absmax = run_extend(case, pool, 256, cluster, impl="split" if cluster == 0 else "cluster",
                                    out_q15=True, out_int8=True)
    eq(got.cpu().numpy(), want)
    wc, wm = oattn.quant_heads_int8(want)
    eq(codes.cpu().numpy(), wc); eq(absmax.cpu().numpy(), wm)


@pytest.mark.parametrize("q_heads,kv_heads", [(2, 2), (4, 2), (8, 2), (8, 1)])
def test_tiled_prefill_vs_oracle(q_heads, kv_heads):
    """The tiled prefill kernel (query rows on the M side, keys streamed per tile) for every group size: ragged
    prompts with and without a cached prefix, single new tokens, prompts that end inside a page and inside a
    tile, Q15.16 and int8 outputs."""
    kv_lens = [16, 32, 64, 128, 37, 5, 200, 1, 131, 333]
    q_lens = [16, 16, 16, 16, 9, 5, 1, 1, 131, 70]
    case = _extend_case(60 + q_heads, kv_lens, q_lens, q_heads, kv_heads, 80)
    pool = device_pool(case, 80, kv_heads)
    want = oattn.paged_attention(case["q8"], case["qm"], case["qs"], case["pool"], case["tables"], kv_lens, q_lens)
    got, codes, absmax = run_extend(case, pool, 512, impl="tiled", out_q15=True, out_int8=True)
    eq(got.cpu().numpy(), want)
    wc, wm = oattn.quant_heads_int8(want)
    eq(codes.cpu().numpy(), wc); eq(absmax.cpu().numpy(), wm)
    # the row-at-a-time kernels give the same bits
    eq(run_extend(case, pool, 512, cluster=1, impl="cluster").cpu().numpy(), want)


@pytest.mark.parametrize("kv_len,q_len", [(1024, 1024), (3584, 512)])
def test_tiled_prefill_long_prompts_vs_oracle(kv_len, q_len):
    """A 1024-token prompt without a prefix, and 512 new tokens over a 3072-token cached prefix."""
    case = _extend_case(70, [kv_len, 40], [q_len, 40], 8, 2, 240)
    pool = device_pool(case, 240, 2)
    want = oattn.paged_attention(case["q8"], case["qm"], case["qs"], case["pool"], case["tables"], [kv_len, 40], [q_len, 40])
    got = run_extend(case, pool, 3584, impl="tiled").cpu().numpy()
    eq(got, want)
    assert np.abs(want).max() > 0


def test_tiled_prefill_uniform_scales_and_explicit_row_starts():
    """Uniform scales (the reference's per-tensor case) through the direct entry point with row offsets that leave
    gaps between the sequences: rows outside every sequence stay untouched."""
    from mini_sgl_integer_b200.attention import prefill_attention_int8_paged
    kv_lens, q_lens = [48, 20, 100], [48, 7, 33]
    case = _extend_case(80, kv_lens, q_lens, 8, 2, 16, uniform=True)
    pool = device_pool(case, 16, 2)
    want = oattn.paged_attention(case["q8"], case["qm"], case["qs"], case["pool"], case["tables"], kv_lens, q_lens)
    T = sum(q_lens)
    starts = np.array([3, 60, 70], dtype=np.int32)                       # sequence b's rows begin at starts[b]
    rows = 110
    q = np.zeros((rows, 8, 128), dtype=np.int8); qm = np.ones((rows, 8), dtype=np.int32); qs = np.full((rows, 8), 44, dtype=np.int32)
    src = 0
    for b, n in enumerate(q_lens):
        q[starts[b]:starts[b] + n] = case["q8"][src:src + n]; qm[starts[b]:starts[b] + n] = case["qm"][src:src + n]
        qs[starts[b]:starts[b] + n] = case["qs"][src:src + n]; src += n
    table = np.pad(case["table"], ((0, 0), (0, 8 - case["table"].shape[1])))
    out = prefill_attention_int8_paged(d(q), d(qm), d(qs), pool, 0, d(table), d(case["kv_lens"]), d(case["q_lens"]), 128, 48,
                                       q_start=d(starts))
    out = out.cpu().numpy()
    src = 0
    for b, n in enumerate(q_lens):
        eq(out[starts[b]:starts[b] + n], want[src:src + n]); src += n


def test_extend_without_prefix_reduces_to_reference(golden):
    """Uniform scales, no prefix: the extend kernel reproduces int8_context_attention_fwd bit for bit."""
    from mini_sgl_integer_b200.attention import Int8PagedKVCache, extend_attention_int8_paged
    ms = golden["attn_ms"]
    q, k, v = golden["attn_q"], golden["attn_k"], golden["attn_v"]
    pool = Int8PagedKVCache(2, 1, 128, 8, "cuda")
    pages = {0: [5], 1: [7, 2]}
    table = np.zeros((2, 2), dtype=np.int32)
    for b, (st, L) in enumerate(((0, 16), (16, 32))):
        table[b, : len(pages[b])] = pages[b]
        loc = np.concatenate([np.arange(16) + 16 * p for p in pages[b]])[:L].astype(np.int32)
        full = lambda val: torch.full((L, 2), int(val), dtype=torch.int32, device="cuda")
        pool.store_codes(d(k[st:st + L]), d(v[st:st + L]), full(ms[1][0]), full(ms[1][1]), full(ms[2][0]),
                         full(ms[2][1]), d(loc), 0)
    qm = np.full((48, 4), ms[0][0], dtype=np.int32); qs = np.full((48, 4), ms[0][1], dtype=np.int32)
    lens = d(np.array([16, 32], dtype=np.int32))
    got = extend_attention_int8_paged(d(q), d(qm), d(qs), pool, 0, d(table), lens, lens, 32, cluster=2).cpu().numpy()
    eq(oattn.q15_to_bf16_bits(got.astype(np.int64)), golden["attn_out_bf16_bits"])


def test_row_order_hint_does_not_change_results():
    lens = [700, 33, 1, 256, 2049, 16, 900]
    case = make_case(9, lens, 8, 2, 300)
    pool = device_pool(case, 300, 2)
    want = oracle_decode(case)
    order = np.argsort(-np.asarray(lens), kind="stable").astype(np.int32)
    for ro in (None, order, order[::-1].copy(), np.arange(len(lens), dtype=np.int32)):
        got = run_decode(case, pool, 2049, row_order=None if ro is None else d(ro)).cpu().numpy()
        eq(got, want)
    # more rows than the in-kernel ranking handles (64): given order and caller's order
    lens = list(np.random.default_rng(3).integers(1, 90, 80))
    case = make_case(10, lens, 4, 1, 600)
    pool = device_pool(case, 600, 1)
    want = oracle_decode(case)
    eq(run_decode(case, pool, 96).cpu().numpy(), want)
    eq(run_decode(case, pool, 96, row_order=d(np.argsort(-np.asarray(lens), kind="stable").astype(np.int32))).cpu().numpy(), want)


def test_auto_falls_back_to_workspace_passes_for_long_contexts():
    """A context too long for the cluster kernel's shared memory (eight query heads per KV head, 48k keys)."""
    from mini_sgl_integer_b200.attention.ops import _cluster_fits
    assert _cluster_fits(4, 4096) and not _cluster_fits(8, 48000)
    lens = [48000, 33]
    case = make_case(5, lens, 8, 1, 3100)
    pool = device_pool(case, 3100, 1)
    got = run_decode(case, pool, 48000).cpu().numpy()          # impl="auto"
    eq(got, oracle_decode(case))


def test_extend_empty_batch():
    from mini_sgl_integer_b200.attention import Int8PagedKVCache, extend_attention_int8_paged
    pool = Int8PagedKVCache(2, 1, 128, 4, "cuda")
    z = lambda *s, dt=torch.int32: torch.zeros(s, dtype=dt, device="cuda")
    out = extend_attention_int8_paged(z(0, 4, 128, dt=torch.int8), z(0, 4), z(0, 4), pool, 0, z(1, 2), z(1), z(1), 32)
    assert out.shape == (0, 4, 128)


@pytest.mark.parametrize("phase", ["prefill", "decode"])
def test_backend_forward_matches_oracle(phase):
    """The plug-in class end to end: metadata from requests, K/V quantised into the pool, q quantised, attention."""
    from types import SimpleNamespace
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.attention.backend import B200Int8Backend, token_locations
    from oracle import fixed_point as ofp
    rng = np.random.default_rng(31)
    HQ, HK, P = 8, 2, 24
    table = rng.permutation(P).astype(np.int32).reshape(4, 6)            # 4 request slots x 6 pages
    if phase == "prefill":
        reqs = [(2, 0, 37), (0, 0, 5), (3, 0, 64)]                         # (table_idx, cached_len, device_len)
    else:
        reqs = [(2, 36, 37), (0, 4, 5), (3, 63, 64)]
    ref_pool = oattn.PagedKV(P, HK, 128)
    pool = Int8PagedKVCache(HK, 1, 128, P, "cuda")
    if phase == "decode":                                                 # cached prefixes
        for t, c, _ in reqs:
            loc = (table[t][np.arange(c) // 16] * 16 + np.arange(c) % 16).astype(np.int32)
            k8 = rng.integers(-127, 128, (c, HK, 128), dtype=np.int8); v8 = rng.integers(-127, 128, (c, HK, 128), dtype=np.int8)
            km = rng.integers(2**30, 2**31, (c, HK)); ks = rng.integers(35, 39, (c, HK))
            vm = rng.integers(2**30, 2**31, (c, HK)); vs = rng.integers(33, 38, (c, HK))
            ref_pool.store_codes(loc, k8, v8, km, ks, vm, vs)
            pool.store_codes(d(k8), d(v8), d(km.astype(np.int32)), d(ks.astype(np.int32)), d(vm.astype(np.int32)),
                             d(vs.astype(np.int32)), d(loc), 0)
    q_lens = [dl - c for _, c, dl in reqs]
    T = sum(q_lens)
    q = rng.integers(-(2**20), 2**20, (T, HQ * 128)).astype(np.int32)
    k = rng.integers(-(2**20), 2**20, (T, HK * 128)).astype(np.int32)
    v = rng.integers(-(2**20), 2**20, (T, HK * 128)).astype(np.int32)
    positions = np.concatenate([np.arange(c, dl) for _, c, dl in reqs]).astype(np.int32)
    row_of = np.concatenate([np.full(n, i) for i, n in enumerate(q_lens)])
    rq = [SimpleNamespace(table_idx=t, cached_len=c, device_len=dl, extend_len=dl - c) for t, c, dl in reqs]
    batch = SimpleNamespace(reqs=rq, padded_reqs=rq, phase=phase, is_prefill=phase == "prefill", is_decode=phase == "decode",
                            size=len(rq), padded_size=len(rq))
    be = B200Int8Backend.from_heads(HQ, HK, pool, d(table))
    be.prepare_metadata(batch)
    batch.out_loc = token_locations(batch.attn_metadata.page_table, d(positions), d(row_of))
    got = be.forward(d(q), d(k), d(v), 0, batch).cpu().numpy()

    out_loc = np.concatenate([table[t][np.arange(c, dl) // 16] * 16 + np.arange(c, dl) % 16 for t, c, dl in reqs]).astype(np.int32)
    eq(batch.out_loc.cpu().numpy(), out_loc)
    ref_pool.store_q15(out_loc, k, v)
    q8, _, qm = ofp.per_token_quant_from_q15(q.reshape(T, HQ, 128))
    q_mul, q_shift = oattn.absmax_to_mul_shift(qm[..., 0])
    want = oattn.paged_attention(q8, q_mul, q_shift, ref_pool, [table[t] for t, _, _ in reqs], [dl for _, _, dl in reqs], q_lens)
    eq(got.reshape(T, HQ, 128), want)
    assert batch.attn_metadata.get_last_indices(3).tolist() == (np.cumsum(q_lens) - 1).tolist()


def test_fused_qkv_preparation_equals_the_separate_steps():
    """One launch for q/k-norm + RoPE + rotation + KV store + q quant gives the bits of the four-call sequence."""
    from mini_sgl_integer_b200.attention import Int8PagedKVCache, qkv_rope_quant_store
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    rng = np.random.default_rng(17)
    T, HQ, HK, P = 37, 8, 2, 12
    qkv = rng.integers(-(2**21), 2**21, (T, (HQ + 2 * HK) * 128)).astype(np.int32)
    qkv[3, HQ * 128: (HQ + 1) * 128] = 0                            # an all-zero K head row
    qkv[5, :128] = 0                                                # an all-zero q head row
    loc = rng.permutation(P * 16)[:T].astype(np.int32)
    loc[7] = P * 16 + 3                                             # outside the pool: dropped
    pos = rng.integers(0, 64, T).astype(np.int32)
    inv = 1.0 / (1000000.0 ** (torch.arange(0, 128, 2, dtype=torch.float) / 128))
    fr = torch.einsum("i,j -> ij", torch.arange(64, dtype=torch.float), inv)
    cache = torch.clamp(torch.round(torch.cat((fr.cos(), fr.sin()), -1) * 32768), -32768, 32767).to(torch.int32).cuda()
    qn = d(rng.integers(2**11, 2**13, 128).astype(np.int32)); kn = d(rng.integers(2**12, 2**14, 128).astype(np.int32))
    for qnw, knw in ((qn, kn), (None, None)):
        a, b = Int8PagedKVCache(HK, 1, 128, P, "cuda"), Int8PagedKVCache(HK, 1, 128, P, "cuda")
        dq = d(qkv)
        q8, q_mul, q_shift = qkv_rope_quant_store(d(pos), dq, HQ, a, 0, d(loc), cache, qnw, knw)
        qd, kd = HQ * 128, HK * 128
        q, k = fp.qk_norm_rope_fwht(d(pos), dq[:, :qd].view(T, HQ, 128), dq[:, qd:qd + kd], cache, qnw, knw)
        b.store_kv(k, dq[:, qd + kd:], d(loc), 0)
        w8, _, am = fp.per_token_quant_int8_from_q15(q.reshape(T * HQ, 128), return_absmax=True)
        wm, ws = fp.absmax_to_mul_shift(am)
        eq(q8.cpu().numpy().reshape(T * HQ, 128), w8.cpu().numpy())
        eq(q_mul.cpu().numpy().reshape(-1), wm.cpu().numpy().reshape(-1)); eq(q_shift.cpu().numpy().reshape(-1), ws.cpu().numpy().reshape(-1))
        eq(a.k_cache(0).cpu().numpy(), b.k_cache(0).cpu().numpy())
        eq(a.v_cache(0).cpu().numpy(), b.v_cache(0).cpu().numpy())
        eq(a.meta(0).cpu().numpy(), b.meta(0).cpu().numpy())


def test_decode_seeded_sweep_of_shapes_and_options():
    """Random batches, group sizes, cluster sizes, row orders and output forms, both implementations."""
    rng = np.random.default_rng(2024)
    for trial in range(14):
        G = int(rng.choice([1, 2, 4, 8]))
        hk = int(rng.choice([1, 2]))
        B = int(rng.integers(1, 10))
        lens = rng.integers(0, 700, B).tolist()
        if trial % 4 == 0:
            lens[0] = 0
        longest = max(max(lens), 1)
        max_kv_len = int(longest + rng.integers(0, 40))
        P = sum((l + 15) // 16 for l in lens) + 4
        case = make_case(1000 + trial, lens, G * hk, hk, P)
        pool = device_pool(case, P, hk)
        want = oracle_decode(case)
        want8, want_m = oattn.quant_heads_int8(want)
        kw = dict(cluster=int(rng.choice([0, 1, 2, 4, 8])), impl="cluster",
                  row_order=d(rng.permutation(B).astype(np.int32)) if trial % 2 else None)
        o32, o8, om = run_decode(case, pool, max_kv_len, out_int8=True, **kw)
        eq(o32.cpu().numpy(), want); eq(o8.cpu().numpy(), want8); eq(om.cpu().numpy(), want_m.reshape(B, -1))
        o32 = run_decode(case, pool, max_kv_len, impl="split")
        eq(o32.cpu().numpy(), want)
