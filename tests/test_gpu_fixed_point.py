"""CUDA row kernels vs the CPU oracle and the reference's golden vectors (bit-exact)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import fixed_point as ofp

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fp():
    from mini_sgl_integer_b200.kernel import fixed_point
    return fixed_point


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.cpu().numpy()


def eq(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (a.shape, b.shape, a.dtype, b.dtype)
    if not np.array_equal(a, b):
        bad = np.argwhere(a != b)
        raise AssertionError(f"{len(bad)} mismatches, first at {bad[0]}: {a[tuple(bad[0])]} vs {b[tuple(bad[0])]}")


# ----------------------------------------------------------------------------- golden vectors
def test_golden_rmsnorm(fp, golden):
    eq(host(fp.rmsnorm_int_only_v2(dev(golden["norm_x"]), dev(golden["norm_w"]))), golden["norm_out"])
    o, r = fp.fused_add_rmsnorm_int_only_v2(dev(golden["norm_r"]), dev(golden["norm_x"]), dev(golden["norm_w"]))
    eq(host(o), golden["fused_out"]); eq(host(r), golden["fused_res"])
    eq(host(fp.rmsnorm_int_only_v2(dev(golden["norm_edge_x"]), dev(golden["norm_edge_w"]))), golden["norm_edge_out"])
    o, r = fp.fused_add_rmsnorm_int_only_v2(dev(golden["fused_edge_r"]), dev(golden["norm_edge_x"]), dev(golden["norm_edge_w"]))
    eq(host(o), golden["fused_edge_out"]); eq(host(r), golden["fused_edge_res"])
    eq(host(fp.rmsnorm_int_only_v2(dev(golden["norm_packed_x"]), dev(golden["norm_packed_w"]))), golden["norm_packed_out"])
    o, r = fp.fused_add_rmsnorm_int_only_v2(dev(golden["fused_wide_r"]), dev(golden["fused_wide_x"]), dev(golden["fused_wide_w"]))
    eq(host(o), golden["fused_wide_out"]); eq(host(r), golden["fused_wide_res"])


def test_golden_silu_fwht_quant_chain(fp, golden):
    s = fp.silu_and_mul_int_only(dev(golden["silu_in"]))
    eq(host(s), golden["silu_out"])
    f = fp.apply_blockwise_fwht_q15(s, 128)
    eq(host(f), golden["bfwht_out"])
    q, sc = fp.per_token_quant_int8_from_q15(f)
    eq(host(q), golden["quant_codes"]); eq(host(sc), golden["quant_scale"])
    # the fused kernel gives the same codes in one pass
    codes, scale, absmax, q15 = fp.silu_mul_fwht_quant(dev(golden["silu_in"]), 128, want_q15=True)
    eq(host(codes), golden["quant_codes"]); eq(host(scale), golden["quant_scale"]); eq(host(q15), golden["bfwht_out"])
    eq(host(fp.silu_and_mul_int_only(dev(golden["silu_edge_in"]))), golden["silu_edge_out"])


def test_golden_fwht(fp, golden):
    for n in (64, 128, 256):
        eq(host(fp.fwht_int_q15(dev(golden[f"fwht{n}_in"]))), golden[f"fwht{n}_out"])
    eq(host(fp.fwht_int_q15(dev(golden["fwht_sat_in"]))), golden["fwht_sat_out"])
    eq(host(fp.fwht_int_q15(dev(golden["fwht_sat_in"]), normalize=False)), golden["fwht_sat_raw"])
    eq(host(fp.fwht_int_q15(dev(golden["fwht_small_in"]))), golden["fwht_small_out"])


def test_golden_quant_edges(fp, golden):
    q, s = fp.per_token_quant_int8_from_q15(dev(golden["quant_edge_in"]))
    eq(host(q), golden["quant_edge_codes"]); eq(host(s), golden["quant_edge_scale"])


def test_golden_quant_rows_holding_int_min(fp, golden):
    """Rows with -2^31 beside ordinary values: the code is -128 on every quantising path (row absmax below 2^22,
    above it, near 2^31, and a row that is otherwise zero)."""
    x = golden["quant_intmin_in"]
    q, s = fp.per_token_quant_int8_from_q15(dev(x))
    eq(host(q), golden["quant_intmin_codes"]); eq(host(s), golden["quant_intmin_scale"])
    # the same rows as V heads on their way into the pool, and quantised with a given absmax
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.tp_linear import quant_given_absmax
    from oracle import attention as oattn
    rows = np.concatenate([x, x], axis=1)                              # [4, 128]: one 128-wide head row per token
    pool = Int8PagedKVCache(1, 1, 128, 2, "cuda")
    loc = np.array([3, 16, 17, 31], dtype=np.int32)
    pool.store_kv(dev(rows), dev(rows), dev(loc), 0)
    ref = oattn.PagedKV(2, 1, 128)
    ref.store_q15(loc, rows, rows)
    eq(host(pool.k_cache(0)), ref.k_codes); eq(host(pool.v_cache(0)), ref.v_codes); eq(host(pool.meta(0)), ref.meta)
    want, _, m = ofp.per_token_quant_from_q15(rows)
    eq(host(quant_given_absmax(dev(rows), dev(m.reshape(-1)))), want)


def test_quant_with_a_given_absmax_below_the_rows_maximum_clamps(fp):
    """per_token_quant_int8_from_q15's clamp to [-128, 127] (layers/quantization/w8a8_int8.py:122-125) when the caller's
    absmax does not bound the row: values far beyond it, at the rails, and -2**31."""
    from mini_sgl_integer_b200.layers.tp_linear import quant_given_absmax
    rng = np.random.default_rng(31)
    x = rng.integers(-(2**24), 2**24, (6, 256)).astype(np.int64)
    x[0, :8] = [2**31 - 1, -(2**31), 2**30, -(2**30), 5 * 2**22, -5 * 2**22, 2**23, -(2**23)]
    x = x.astype(np.int32)
    m = np.array([2**22, 1, 7, 2**24, 2**20 + 3, 2**30], dtype=np.int32)
    q = (x.astype(np.float32) * np.float32(127.0)) / m.astype(np.float32)[:, None]
    want = np.clip(np.rint(q), -128, 127).astype(np.int8)
    eq(host(quant_given_absmax(dev(x), dev(m))), want)


def test_golden_per_tensor_quantiser(golden):
    """quantize_per_tensor_int8_ms (the reference's prefill quantiser) on the device: codes, multiplier, shift."""
    from mini_sgl_integer_b200.attention import quantize_per_tensor_int8_ms
    for key in ("ptq", "ptq0", "ptq1", "ptq2", "ptq3"):
        bits = golden[f"{key}_in_bf16_bits"]
        q, mul, shift = quantize_per_tensor_int8_ms(dev(bits).view(torch.bfloat16))
        eq(host(q), golden[f"{key}_codes"])
        want_mul, want_shift = (int(v) for v in golden[f"{key}_ms"])
        assert int(shift) == want_shift, key
        # ptq0: the multiplier exceeds int32; the x86 fixture wrapped, a CUDA device (the reference's too) saturates
        assert int(mul) == (2**31 - 1 if key == "ptq0" else want_mul), key
    with pytest.raises(TypeError):
        quantize_per_tensor_int8_ms(torch.zeros(4, device="cuda"))


def _cache(pos, rows, n=4096):
    c = np.zeros((n, rows.shape[1]), dtype=np.int32)
    c[pos] = rows
    return c


def test_golden_rope(fp, golden):
    cache = dev(_cache(golden["rope_pos"], golden["rope_cache_rows"]))
    q, k = fp.rope_int_q15(dev(golden["rope_pos"]), dev(golden["rope_q"]), dev(golden["rope_k"]), cache)
    eq(host(q), golden["rope_q_out"]); eq(host(k), golden["rope_k_out"])
    q, k = fp.rope_fwht_int_q15(dev(golden["rope_pos"]), dev(golden["rope_q"]), dev(golden["rope_k"]), cache)
    eq(host(q), golden["ropefwht_q_out"]); eq(host(k), golden["ropefwht_k_out"])
    cache = dev(_cache(golden["rope_edge_pos"], golden["rope_edge_cache_rows"]))
    q, k = fp.rope_int_q15(dev(golden["rope_edge_pos"]), dev(golden["rope_edge_q"]), dev(golden["rope_edge_k"]), cache)
    eq(host(q), golden["rope_edge_q_out"]); eq(host(k), golden["rope_edge_k_out"])


def test_golden_to_from_fixed(fp, golden):
    x = golden["tofixed_in"]
    got = host(fp.to_fixed(dev(x)))
    want = golden["tofixed_out"]
    eq(got, want)
    xb = torch.from_numpy(golden["tofixed_bf16_in_bits"]).view(torch.bfloat16).cuda()
    got, want = host(fp.to_fixed(xb)), golden["tofixed_bf16_out"].copy()
    over = xb.float().cpu().numpy() >= 32768.0   # Q15.16 overflow: CUDA saturates, the x86 run wrapped
    assert (got[over] == 2**31 - 1).all()
    eq(got[~over], want[~over])
    eq(host(fp.from_fixed(dev(golden["fromfixed_in"]), torch.float32)), golden["fromfixed_f32"])
    eq(host(fp.from_fixed(dev(golden["fromfixed_in"]), torch.bfloat16).view(torch.int16)), golden["fromfixed_bf16_bits"])


# ----------------------------------------------------------------------------- oracle, seeded
@pytest.mark.parametrize("rows,hidden", [(1, 4), (3, 128), (5, 1024), (2, 1028), (7, 4096), (3, 5120), (2, 8192),
                                         (2, 12288), (1, 32768)])
def test_rmsnorm_shapes_vs_oracle(fp, rows, hidden):
    rng = np.random.default_rng(hidden + rows)
    x = rng.integers(-(2**24), 2**24, (rows, hidden)).astype(np.int32)
    r = rng.integers(-(2**24), 2**24, (rows, hidden)).astype(np.int32)
    w = rng.integers(2**13, 2**15 + 1, hidden).astype(np.int32)
    eq(host(fp.rmsnorm_int_only_v2(dev(x), dev(w))), ofp.rmsnorm_v2(x, w))
    o, ro = fp.fused_add_rmsnorm_int_only_v2(dev(r), dev(x), dev(w))
    eo, er = ofp.fused_add_rmsnorm_v2(r, x, w)
    eq(host(o), eo); eq(host(ro), er)
    codes, scale, absmax, res_out, norm = fp.fused_add_rmsnorm_quant(dev(x), dev(r), dev(w), want_norm=True)
    q, s, m = ofp.per_token_quant_from_q15(eo)
    eq(host(codes), q); eq(host(scale), s); eq(host(absmax), m); eq(host(res_out), er); eq(host(norm), eo)
    codes, scale, absmax, res_out, norm = fp.fused_add_rmsnorm_quant(dev(x), None, dev(w))
    q, s, m = ofp.per_token_quant_from_q15(ofp.rmsnorm_v2(x, w))
    eq(host(codes), q); eq(host(scale), s); eq(host(absmax), m)
    assert res_out is None and norm is None


def test_rmsnorm_3d_and_packed(fp):
    rng = np.random.default_rng(5)
    x = rng.integers(-(2**22), 2**22, (3, 5, 4 * 128)).astype(np.int32)
    w = rng.integers(2**12, 2**16, 128).astype(np.int32)
    eq(host(fp.rmsnorm_int_only_v2(dev(x), dev(w))), ofp.rmsnorm_v2(x, w))


@pytest.mark.parametrize("rows,inter", [(2, 128), (3, 3072), (2, 12288), (2, 17408), (1, 25600), (1, 32768)])
def test_silu_fused_vs_oracle(fp, rows, inter):
    rng = np.random.default_rng(inter)
    x = np.clip(np.rint(rng.normal(0, 2**17, (rows, 2 * inter))), -(2**31), 2**31 - 1).astype(np.int32)
    s = ofp.silu_and_mul(x)
    eq(host(fp.silu_and_mul_int_only(dev(x))), s)
    f = ofp.blockwise_fwht_q15(s, 128)
    q, sc, m = ofp.per_token_quant_from_q15(f)
    codes, scale, absmax, q15 = fp.silu_mul_fwht_quant(dev(x), 128, want_q15=True)
    eq(host(q15), f); eq(host(codes), q); eq(host(scale), sc); eq(host(absmax), m)
    codes, scale, absmax, q15 = fp.silu_mul_fwht_quant(dev(x), 128)
    eq(host(codes), q); assert q15 is None
    q0, s0, m0 = ofp.per_token_quant_from_q15(s)
    codes, scale, absmax, _ = fp.silu_mul_fwht_quant(dev(x), 0)
    eq(host(codes), q0); eq(host(scale), s0); eq(host(absmax), m0)


def test_silu_fused_magnitude_threshold(fp):
    """Warps whose gate / up magnitudes all lie below 2**20 take a path without saturation checks: values at and
    around the limit, and single outliers far above it, in some 128-blocks of a row and not in others."""
    rng = np.random.default_rng(23)
    rows, inter = 6, 4096
    x = np.rint(rng.normal(0, 2**17, (rows, 2 * inter))).astype(np.int64)
    x = np.clip(x, -(2**20) + 1, 2**20 - 1)
    edge = [2**20 - 1, -(2**20) + 1, 2**20, -(2**20), 2**20 + 1, -(2**20) - 1, 2**23, -(2**23), 2**24, 2**27, -(2**31), 2**31 - 1]
    for r in range(rows):
        for j, e in enumerate(edge):
            blk = (3 * j + r) % (inter // 128)
            col = blk * 128 + int(rng.integers(0, 128))
            x[r, col + (inter if (j + r) % 2 else 0)] = e                     # gate half or up half
            if r == rows - 1:
                x[r, col], x[r, col + inter] = e, edge[(j + 5) % len(edge)]    # both halves of one element
    x[0, :] = np.clip(x[0, :], -(2**20) + 1, 2**20 - 1)                        # one row entirely on the short path
    x[0, 5], x[0, inter + 5] = -(2**20) + 1, 2**20 - 1                         # the largest product the short path sees
    x[0, 6], x[0, inter + 6] = 2**20 - 1, -(2**20)
    x = x.astype(np.int32)
    s = ofp.silu_and_mul(x)
    f = ofp.blockwise_fwht_q15(s, 128)
    q, sc, m = ofp.per_token_quant_from_q15(f)
    codes, scale, absmax, q15 = fp.silu_mul_fwht_quant(dev(x), 128, want_q15=True)
    eq(host(q15), f); eq(host(codes), q); eq(host(scale), sc); eq(host(absmax), m)
    q0, s0, m0 = ofp.per_token_quant_from_q15(s)
    codes, scale, absmax, _ = fp.silu_mul_fwht_quant(dev(x), 0)
    eq(host(codes), q0); eq(host(absmax), m0)


def test_silu_large_magnitudes_and_odd_width(fp):
    rng = np.random.default_rng(11)
    x = rng.integers(-(2**31), 2**31, (4, 2 * 256), dtype=np.int64).astype(np.int32)
    s = ofp.silu_and_mul(x)
    eq(host(fp.silu_and_mul_int_only(dev(x))), s)
    codes, scale, absmax, q15 = fp.silu_mul_fwht_quant(dev(x), 128, want_q15=True)   # saturating butterflies
    f = ofp.blockwise_fwht_q15(s, 128)
    eq(host(q15), f)
    q, sc, m = ofp.per_token_quant_from_q15(f)
    eq(host(codes), q); eq(host(absmax), m)
    y = rng.integers(-(2**20), 2**20, (3, 2 * 36)).astype(np.int32)      # inter = 36: not a multiple of 128
    eq(host(fp.silu_and_mul_int_only(dev(y))), ofp.silu_and_mul(y))


@pytest.mark.parametrize("n", [2, 4, 16, 32, 64, 128, 256, 512, 1024])
def test_fwht_sizes_vs_oracle(fp, n):
    rng = np.random.default_rng(n)
    x = rng.integers(-(2**24), 2**24, (37, n)).astype(np.int32)
    eq(host(fp.fwht_int_q15(dev(x))), ofp.fwht_q15(x))
    eq(host(fp.fwht_int_q15(dev(x), normalize=False)), ofp.fwht_q15(x, False))
    big = rng.integers(-(2**31), 2**31, (5, n), dtype=np.int64).astype(np.int32)
    eq(host(fp.fwht_int_q15(dev(big))), ofp.fwht_q15(big))


def test_fwht_blockwise_equals_manual_view(fp):
    """tests/kernel/test_q15_layer_flow.py:145-161 of the reference, on the CUDA path."""
    x = torch.randint(-(2**20), 2**20, (4, 512), dtype=torch.int32, device="cuda")
    manual = fp.fwht_int_q15(x.view(-1, 4, 128)).view_as(x)
    assert torch.equal(fp.apply_blockwise_fwht_q15(x, 128), manual)
    eq(host(manual), ofp.blockwise_fwht_q15(host(x), 128))


def _rope_cache(max_pos=512, base=10000.0):
    inv = 1.0 / (base ** (torch.arange(0, 128, 2, dtype=torch.float) / 128))
    fr = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv)
    c = torch.cat((fr.cos(), fr.sin()), dim=-1)
    return torch.clamp(torch.round(c * 32768), -32768, 32767).to(torch.int32).numpy()


def test_rope_and_qk_norm_fused_vs_oracle(fp):
    rng = np.random.default_rng(2)
    T, Hq, Hk = 9, 8, 2
    cache = _rope_cache()
    pos = rng.integers(0, 512, T).astype(np.int32)
    qkv = rng.integers(-(2**22), 2**22, (T, (Hq + 2 * Hk) * 128)).astype(np.int32)
    q, k = qkv[:, : Hq * 128], qkv[:, Hq * 128 : (Hq + Hk) * 128]
    eq_, ek_ = ofp.rope_q15(pos, q.reshape(T, Hq, 128), k.reshape(T, Hk, 128), cache)
    dq = dev(qkv)
    q3 = dq[:, : Hq * 128].view(T, Hq, 128)                              # strided views into the qkv buffer
    k2 = dq[:, Hq * 128 : (Hq + Hk) * 128]
    gq, gk = fp.rope_int_q15(dev(pos), q3, k2, dev(cache))
    assert gq.shape == (T, Hq, 128) and gk.shape == (T, Hk * 128)      # 3-D in -> 3-D out, 2-D in -> 2-D out
    eq(host(gq), eq_); eq(host(gk).reshape(T, Hk, 128), ek_)
    with pytest.raises(ValueError, match="Ambiguous"):                  # as the reference: 2-D q and k of 1024 / 256
        fp.rope_int_q15(dev(pos), dq[:, : Hq * 128], k2, dev(cache))
    fq, fk = ofp.rope_fwht_q15(pos, q.reshape(T, Hq, 128), k.reshape(T, Hk, 128), cache)
    gq, gk = fp.rope_fwht_int_q15(dev(pos), dev(q.reshape(T, Hq, 128)), dev(k.reshape(T, Hk, 128)), dev(cache))
    eq(host(gq), fq); eq(host(gk), fk)
    qw = rng.integers(2**10, 2**14, 128).astype(np.int32)
    kw = rng.integers(2**13, 2**16, 128).astype(np.int32)
    nq = ofp.rmsnorm_v2(np.ascontiguousarray(q), qw).reshape(T, Hq, 128)
    nk = ofp.rmsnorm_v2(np.ascontiguousarray(k), kw).reshape(T, Hk, 128)
    fq, fk = ofp.rope_fwht_q15(pos, nq, nk, cache)
    gq, gk = fp.qk_norm_rope_fwht(dev(pos), q3, k2, dev(cache), dev(qw), dev(kw))
    eq(host(gq), fq); eq(host(gk).reshape(T, Hk, 128), fk)


@pytest.mark.parametrize("rows,k", [(1, 4), (5, 128), (3, 1000), (4, 5120), (2, 17408), (1, 32768)])
def test_quant_vs_oracle(fp, rows, k):
    rng = np.random.default_rng(k)
    x = rng.integers(-(2**26), 2**26, (rows, k)).astype(np.int32)
    x[0, : min(k, 3)] = 0
    q, s, m = ofp.per_token_quant_from_q15(x)
    gq, gs, gm = fp.per_token_quant_int8_from_q15(dev(x), return_absmax=True)
    eq(host(gq), q); eq(host(gs), s); eq(host(gm), m)
    from oracle.attention import absmax_to_mul_shift
    mul, sh = fp.absmax_to_mul_shift(gm)
    emul, esh = absmax_to_mul_shift(m)
    eq(host(mul), emul); eq(host(sh), esh)


def test_empty_inputs(fp):
    z = torch.zeros((0, 128), dtype=torch.int32, device="cuda")
    w = torch.ones(128, dtype=torch.int32, device="cuda")
    assert fp.rmsnorm_int_only_v2(z, w).shape == (0, 128)
    assert fp.fwht_int_q15(z).shape == (0, 128)
    assert fp.silu_and_mul_int_only(torch.zeros((0, 256), dtype=torch.int32, device="cuda")).shape == (0, 128)
    assert fp.per_token_quant_int8_from_q15(z)[0].shape == (0, 128)
    assert fp.to_fixed(torch.zeros(0, device="cuda")).numel() == 0


def test_zero_rows_and_canaries(fp):
    """All-zero rows stay zero and neighbouring memory is untouched."""
    x = torch.zeros((3, 1024), dtype=torch.int32, device="cuda")
    w = torch.full((1024,), 65536, dtype=torch.int32, device="cuda")
    assert int(fp.rmsnorm_int_only_v2(x, w).abs().max()) == 0
    codes, scale, absmax, _, _ = fp.fused_add_rmsnorm_quant(x, None, w)
    assert int(codes.abs().max()) == 0 and int(absmax.min()) == 1
    big = torch.full((5, 2 * 384), 7, dtype=torch.int32, device="cuda")
    mid = big[1:4]                                # rows 1..3 are the op's input; 0 and 4 are canaries
    out = fp.silu_and_mul_int_only(mid.contiguous())
    assert out.shape == (3, 384) and int(big[0].min()) == 7 and int(big[4].max()) == 7
