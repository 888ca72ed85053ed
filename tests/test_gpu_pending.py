"""Linears whose requantisation is left to the consuming row kernel: the split-K GEMM that adds into a workspace kept
zero, add + RMSNorm + quant and the q/k/v preparation reading exact accumulators.  Each must give the bits of the
materialised path (itself checked against the oracle elsewhere) and of the oracle, and leave the workspace zero."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import fixed_point as ofp
from oracle import linear as olin

pytestmark = pytest.mark.gpu


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _linear_case(seed, m, n, k, shift=True):
    rng = np.random.default_rng(seed)
    x = np.clip(np.rint(rng.normal(0, 2**16, (m, k))), -(2**24), 2**24).astype(np.int32)
    if m > 2:
        x[1, :] = 0
    w8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
    wm = rng.integers(2**29, 2**30, n).astype(np.int32)
    ws = rng.integers(31, 35, n).astype(np.int32) if shift else None
    codes, _, absmax = ofp.per_token_quant_from_q15(x)
    xm, xs = oattn.absmax_to_mul_shift(absmax.reshape(-1))
    acc = olin.int32_accumulate(codes, w8)
    q15 = olin.requant_q15(acc, xm, xs, wm, ws if ws is not None else np.full(n, 31, np.int32))
    return codes, absmax.reshape(-1).astype(np.int32), w8, wm, ws, acc, q15


def _layer(w8, wm, ws):
    from mini_sgl_integer_b200.layers.decoder_layer import _Linear
    return _Linear(d(w8), weight_mul=d(wm), weight_shift=None if ws is None else d(ws))


def _workspaces_zero():
    from mini_sgl_integer_b200.kernel.pending import _workspaces
    return all(int(b.abs().max()) == 0 for b in _workspaces.values())


# (m, n, k): every K-split shape of the decode GEMM (few weight blocks -> deep splits; more blocks than SMs ->
# unsplit waves plus a split tail; one block), ragged n, and sizes where nothing is split
SHAPES = [(1, 256, 512), (33, 1028, 1024), (256, 4096, 4096), (200, 6144, 4096), (64, 148 * 128 + 384, 2048), (256, 128, 8192)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_linear_with_zero_workspace_equals_the_plain_linear(m, n, k):
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod, int8_gemm_q15
    codes, absmax, w8, wm, ws, acc, q15 = _linear_case(m + n, m, n, k)
    layer, meth = _layer(w8, wm, ws), W8A8Int8LinearMethod()
    for _ in range(3):                                                # the workspace is reused: it must be zero again
        got = meth.apply_quantised(layer, d(codes), d(absmax))
        np.testing.assert_array_equal(got.cpu().numpy(), q15)
        assert _workspaces_zero()
    plain = int8_gemm_q15(d(codes), None, None, layer.weight, layer.weight_mul, layer.weight_shift, x_absmax=d(absmax))
    assert torch.equal(plain, got)


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("with_residual", [True, False])
def test_rmsnorm_on_a_pending_linear(m, n, k, with_residual):
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    from mini_sgl_integer_b200.kernel.pending import PendingLinear
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod
    codes, absmax, w8, wm, ws, acc, q15 = _linear_case(2 * m + n, m, n, k, shift=(m != 33))
    rng = np.random.default_rng(5)
    res = np.clip(np.rint(rng.normal(0, 2**15, (m, n))), -(2**23), 2**23).astype(np.int32) if with_residual else None
    nw = rng.integers(2**12, 2**15, n).astype(np.int32)
    layer, meth = _layer(w8, wm, ws), W8A8Int8LinearMethod()
    want = fp.fused_add_rmsnorm_quant(d(q15), None if res is None else d(res), d(nw), want_norm=True)
    # the oracle on the same row: add, fixed-point RMSNorm, quant
    summed = q15 if res is None else (q15.astype(np.int64) + res).astype(np.int32)
    o_norm = ofp.rmsnorm_v2(summed, nw)
    np.testing.assert_array_equal(want[4].cpu().numpy(), o_norm)
    for _ in range(2):
        pend = meth.apply_pending(layer, d(codes), d(absmax))
        assert isinstance(pend, PendingLinear) and tuple(pend.shape) == (m, n)
        np.testing.assert_array_equal(pend.acc.cpu().numpy(), acc)       # the exact accumulators
        got = fp.fused_add_rmsnorm_quant(pend, None if res is None else d(res), d(nw), want_norm=True)
        for name, g, wv in zip(("codes", "scale", "absmax", "residual", "norm"), got, want):
            assert (g is None and wv is None) or torch.equal(g, wv), name
        assert _workspaces_zero()
    pend = meth.apply_pending(layer, d(codes), d(absmax))
    np.testing.assert_array_equal(pend.materialise().cpu().numpy(), q15)
    assert _workspaces_zero()


@pytest.mark.parametrize("tokens,hq,hk", [(1, 4, 1), (37, 16, 8), (256, 32, 8)])
def test_qkv_preparation_on_a_pending_linear(tokens, hq, hk):
    """q/k-norm, RoPE, rotation, pool store and q quant from the qkv accumulators: the bits of the same step on the
    materialised qkv tensor (pool contents, q codes and scales); out-of-pool locations are dropped and still cleared."""
    from mini_sgl_integer_b200.attention import Int8PagedKVCache, qkv_rope_quant_store
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod
    from tests.layer_util import rope_cache
    n, k = (hq + 2 * hk) * 128, 1024
    codes, absmax, w8, wm, ws, acc, q15 = _linear_case(tokens * 7 + hq, tokens, n, k)
    rng = np.random.default_rng(tokens)
    num_pages = (tokens + 15) // 16 + 2
    out_loc = rng.permutation(num_pages * 16)[:tokens].astype(np.int32)
    if tokens > 4:
        out_loc[3] = -1                                                # dropped
        out_loc[4] = num_pages * 16 + 5                                # outside the pool: dropped
    positions = rng.integers(0, 200, tokens).astype(np.int32)
    cache = d(rope_cache())
    qn, kn = d(rng.integers(2**11, 2**13, 128).astype(np.int32)), d(rng.integers(2**12, 2**14, 128).astype(np.int32))
    layer, meth = _layer(w8, wm, ws), W8A8Int8LinearMethod()
    pool_a = Int8PagedKVCache(hk, 1, 128, num_pages, "cuda")
    pool_b = Int8PagedKVCache(hk, 1, 128, num_pages, "cuda")
    want = qkv_rope_quant_store(d(positions), d(q15), hq, pool_a, 0, d(out_loc), cache, qn, kn)
    pend = meth.apply_pending(layer, d(codes), d(absmax))
    got = qkv_rope_quant_store(d(positions), pend, hq, pool_b, 0, d(out_loc), cache, qn, kn)
    for name, g, wv in zip(("q8", "q_mul", "q_shift"), got, want):
        assert torch.equal(g, wv), name
    assert torch.equal(pool_a.k_cache(0), pool_b.k_cache(0)) and torch.equal(pool_a.v_cache(0), pool_b.v_cache(0))
    assert torch.equal(pool_a.meta(0), pool_b.meta(0))
    assert _workspaces_zero()


def test_a_pending_linear_that_nobody_consumed_is_cleared_by_reset():
    from mini_sgl_integer_b200.kernel.pending import reset_workspaces, workspace_scope
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod
    codes, absmax, w8, wm, ws, acc, q15 = _linear_case(3, 40, 512, 1024)
    layer, meth = _layer(w8, wm, ws), W8A8Int8LinearMethod()
    with workspace_scope("scratch"):                         # a buffer set of its own: the default one stays clean
        pend = meth.apply_pending(layer, d(codes), d(absmax))
        assert int(pend.acc.abs().max()) > 0 and not _workspaces_zero()
    reset_workspaces()
    assert _workspaces_zero()
    np.testing.assert_array_equal(meth.apply_quantised(layer, d(codes), d(absmax)).cpu().numpy(), q15)


@pytest.mark.parametrize("m,inter,k,block", [(1, 128, 256, 128), (65, 3072, 1024, 128), (200, 12288, 4096, 128), (256, 12288, 4096, 128),
                                            (33, 9472 + 128, 512, 128), (256, 1536, 2048, 0), (130, 256, 8192, 128)])
def test_gate_up_with_silu_in_the_epilogue(m, inter, k, block):
    """gate_up GEMM with SiLU(gate) * up in its epilogue, then rotation + quant: the bits of the unfused chain (GEMM,
    then the SiLU row kernel) and of the oracle.  Shapes with only whole blocks, with a split tail (96 blocks on 74 CTA
    pairs), with fewer blocks than pairs (deep splits) and with a single block."""
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod
    codes, absmax, w8, wm, ws, acc, q15 = _linear_case(m + inter + k, m, 2 * inter, k)
    layer, meth = _layer(w8, wm, ws), W8A8Int8LinearMethod()
    assert meth.can_fuse_gate_up_silu(layer, m)
    want_act = ofp.silu_and_mul(q15)
    want_rot = ofp.blockwise_fwht_q15(want_act, block) if block else want_act
    want_codes, _, want_absmax = ofp.per_token_quant_from_q15(want_rot)
    for _ in range(2):
        act = meth.apply_gate_up_silu(layer, d(codes), d(absmax))
        np.testing.assert_array_equal(act.cpu().numpy(), want_act)
        assert _workspaces_zero()
        got_codes, got_scale, got_absmax = fp.fwht_quant_q15(act, block)
        np.testing.assert_array_equal(got_codes.cpu().numpy(), want_codes)
        np.testing.assert_array_equal(got_absmax.cpu().numpy().reshape(-1), want_absmax.reshape(-1))
    ref = fp.silu_mul_fwht_quant(meth.apply_quantised(layer, d(codes), d(absmax)), block)
    assert torch.equal(ref[0], got_codes) and torch.equal(ref[1], got_scale) and torch.equal(ref[2], got_absmax)
