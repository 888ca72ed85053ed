"""One integer decoder layer on the CUDA kernels vs the oracle composition, bit-exact at every hand-off (int8
codes, Q15.16 tensors, and the pool contents).  The Qwen3-0.6B-shaped case: hidden 1024, 16 q / 8 kv heads,
head_dim 128, intermediate 3072, 64 new tokens = 16 per sequence over cached prefixes so that the sequences
reach 16 / 32 / 64 / 128 keys, page size 16, seed 0.  The Qwen3-8B-shaped case (hidden 4096, 32 q / 8 kv heads,
intermediate 12288) runs a few tokens so that the host oracle stays cheap."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import layer as olayer
from tests.layer_util import HID, HK, HQ, INTER, build, d, device_layer_weights, make_weights, rope_cache

pytestmark = pytest.mark.gpu


def _same(name, got, want):
    g = got.cpu().numpy().reshape(want.shape)
    assert g.dtype == want.dtype, (name, g.dtype, want.dtype)
    if not np.array_equal(g, want):
        bad = np.argwhere(g != want)
        raise AssertionError(f"{name}: {len(bad)} of {g.size} differ, first {bad[0]}: {g[tuple(bad[0])]} vs {want[tuple(bad[0])]}")


def _run_case(seed, kv_lens, q_lens, decode, hq, hk, hid, inter, num_pages, wide=False):
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger
    rng = np.random.default_rng(seed)
    T = sum(q_lens)
    w = make_weights(rng, hq, hk, hid, inter, wide)
    cache = rope_cache()
    ref_pool, pre, tables, table, positions, out_loc = build(rng, kv_lens, q_lens, num_pages, hk)
    x = np.clip(np.rint(rng.normal(0, 2**15, (T, hid))), -(2**23), 2**23).astype(np.int32)
    res = np.clip(np.rint(rng.normal(0, 2**15, (T, hid))), -(2**23), 2**23).astype(np.int32)

    want_x, want_res, wt = olayer.decoder_layer(x, res, w, cache, ref_pool, positions, out_loc, tables, kv_lens, q_lens, hq, hk)

    pool = Int8PagedKVCache(hk, 2, 128, num_pages, "cuda")
    for b, (k8, v8, km, ks, vm, vs, l) in pre.items():
        pool.store_codes(d(k8), d(v8), d(km), d(ks), d(vm), d(vs), d(l), 1)
    layer = Qwen3DecoderLayerInteger(1, hq, hk, hid, inter, device_layer_weights(w), d(cache), pool)
    batch = AttnBatch(d(positions), d(out_loc), d(table), d(np.asarray(kv_lens, np.int32)),
                      None if decode else d(np.asarray(q_lens, np.int32)), max(kv_lens))
    trace = {}
    got_x, got_res = layer.forward_q15(d(x), d(res), batch, trace)
    for name in ("ln1_codes", "qkv", "q_rot", "k_rot", "q8", "attn", "o", "ln2_codes", "res2", "gate_up", "act_codes", "down"):
        _same(name, trace[name], wt[name])
    _same("pool.k", pool.k_cache(1), ref_pool.k_codes); _same("pool.v", pool.v_cache(1), ref_pool.v_codes)
    _same("pool.meta", pool.meta(1), ref_pool.meta)
    _same("x_out", got_x, want_x); _same("residual_out", got_res, want_res)
    # the fused path (one launch between the qkv projection and attention, no intermediates kept) gives the same layer
    pool2 = Int8PagedKVCache(hk, 2, 128, num_pages, "cuda")
    for b, (k8, v8, km, ks, vm, vs, l) in pre.items():
        pool2.store_codes(d(k8), d(v8), d(km), d(ks), d(vm), d(vs), d(l), 1)
    layer2 = Qwen3DecoderLayerInteger(1, hq, hk, hid, inter, device_layer_weights(w), d(cache), pool2)
    fx, fres = layer2.forward_q15(d(x), d(res), batch)
    _same("x_out (fused path)", fx, want_x); _same("residual_out (fused path)", fres, want_res)
    _same("pool.k (fused path)", pool2.k_cache(1), ref_pool.k_codes); _same("pool.v (fused path)", pool2.v_cache(1), ref_pool.v_codes)
    _same("pool.meta (fused path)", pool2.meta(1), ref_pool.meta)
    # the down projection handed over pending: the next add + RMSNorm + quant finishes it, and so does materialise()
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    from mini_sgl_integer_b200.kernel.pending import PendingLinear, _workspaces
    px, pres = layer2.forward_q15(d(x), d(res), batch, defer_down=True)
    if T <= 256:
        assert isinstance(px, PendingLinear)
        got = fp.fused_add_rmsnorm_quant(px, pres, d(w["input_norm"]), want_norm=True)
        want = fp.fused_add_rmsnorm_quant(d(want_x), d(want_res), d(w["input_norm"]), want_norm=True)
        for name, g, wv in zip(("codes", "scale", "absmax", "residual", "norm"), got, want):
            assert torch.equal(g, wv), f"pending down -> norm: {name}"
        px, _ = layer2.forward_q15(d(x), d(res), batch, defer_down=True)
        _same("x_out (materialised)", px.materialise(), want_x)
        assert all(int(b.abs().max()) == 0 for b in _workspaces.values())        # every workspace is zero again
    else:
        _same("x_out (defer_down at a size that is not deferred)", px, want_x)
    assert np.abs(want_x).max() > 0 and np.abs(wt["attn"]).max() > 0
    assert np.abs(want_x).max() < 2**31 - 1           # the case exercises the arithmetic, not the saturation rails


@pytest.mark.parametrize("mode", ["extend", "decode"])
def test_decoder_layer_bit_exact(mode):
    kv_lens = [16, 32, 64, 128]
    q_lens = [16, 16, 16, 16] if mode == "extend" else [1, 1, 1, 1]
    _run_case(0, kv_lens, q_lens, mode == "decode", HQ, HK, HID, INTER, 32)


@pytest.mark.parametrize("mode", ["extend", "decode"])
def test_decoder_layer_8b_shape_bit_exact(mode):
    """hidden 4096, 32 q / 8 kv heads, intermediate 12288: the layer of the 8B-shaped model, on a few tokens."""
    kv_lens = [5, 40, 17, 130, 64, 33]
    q_lens = [2, 1, 3, 1, 1, 2] if mode == "extend" else [1] * 6
    _run_case(3, kv_lens, q_lens, mode == "decode", 32, 8, 4096, 12288, 40, wide=True)


def test_decoder_layer_with_silu_in_the_gate_up_epilogue(monkeypatch):
    """The optional form that applies SiLU * up in the gate_up GEMM's epilogue (off by default): the same layer bits."""
    from mini_sgl_integer_b200.layers import decoder_layer
    monkeypatch.setattr(decoder_layer, "_GATE_UP_SILU_ON", True)
    _run_case(0, [16, 32, 64, 128], [1, 1, 1, 1], True, HQ, HK, HID, INTER, 32)
    _run_case(3, [5, 40, 17, 130, 64, 33], [2, 1, 3, 1, 1, 2], False, 32, 8, 4096, 12288, 40, wide=True)
