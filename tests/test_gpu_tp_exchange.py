"""The tensor-parallel exchange kernels on ONE GPU: the calls of 2, 4 or 8 ranks are issued one after the other on
one stream over exchange blocks that all live on this device, so every wait finds its flags already set.  The
row-split linear must give the bits of the unsplit linear (the oracle's), repeatedly (both halves of the blocks
get reused and cleared), and a wait that nothing satisfies must end by itself with a status code."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import fixed_point as ofp
from oracle import linear as olin

pytestmark = pytest.mark.gpu


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _case(seed, m, n, k):
    rng = np.random.default_rng(seed)
    x = np.clip(np.rint(rng.normal(0, 2**16, (m, k))), -(2**24), 2**24).astype(np.int32)
    x[0, :] = 0                                                     # an all-zero row: absmax 1
    w8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
    wm = rng.integers(2**29, 2**30, n).astype(np.int32)
    ws = rng.integers(30, 34, n).astype(np.int32)
    codes, _, absmax = ofp.per_token_quant_from_q15(x)
    xm, xs = oattn.absmax_to_mul_shift(absmax.reshape(-1))
    want = olin.requant_q15(olin.int32_accumulate(codes, w8), xm, xs, wm, ws)
    return x, w8, wm, ws, want


@pytest.mark.parametrize("size", [1, 2, 4, 8])
@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (33, 1028, 1024), (256, 1024, 2048), (8, 5120, 8192)])
def test_row_split_linear_over_exchange_blocks(size, m, n, k):
    """The last shape is the o-projection of the 32B-shaped model (hidden 5120, 64 x 128 input features) on 8 tokens."""
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    x, w8, wm, ws, want = _case(size * 1000 + m, m, n, k)
    ks = k // size
    ranks = TpExchange.emulated(size, 256, n)
    xs_ = [d(x[:, r * ks:(r + 1) * ks]) for r in range(size)]
    w_ = [d(w8[:, r * ks:(r + 1) * ks]) for r in range(size)]
    wm_d, ws_d = d(wm), d(ws)
    for rnd in range(3):
        for r in range(size):
            ranks[r].absmax_put(xs_[r])
        q = [ranks[r].quant_wait(xs_[r]) for r in range(size)]
        for r in range(size):
            ranks[r].gemm_add(q[r][0], w_[r])
        if ranks[0].direct:
            outs = [ranks[r].requant_direct(q[r][1], wm_d, ws_d) for r in range(size)]
        else:
            for r in range(size):
                ranks[r].requant_scatter(q[r][1], wm_d, ws_d)
            outs = [ranks[r].collect(m, "cuda") for r in range(size)]
        for r in range(size):
            np.testing.assert_array_equal(outs[r].cpu().numpy(), want, err_msg=f"round {rnd}, rank {r}")
    assert TpExchange.status() == 0
    # the absmax words have been cleared again, and so has the accumulator half of the exchange before the last one
    words = ranks[0].nbytes // 4
    half = (256 * n + 63) // 64 * 64
    for r in range(size):
        body = ranks[r]._buf[r].view(torch.int32)
        assert int(body[128:words - 4 * half].abs().max()) == 0              # everything in front of the accumulators
        acc = body[words - 4 * half: words - 2 * half].view(2, half)
        assert int(acc[0].abs().max()) == 0 or int(acc[1].abs().max()) == 0


@pytest.mark.parametrize("size", [1, 2, 4, 8])
@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (33, 1040, 1024), (256, 4096, 2048), (8, 5120, 8192), (5, 8192 + 64, 512)])
def test_row_split_linear_finished_and_normalised_by_row_owners(size, m, n, k):
    """The row-split linear fused with the residual add + RMSNorm + quant that follows it: every token row is finished
    by one owner rank, all ranks receive the codes and the absmax of all rows (the oracle's bits), and an owner's
    residual rows are updated in place.  Three rounds reuse and clear both halves of the blocks."""
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    x, w8, wm, ws, lin = _case(size * 77 + m, m, n, k)
    rng = np.random.default_rng(n + size)
    res = np.clip(np.rint(rng.normal(0, 2**15, (m, n))), -(2**23), 2**23).astype(np.int32)
    nw = rng.integers(2**11, 2**15, n).astype(np.int32)
    norm, summed = ofp.fused_add_rmsnorm_v2(res, lin, nw)
    want_codes, _, want_absmax = ofp.per_token_quant_from_q15(norm)
    ks = k // size
    ranks = TpExchange.emulated(size, 256, n)
    xs_ = [d(x[:, r * ks:(r + 1) * ks]) for r in range(size)]
    w_ = [d(w8[:, r * ks:(r + 1) * ks]) for r in range(size)]
    wm_d, ws_d, nw_d = d(wm), d(ws), d(nw)
    for rnd in range(3):
        resid = [d(res) for _ in range(size)]
        for r in range(size):
            ranks[r].absmax_put(xs_[r])
        q = [ranks[r].quant_wait(xs_[r]) for r in range(size)]
        for r in range(size):
            ranks[r].gemm_add(q[r][0], w_[r])
        for r in range(size):
            ranks[r].owner_norm(q[r][1], wm_d, ws_d, resid[r], nw_d)
        for r in range(size):
            codes, absmax = ranks[r].collect_codes(m, "cuda")
            np.testing.assert_array_equal(codes.cpu().numpy(), want_codes, err_msg=f"codes, round {rnd}, rank {r}")
            np.testing.assert_array_equal(absmax.cpu().numpy(), want_absmax.reshape(-1), err_msg=f"absmax, round {rnd}, rank {r}")
            own = ranks[r].owner_rows(m)
            np.testing.assert_array_equal(resid[r][own].cpu().numpy(), summed[own], err_msg=f"residual, round {rnd}, rank {r}")
            other = np.ones(m, bool); other[own] = False
            np.testing.assert_array_equal(resid[r].cpu().numpy()[other], res[other])       # the other rows are not touched
    assert TpExchange.status() == 0
    # without a residual: the norm of the linear's output alone
    norm0 = ofp.rmsnorm_v2(lin, nw)
    c0, _, a0 = ofp.per_token_quant_from_q15(norm0)
    for r in range(size):
        ranks[r].absmax_put(xs_[r])
    q = [ranks[r].quant_wait(xs_[r]) for r in range(size)]
    for r in range(size):
        ranks[r].gemm_add(q[r][0], w_[r])
    for r in range(size):
        ranks[r].owner_norm(q[r][1], wm_d, ws_d, None, nw_d)
    codes, absmax = ranks[size - 1].collect_codes(m, "cuda")
    np.testing.assert_array_equal(codes.cpu().numpy(), c0)
    np.testing.assert_array_equal(absmax.cpu().numpy(), a0.reshape(-1))
    assert TpExchange.status() == 0


@pytest.mark.parametrize("size", [1, 3])
@pytest.mark.parametrize("rows,inter,block", [(5, 256, 128), (64, 3072, 128), (9, 1536, 0), (3, 12288, 128)])
def test_silu_fused_with_the_absmax_agreement(size, rows, inter, block):
    """SiLU * up + rotation + agreement + quant in one launch.  The ranks' calls are issued one after the other, so
    only the LAST rank's kernel finds every rank's word (the earlier ones run into a short time limit); its codes
    must be the oracle's codes of its slice under the maximum of all slices' absmax."""
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    rng = np.random.default_rng(rows + inter + size)
    gus = [np.clip(np.rint(rng.normal(0, 2**17, (rows, 2 * inter))), -(2**22), 2**22).astype(np.int32) for _ in range(size)]
    gus[0][:, :] //= 7                                    # one rank with clearly smaller values
    acts = []
    for gu in gus:
        a = ofp.silu_and_mul(gu)
        acts.append(ofp.blockwise_fwht_q15(a, block) if block else a)
    agreed = np.maximum(1, np.max([np.abs(a.astype(np.int64)).max(axis=1) for a in acts], axis=0)).astype(np.int32)
    last = size - 1
    # the oracle's per-token quant of the row [own slice | a column holding the agreed absmax]
    want = ofp.per_token_quant_from_q15(np.concatenate([acts[last], agreed.reshape(-1, 1)], axis=1))[0][:, :-1]
    for rnd in range(2):
        ranks = TpExchange.emulated(size, 64, 256)        # fresh blocks: the early ranks leave stale words behind
        TpExchange.set_timeout_us(2000)
        try:
            outs = [ranks[r].silu_absmax_quant(d(gus[r]), block) for r in range(size)]
            torch.cuda.synchronize()
        finally:
            TpExchange.set_timeout_us(2_000_000)
        codes, absmax = outs[last]
        np.testing.assert_array_equal(absmax.cpu().numpy(), agreed)
        np.testing.assert_array_equal(codes.cpu().numpy(), want)
    assert TpExchange.status() == (1 if size > 1 else 0)   # the early ranks' waits ran out (channel 0)
    assert TpExchange.status() == 0


def test_single_rank_exchange_equals_the_plain_linear():
    """size 1 through the calls the layers make (absmax + quant in one launch): the plain linear's bits."""
    from mini_sgl_integer_b200.layers.decoder_layer import _Linear
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod
    x, w8, wm, ws, want = _case(5, 200, 512, 8192 + 1024)            # rows longer than a CTA keeps in registers
    ex = TpExchange.emulated(1, 256, 512)[0]
    layer = _Linear(d(w8), weight_mul=d(wm), weight_shift=d(ws))
    for _ in range(3):
        got = ex.row_parallel_q15(W8A8Int8LinearMethod(), layer, d(x))
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert TpExchange.status() == 0


def test_all_gather_over_exchange_blocks():
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    size, words = 4, 37
    ranks = TpExchange.emulated(size, 32, 64)
    rng = np.random.default_rng(1)
    for rnd in range(3):
        src = rng.integers(-2**31, 2**31, (size, words), dtype=np.int64).astype(np.int32)
        # a rank's gather kernel signals and then waits for everybody: with the ranks emulated one after the other
        # only the LAST rank's call finds all slots filled, so the earlier calls are issued with a short time limit
        TpExchange.set_timeout_us(2000)
        outs = [ranks[r].all_gather(d(src[r])) for r in range(size)]
        torch.cuda.synchronize()
        np.testing.assert_array_equal(outs[size - 1].cpu().numpy(), src, err_msg=f"round {rnd}")
    assert TpExchange.status() == 3                                   # the early ranks' waits ran out (channel 2)
    TpExchange.set_timeout_us(2_000_000)
    assert TpExchange.status() == 0


def test_wait_that_nothing_satisfies_ends_with_a_status():
    """Rank 0 of two: its peer never signals.  The consumer kernel gives up after the time limit, the context stays
    usable, and the status word names the channel."""
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    ranks = TpExchange.emulated(2, 16, 64)
    x = d(np.arange(16 * 64, dtype=np.int32).reshape(16, 64))
    TpExchange.set_timeout_us(20_000)
    try:
        ranks[0].absmax_put(x)
        codes, absmax = ranks[0].quant_wait(x)
        torch.cuda.synchronize()
        assert TpExchange.status() == 1
        assert TpExchange.status() == 0                              # cleared by the read above
        assert codes.shape == (16, 64) and int(absmax[15]) == 16 * 64 - 1   # rank 0's own maxima were there
    finally:
        TpExchange.set_timeout_us(2_000_000)


@pytest.mark.parametrize("n_peers", [1, 2])
@pytest.mark.parametrize("m,n,k", [(1, 384, 512), (33, 1028, 1024), (256, 4096, 2048)])
def test_gemm_reduce_peers_adds_into_every_buffer(n_peers, m, n, k):
    """b200_gemm_w8a8_reduce_peers with the peers' accumulators on this device: every buffer receives the exact
    int32 accumulators once per call (split and unsplit tiles, ragged n), also on top of earlier contents."""
    from mini_sgl_integer_b200._lib import call, ptr, stream
    rng = np.random.default_rng(7 * m + n_peers)
    x8 = rng.integers(-127, 128, (m, k), dtype=np.int8)
    w8 = rng.integers(-127, 128, (n, k), dtype=np.int8)
    acc = olin.int32_accumulate(x8, w8)
    bufs = [torch.zeros((m, n), dtype=torch.int32, device="cuda") for _ in range(n_peers)]
    arr = (ctypes.c_void_p * n_peers)(*[b.data_ptr() for b in bufs])
    xd, wd = d(x8), d(w8)
    for rnd in range(3):
        call("b200_gemm_w8a8_reduce_peers", ptr(xd), ptr(wd), arr, n_peers, m, n, k, stream())
        for b in bufs:
            np.testing.assert_array_equal(b.cpu().numpy(), acc * (rnd + 1))
    st = ctypes.c_int(0)
    call("b200_gemm_status", ctypes.byref(st), 1)
    assert st.value == 0
