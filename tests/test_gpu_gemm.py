"""tcgen05 int8 GEMM + fixed-point epilogue vs the CPU oracle (exact int32 accumulators, bit-exact Q15.16)."""
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


def gemm_status(reset=True):
    from mini_sgl_integer_b200 import _lib
    v = ctypes.c_int(0)
    _lib.call("b200_gemm_status", ctypes.cast(ctypes.pointer(v), ctypes.c_void_p), int(reset))
    return v.value


def run_case(M, N, K, seed, per_channel_shift=False):
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    rng = np.random.default_rng(seed)
    x8 = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    x_mul = rng.integers(2**30, 2**31, M).astype(np.int32)
    x_shift = rng.integers(36, 44, M).astype(np.int32)
    w_mul = rng.integers(2**29, 2**30, N).astype(np.int32)
    w_shift = rng.integers(31, 39, N).astype(np.int32) if per_channel_shift else None
    out, acc = int8_gemm_q15(d(x8), d(x_mul), d(x_shift), d(w8), d(w_mul), None if w_shift is None else d(w_shift),
                             want_acc=True)
    torch.cuda.synchronize()
    assert gemm_status() == 0
    want_acc = olin.int32_accumulate(x8, w8)
    assert np.array_equal(acc.cpu().numpy(), want_acc), "int32 accumulators differ"
    want = olin.requant_q15(want_acc, x_mul, x_shift, w_mul, np.full(N, 31) if w_shift is None else w_shift)
    got = out.cpu().numpy()
    if not np.array_equal(got, want):
        bad = np.argwhere(got != want)
        raise AssertionError(f"{len(bad)} mismatches, first {bad[0]}: {got[tuple(bad[0])]} vs {want[tuple(bad[0])]}")


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 128, 512), (64, 256, 1024), (1, 128, 256), (200, 384, 2048),
                                   (130, 200, 144), (64, 4096, 1024), (64, 1024, 3072), (256, 6144, 1024),
                                   (48, 24576, 512), (100, 19240, 1024)])   # more weight blocks than SMs: split tail
def test_gemm_vs_oracle(M, N, K):
    run_case(M, N, K, M + N + K)


@pytest.mark.parametrize("M,N,K", [(256, 4096, 12288), (33, 1024, 3072), (129, 6144, 4096), (7, 200, 2064), (256, 24576, 1024),
                                   (64, 24576, 1024), (17, 19240, 2048)])
def test_decode_sizes_without_accumulator_output(M, N, K):
    """M <= 256 runs weights-stationary with K split over CTAs; with only the Q15.16 output requested the
    partial sums are gathered in that buffer and requantised in place."""
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    rng = np.random.default_rng(M * 7 + N + K)
    x8 = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    x_mul = rng.integers(2**30, 2**31, M).astype(np.int32)
    x_shift = rng.integers(36, 44, M).astype(np.int32)
    w_mul = rng.integers(2**29, 2**30, N).astype(np.int32)
    w_shift = rng.integers(31, 39, N).astype(np.int32)
    want = olin.requant_q15(olin.int32_accumulate(x8, w8), x_mul, x_shift, w_mul, w_shift)
    for _ in range(2):                                     # the second call finds the buffer dirty
        out = int8_gemm_q15(d(x8), d(x_mul), d(x_shift), d(w8), d(w_mul), d(w_shift))
        torch.cuda.synchronize()
        assert gemm_status() == 0
        np.testing.assert_array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("M,N,K", [(256, 24576, 4096), (200, 19208, 2048), (129, 132, 512), (256, 256, 8192), (177, 6144, 4096),
                                   (65, 4096, 4096), (100, 6144, 1024), (128, 19208, 512)])
def test_pair_weights_stationary_tiles(M, N, K):
    """65..256 tokens run on CTA pairs over blocks of 256 weight rows with half of the tokens staged per CTA: unsplit
    waves followed by a split tail, a ragged last block, a single block with the deepest split, both outputs."""
    run_case(M, N, K, M + N + K, per_channel_shift=True)


@pytest.mark.parametrize("M,N,K", [(300, 512, 1024), (64, 1024, 2048), (256, 20000, 256)])
def test_token_scale_from_absmax(M, N, K):
    """The entry point that takes the row kernels' integer absmax derives the same (multiplier, shift)."""
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    rng = np.random.default_rng(M + N + K)
    x8 = rng.integers(-127, 128, (M, K), dtype=np.int8)
    w8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    absmax = rng.integers(1, 2**24, M).astype(np.int32)
    absmax[0], absmax[1] = 1, 2**31 - 1
    w_mul = rng.integers(2**29, 2**30, N).astype(np.int32)
    w_shift = rng.integers(31, 39, N).astype(np.int32)
    x_mul, x_shift = oattn.absmax_to_mul_shift(absmax)
    want = olin.requant_q15(olin.int32_accumulate(x8, w8), x_mul, x_shift, w_mul, w_shift)
    out = int8_gemm_q15(d(x8), None, None, d(w8), d(w_mul), d(w_shift), x_absmax=d(absmax))
    torch.cuda.synchronize()
    assert gemm_status() == 0
    np.testing.assert_array_equal(out.cpu().numpy(), want)


@pytest.mark.parametrize("M,N,K", [(2304, 2304, 256), (2050, 2400, 1040), (4096, 1280, 2048)])
def test_two_cta_tiles(M, N, K):
    """Problems with at least one 256 x 256 tile per CTA pair run on tcgen05.mma.cta_group::2 (ragged edges,
    k-blocks that wrap the stage ring several times)."""
    run_case(M, N, K, M + N + K, per_channel_shift=True)


def test_gemm_per_channel_shifts_and_deep_k():
    run_case(96, 256, 12288, 7, per_channel_shift=True)


def test_gemm_extreme_codes_do_not_overflow():
    """K = 25600 of +-127 products: |acc| = 4.1e8 < 2**31, accumulators must be exact."""
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    M, N, K = 32, 128, 25600
    x8 = np.full((M, K), 127, dtype=np.int8); x8[1::2] = -127
    w8 = np.full((N, K), 127, dtype=np.int8); w8[::3] = -127
    acc = int8_gemm_q15(d(x8), None, None, d(w8), None, want_q15=False, want_acc=True)
    assert np.array_equal(acc.cpu().numpy(), olin.int32_accumulate(x8, w8))
    assert gemm_status() == 0


def test_linear_method_matches_oracle_and_float_reference():
    """apply_weights_q15: codes as the reference's per-token quant, accumulators exact, integer epilogue;
    the result stays within the reference's own tolerance (cosine > 0.999) of its float path."""
    from mini_sgl_integer_b200.layers import W8A8Int8LinearMethod
    rng = np.random.default_rng(3)
    T, K, N = 64, 1024, 4096
    x = np.clip(np.rint(rng.normal(0, 2**15, (T, K))), -(2**23), 2**23).astype(np.int32)
    w8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    w_scale = rng.uniform(0.002, 0.02, (N, 1)).astype(np.float32)

    class Layer(torch.nn.Module):
        pass
    layer = Layer()
    layer.weight = d(w8)
    layer.weight_scale = d(w_scale)
    method = W8A8Int8LinearMethod()
    got = method.apply_weights_q15(layer, d(x)).cpu().numpy()

    codes, scale, absmax = ofp.per_token_quant_from_q15(x)
    x_mul, x_shift = oattn.absmax_to_mul_shift(absmax[:, 0])
    w_mul, w_shift = olin.weight_scale_to_mul_shift(w_scale)
    assert np.array_equal(layer.weight_mul.cpu().numpy(), w_mul) and np.array_equal(layer.weight_shift.cpu().numpy(), w_shift)
    want = olin.requant_q15(olin.int32_accumulate(codes, w8), x_mul, x_shift, w_mul, w_shift)
    assert np.array_equal(got, want)
    ref = olin.linear_q15_float_reference(codes, scale, w8, w_scale).astype(np.float64).reshape(-1)
    g = got.astype(np.float64).reshape(-1)
    cos = float(g @ ref / (np.linalg.norm(g) * np.linalg.norm(ref)))
    assert cos > 0.999999, cos
    assert np.abs(g - ref).max() <= 4 + 1e-6 * np.abs(ref).max()


def test_gemm_empty_and_bad_k():
    from mini_sgl_integer_b200 import _lib
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    w8 = torch.zeros((128, 256), dtype=torch.int8, device="cuda")
    out = int8_gemm_q15(torch.zeros((0, 256), dtype=torch.int8, device="cuda"), None, None, w8, None,
                        want_q15=False, want_acc=True)
    assert out.shape == (0, 128)
    with pytest.raises(_lib.B200Error, match="multiple of 16"):
        int8_gemm_q15(torch.zeros((4, 24), dtype=torch.int8, device="cuda"), None, None,
                      torch.zeros((8, 24), dtype=torch.int8, device="cuda"), None, want_q15=False, want_acc=True)


def test_static_input_scale_path(golden):
    """Checkpoints with an `input_scale`: the reference's static codes, then the GEMM with one token scale."""
    from mini_sgl_integer_b200.layers import W8A8Int8LinearMethod
    from mini_sgl_integer_b200.layers.w8a8_int8 import per_tensor_quant_int8_static_from_q15, weight_scale_to_mul_shift
    x = golden["static_in"]
    for i, scale in enumerate(golden["static_scales"]):
        got = per_tensor_quant_int8_static_from_q15(d(x), torch.tensor([scale], dtype=torch.float32).cuda())
        np.testing.assert_array_equal(got.cpu().numpy(), golden[f"static_codes_{i}"])
    rng = np.random.default_rng(12)
    N, K = 256, x.shape[1]
    layer = torch.nn.Module()
    layer.weight = d(rng.integers(-127, 128, (N, K), dtype=np.int8))
    layer.weight_scale = d(rng.uniform(1e-3, 3e-2, (N, 1)).astype(np.float32))
    layer.input_scale = torch.tensor([0.05], dtype=torch.float32).cuda()
    out = W8A8Int8LinearMethod().apply_weights_q15(layer, d(x))
    torch.cuda.synchronize()
    assert gemm_status() == 0
    codes = ofp.static_quant_from_q15(x, np.float32(0.05))
    w_mul, w_shift = olin.weight_scale_to_mul_shift(layer.weight_scale.cpu().numpy().reshape(-1))
    x_mul, x_shift = olin.weight_scale_to_mul_shift(np.array([0.05], dtype=np.float32))
    want = olin.requant_q15(olin.int32_accumulate(codes, layer.weight.cpu().numpy()), np.repeat(x_mul, x.shape[0]),
                            np.repeat(x_shift, x.shape[0]), w_mul, w_shift)
    np.testing.assert_array_equal(out.cpu().numpy(), want)
    # sanity against the float formula of the reference's fallback (w8a8_int8.py:280-284)
    ref = (codes.astype(np.float64) * 0.05) @ (layer.weight.cpu().numpy().astype(np.float64) * layer.weight_scale.cpu().numpy().astype(np.float64)).T
    err = np.abs(out.cpu().numpy() / 65536.0 - ref).max()
    assert err < 2e-3 * max(1.0, np.abs(ref).max()), err
