"""numpy restatement of the reference's Q15.16 fixed-point ops (TEST INFRASTRUCTURE ONLY).

Each function follows the reference file:line named in its docstring.  All
arithmetic is done in explicit numpy integer types so that int32 / int64
wrap-around happens exactly where the reference's kernels wrap.
"""
from __future__ import annotations

import math

import numpy as np

from . import luts

I32_MIN = -(1 << 31)
I32_MAX = (1 << 31) - 1
FIXED_POINT_SCALE = 1 << 16


# --------------------------------------------------------------------------- helpers
def _wrap32(a64: np.ndarray) -> np.ndarray:
    """Keep the low 32 bits of an int64 array, as int32 (two's-complement wrap)."""
    return np.asarray(a64, dtype=np.int64).astype(np.int32)


def msb(v: np.ndarray) -> np.ndarray:
    """Index of the leading one of a positive integer (0 for v == 1).

    The reference gets this number from a de-Bruijn multiply
    (kernel/fixed_point/rmsnorm_int_only_v2.py:63-86); for 1 <= v < 2**31 that
    table returns exactly floor(log2 v).
    """
    v = np.asarray(v, dtype=np.int64)
    out = np.zeros(v.shape, dtype=np.int32)
    t = v.copy()
    for s in (16, 8, 4, 2, 1):
        big = t >= (np.int64(1) << s)
        out = np.where(big, out + s, out)
        t = np.where(big, t >> s, t)
    return out.astype(np.int32)


def sat32(a64: np.ndarray) -> np.ndarray:
    return np.clip(a64, I32_MIN, I32_MAX).astype(np.int32)


def rsr(v64: np.ndarray, shift: int) -> np.ndarray:
    """Sign-dependent rounding right shift (kernel/fixed_point/rope_int.py:13-15)."""
    bias = np.int64(1) << (shift - 1)
    v64 = v64.astype(np.int64)
    return np.where(v64 >= 0, (v64 + bias) >> shift, (v64 - bias) >> shift)


# --------------------------------------------------------------------------- Q15.16
def to_fixed(x: np.ndarray) -> np.ndarray:
    """kernel/fixed_point/q15_tensor.py:17-22.  fp32 multiply, round-half-even, clamp.

    The reference clamps to 2**31 - 1 in fp32, which rounds to 2**31, and then
    converts to int32: the result for inputs >= 32768.0 depends on the device
    (x86 gives -2**31, CUDA's saturating convert gives 2**31 - 1).  The oracle
    takes the CUDA behaviour, the device the reference model runs on.
    """
    f = np.asarray(x, dtype=np.float32) * np.float32(FIXED_POINT_SCALE)
    r = np.rint(f).astype(np.float64)
    return np.clip(r, I32_MIN, I32_MAX).astype(np.int64).astype(np.int32)


def from_fixed_f32(x: np.ndarray) -> np.ndarray:
    """kernel/fixed_point/q15_tensor.py:25-27 up to (not including) the final dtype cast."""
    return np.asarray(x, dtype=np.int32).astype(np.float32) / np.float32(FIXED_POINT_SCALE)


# --------------------------------------------------------------------------- RMSNorm v2
def _inverse_sqrt_q0_31(ms: np.ndarray) -> np.ndarray:
    """kernel/fixed_point/rmsnorm_int_only_v2.py:89-117 on an int32 vector; int32 result."""
    ms = ms.astype(np.int32)
    is_zero = ms <= 0
    safe = np.where(is_zero, 1, ms).astype(np.int64)
    pos = msb(safe).astype(np.int64)
    even = ((pos + 1) >> 1) << 1
    xn = _wrap32(safe << (30 - even)).astype(np.int64) >> 21
    xn = np.clip(xn, 0, 1023)
    m = luts.inv_sqrt()[xn].astype(np.int64)
    res = _wrap32(m << (16 - (even >> 1)))
    return np.where(is_zero, 0, res).astype(np.int32)


def _rmsnorm_rows(r: np.ndarray, w: np.ndarray) -> np.ndarray:
    """Steps 1-5 of rmsnorm_int_only_v2.py:144-218 on int32 rows ``r`` [R, H]."""
    R, H = r.shape
    r = r.astype(np.int32)
    neg = _wrap32(-(r.astype(np.int64)))
    r_abs = np.where(r < 0, neg, r)
    m = np.maximum(r_abs.max(axis=1), 0).astype(np.int32)
    zero = m == 0
    p = np.where(zero, 0, msb(np.where(zero, 1, m))).astype(np.int64)
    n = _wrap32(r.astype(np.int64) << (30 - p)[:, None]).astype(np.int32) >> 16
    sq = _wrap32(n.astype(np.int64) * n.astype(np.int64)).astype(np.int64)
    S = sq.sum(axis=1)
    ms = _wrap32((S // H) >> 1).astype(np.int64) + 1
    inv = _inverse_sqrt_q0_31(_wrap32(ms)).astype(np.int64)
    with np.errstate(over="ignore"):
        prod = r.astype(np.int64) * inv[:, None]
        prod = prod * w.astype(np.int64)[None, :]
    out = prod >> (p + 18)[:, None]
    out = sat32(out)
    out[zero] = 0
    return out


def rmsnorm_v2(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """rmsnorm_int_only_v2 (rmsnorm_int_only_v2.py:319-390).

    ``x`` int32 [..., H] or [..., g*H] (packed groups, each normalised alone),
    ``weight`` int32 [H].  The float ``eps`` of the reference is ignored there
    (integer 1 is used, :369) and is therefore not a parameter here.
    """
    x = np.asarray(x, dtype=np.int32)
    weight = np.asarray(weight, dtype=np.int32)
    H = weight.shape[0]
    if x.ndim < 2:
        raise ValueError("x must have at least 2 dims")
    if x.shape[-1] % H != 0:
        raise ValueError("last dim must be a multiple of the weight length")
    out = _rmsnorm_rows(x.reshape(-1, H), weight)
    return out.reshape(x.shape)


def fused_add_rmsnorm_v2(residual: np.ndarray, x: np.ndarray, weight: np.ndarray):
    """fused_add_rmsnorm_int_only_v2 (rmsnorm_int_only_v2.py:393-475, kernel :221-312).

    The residual add wraps in int32 (the clamp at :255-257 acts on an int32 value
    and cannot change it).  Returns (normalised, residual_out).
    """
    residual = np.asarray(residual, dtype=np.int32)
    x = np.asarray(x, dtype=np.int32)
    weight = np.asarray(weight, dtype=np.int32)
    if residual.shape != x.shape:
        raise ValueError("residual and x must have the same shape")
    H = weight.shape[0]
    if x.shape[-1] % H != 0:
        raise ValueError("last dim must be a multiple of the weight length")
    r = _wrap32(residual.astype(np.int64) + x.astype(np.int64))
    out = _rmsnorm_rows(r.reshape(-1, H), weight)
    return out.reshape(x.shape), r.reshape(x.shape)


# --------------------------------------------------------------------------- SiLU * up
LOG2E_SILU = 94549  # silu_and_mul_int_only.py:28 (the attention path uses 94548)


def silu_and_mul(x: np.ndarray) -> np.ndarray:
    """silu_and_mul_int_only (silu_and_mul_int_only.py:115-226, wrapper :233-275).

    ``x`` int32 [B, 2I] laid out gate(0:I) || up(I:2I); returns int32 [B, I].
    """
    x = np.asarray(x, dtype=np.int32)
    if x.ndim != 2:
        raise ValueError("x must be 2-D [batch, 2*hidden]")
    I = x.shape[1] // 2
    g = x[:, :I].astype(np.int64)
    u = x[:, I : 2 * I].astype(np.int64)
    pos = g > 0
    a = np.where(pos, -g, g)
    y = (a * LOG2E_SILU) >> 16
    yi = y >> 16
    yf = y & 0xFFFF
    idx = (yf >> 6) & 0x3FF
    e2 = luts.exp2_silu()[idx].astype(np.int64)
    shift = 13 - yi  # >= 13 because a <= 0
    E = np.where(shift >= 63, 0, e2 >> np.minimum(shift, 62))
    E = np.minimum(E, 65536)
    s = (E * 65536) // (65536 + E)
    sig = np.where(pos, 65536 - s, s)
    t = (g * sig) >> 16
    with np.errstate(over="ignore"):
        out = (t * u) >> 16
    return sat32(out)


# --------------------------------------------------------------------------- FWHT
def fwht_q15(x: np.ndarray, normalize: bool = True) -> np.ndarray:
    """fwht_int_q15 (fwht_int.py:76-96 torch twin, kernels :19-68).

    Butterflies over the last dim (a power of two) with int32 saturation after
    every stage, then an optional Q15 scale by round(2**15 / sqrt(n)).
    """
    x = np.asarray(x, dtype=np.int32)
    if x.ndim < 2:
        raise ValueError("x must have at least 2 dims")
    n = x.shape[-1]
    if n <= 0 or n & (n - 1):
        raise ValueError("last dim must be a power of two")
    cur = x.reshape(-1, n).astype(np.int64)
    idx = np.arange(n)
    step = 1
    while step < n:
        partner = cur[:, idx ^ step]
        lower = ((idx & step) == 0)[None, :]
        cur = np.clip(np.where(lower, cur + partner, partner - cur), I32_MIN, I32_MAX)
        step <<= 1
    if normalize:
        k = int(round((1.0 / math.sqrt(n)) * (1 << 15)))
        cur = np.clip(rsr(cur * k, 15), I32_MIN, I32_MAX)
    return cur.astype(np.int32).reshape(x.shape)


def blockwise_fwht_q15(x: np.ndarray, block: int) -> np.ndarray:
    """apply_blockwise_fwht_q15 (models/utils_integer.py:46-60)."""
    x = np.asarray(x, dtype=np.int32)
    if block <= 0:
        raise ValueError("block must be > 0")
    hidden = x.shape[-1]
    if hidden % block != 0:
        raise ValueError("last dim must be divisible by the block size")
    y = fwht_q15(x.reshape(-1, hidden // block, block), normalize=True)
    return y.reshape(x.shape)


# --------------------------------------------------------------------------- RoPE
def rope_q15(positions, q, k, cos_sin_cache):
    """rope_int_q15 (rope_int.py:88-125): neox halves, Q1.15 trig, rsr 15, saturate.

    ``q`` int32 [T, Hq, D], ``k`` int32 [T, Hk, D], ``cos_sin_cache`` int32
    [max_pos, D] = cos(0:D/2) || sin(D/2:D).
    """
    positions = np.asarray(positions).astype(np.int64)
    cache = np.asarray(cos_sin_cache, dtype=np.int32)

    def apply(x):
        x = np.asarray(x, dtype=np.int32)
        D = x.shape[-1]
        h = D // 2
        trig = cache[positions]
        c = trig[:, None, :h].astype(np.int64)
        s = trig[:, None, h:D].astype(np.int64)
        lo = x[..., :h].astype(np.int64)
        hi = x[..., h:D].astype(np.int64)
        ylo = rsr(lo * c - hi * s, 15)
        yhi = rsr(lo * s + hi * c, 15)
        return sat32(np.concatenate([ylo, yhi], axis=-1))

    return apply(q), apply(k)


def rope_fwht_q15(positions, q, k, cos_sin_cache):
    """rope_fwht_int_q15 (rope_fwht_int.py:9-23): RoPE, then FWHT over every head."""
    qr, kr = rope_q15(positions, q, k, cos_sin_cache)
    return fwht_q15(qr, True), fwht_q15(kr, True)


# --------------------------------------------------------------------------- int8 quant
def per_token_quant_from_q15(x: np.ndarray):
    """per_token_quant_int8_from_q15 (layers/quantization/w8a8_int8.py:104-131).

    Returns (codes int8 [.., K], scale fp32 [.., 1], absmax int32 [.., 1]).  The
    reference does not return the integer absmax; it is exposed because the
    fixed-point requant multiplier is derived from it.
    """
    x = np.asarray(x, dtype=np.int32)
    x2 = x.reshape(-1, x.shape[-1])
    neg = _wrap32(-(x2.astype(np.int64)))
    m = np.maximum(np.where(x2 < 0, neg, x2).max(axis=1, keepdims=True), 1).astype(np.int32)
    q = (x2.astype(np.float32) * np.float32(127.0)) / m.astype(np.float32)
    q = np.clip(np.rint(q), -128, 127).astype(np.int8)          # clamp first: a row's -2^31 gives a quotient beyond int32
    scale = m.astype(np.float32) / np.float32(127.0 * float(FIXED_POINT_SCALE))
    lead = x.shape[:-1] + (1,)
    return q.reshape(x.shape), scale.reshape(lead), m.reshape(lead)


def static_quant_from_q15(x: np.ndarray, input_scale: float) -> np.ndarray:
    """Static per-tensor int8 codes of a Q15.16 tensor: from_fixed (fp32(x) / 65536), divided by the checkpoint's
    fp32 ``input_scale``, rounded half to even, clamped (per_tensor_quant_int8_static, w8a8_int8.py:75-92, on the
    from_fixed value of apply_weights_q15, :251-254).  All arithmetic in fp32."""
    scale = np.maximum(np.float32(input_scale), np.float32(1e-10))
    xf = x.astype(np.float32) / np.float32(65536.0)
    q = np.rint((xf / scale).astype(np.float32))
    return np.clip(q, -128, 127).astype(np.int8)
