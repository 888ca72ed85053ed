"""numpy restatement of the integer attention core (TEST INFRASTRUCTURE ONLY).

Two levels:

* ``context_attention`` restates ``int8_context_attention_fwd``
  (kernel/triton/int8_attention_kernels.py:229-383) one to one: per-tensor
  (multiplier, shift) scales, contiguous K/V, causal mask inside the new tokens,
  no cached prefix.  Pinned against the reference by golden vectors.

* ``paged_attention`` is the generalisation the CUDA kernels implement
  (parity unpinned: the reference has no integer decode and no int8 KV pool):
  int8 K/V held in 16-token pages with a (multiplier, shift) per token and KV
  head, a cached prefix in front of the new tokens, one query scale per token and
  head.  For uniform scales and no prefix it gives the pinned function's Q15.16
  result bit for bit, which the test-suite checks.

Definition of ``paged_attention`` for one sequence with L keys and n_q new
queries (query i may see keys 0 .. L-n_q+i), query head h, KV head h // group:

  dot_j   = sum_d q[d] * k_j[d]                                   (int32)
  cm_j    = (q_mul * k_mul_j) >> 32 ;  s_j = q_shift + k_shift_j - 48
  score_j = sat32(mul_shift(dot_j, cm_j, s_j))                     (Q15.16)
  x_j     = clamp(score_j - max_j score_j, -2**30, 0)
  e_j     = LUT[((y & 0xFFFF) >> 6)] >> clamp(13 - (y >> 16), 0, 31),  y = (x_j*94548) >> 16
  inv     = (2**31 - 1) // max(1, sum_j e_j) ;  p_j = (e_j * inv) >> 16   (Q0.15)
  V reference scale of the call = the (v_mul, v_shift) with the smallest shift,
  then the largest multiplier, over all L keys of the sequence and KV head
  r_j     = min(65535, ((v_mul_j << 15) // v_mul_ref) >> (v_shift_j - v_shift_ref))   (Q0.15; <= 32768
            for multipliers normalised to [2**30, 2**31))
  w_j     = (p_j * r_j + 2**14) >> 15
  acc[d]  = sum_j w_j * v_j[d]
  out[d]  = sat32(mul_shift(acc[d], v_mul_ref, v_shift_ref - 1))   (Q15.16)

With one common V scale r_j == 32768 and w_j == p_j, which is the reference.
The only other deviation from the reference is sat32 on the scores (the
reference carries them as int64; they differ only for logits beyond +-32768.0).
"""
from __future__ import annotations

import numpy as np

from . import luts
from .fixed_point import I32_MAX, I32_MIN, per_token_quant_from_q15, sat32

PAGE = 16
LOG2E_ATTN = 94548  # int8_attention_kernels.py:24


def mul_shift(x, multiplier, shift):
    """_apply_mul_shift_torch (int8_attention_kernels.py:278-285), element-wise.

    shift >= 0: (x*m + (shift > 0 ? 2**(shift-1) : 0)) >> shift ; shift < 0: (x*m) << -shift.
    ``multiplier`` and ``shift`` may be arrays that broadcast against ``x``.
    """
    x = np.asarray(x, dtype=np.int64)
    m = np.asarray(multiplier, dtype=np.int64)
    s = np.asarray(shift, dtype=np.int64)
    prod = x * m
    sp = np.clip(s, 0, 62)
    rnd = np.where(s > 0, np.int64(1) << np.clip(s - 1, 0, 62), 0)
    right = np.where(s >= 63, np.where(prod + rnd < 0, -1, 0), (prod + rnd) >> sp)
    left = prod << np.clip(-s, 0, 62)
    return np.where(s >= 0, right, left)


def exp_q15_16(x_diff: np.ndarray) -> np.ndarray:
    """_exp_q15_16_torch (int8_attention_kernels.py:287-295); x_diff int32 <= 0."""
    y = ((x_diff.astype(np.int64) * LOG2E_ATTN) >> 16).astype(np.int32)
    yi = y >> 16
    yf = y & 0xFFFF
    idx = (yf >> 6) & 0x3FF
    e2 = luts.exp2_attn()[idx]
    sh = np.clip(13 - yi, 0, 31)
    return (e2 >> sh).astype(np.int32)


def softmax_q0_15(scores: np.ndarray, mask: np.ndarray | None):
    """_softmax_q15_16_torch (int8_attention_kernels.py:297-317).

    ``scores`` int64 [..., Lk]; ``mask`` bool broadcastable, True = masked out.
    """
    s = scores.astype(np.int64)
    if mask is not None:
        s = np.where(mask, -(1 << 30), s)
    row_max = s.max(axis=-1, keepdims=True)
    x = np.clip(s - row_max, -(1 << 30), 0).astype(np.int32)
    e = exp_q15_16(x)
    if mask is not None:
        e = np.where(mask, 0, e)
    tot = np.maximum(e.astype(np.int64).sum(axis=-1, keepdims=True), 1)
    inv = ((1 << 31) - 1) // tot
    return ((e.astype(np.int64) * inv) >> 16).astype(np.int32)


def _imatmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Exact integer matmul through float64 BLAS (all partial sums stay below 2**53)."""
    return np.rint(a.astype(np.float64) @ b.astype(np.float64)).astype(np.int64)


def context_attention(q, k, v, q_ms, k_ms, v_ms, b_start_loc, b_seq_len, is_causal=True):
    """int8_context_attention_fwd (int8_attention_kernels.py:229-383) up to the Q15.16 result.

    q int8 [T, Hq, D]; k, v int8 [T, Hk, D]; *_ms = (multiplier, shift) python ints.
    Returns int64 [T, Hq, D] holding the Q15.16 output (rows outside every sequence
    stay 0).  The reference then stores bf16(out / 65536); see ``q15_to_bf16_bits``.
    """
    q = np.asarray(q, dtype=np.int8)
    k = np.asarray(k, dtype=np.int8)
    v = np.asarray(v, dtype=np.int8)
    T, Hq, D = q.shape
    Hk = k.shape[1]
    G = Hq // Hk
    q_mul, q_shift = int(q_ms[0]), int(q_ms[1])
    k_mul, k_shift = int(k_ms[0]), int(k_ms[1])
    v_mul, v_shift = int(v_ms[0]), int(v_ms[1])
    cm = (q_mul * k_mul) >> 32
    score_shift = q_shift + k_shift - 32 - 16
    out = np.zeros((T, Hq, D), dtype=np.int64)
    for b in range(len(b_seq_len)):
        st, L = int(b_start_loc[b]), int(b_seq_len[b])
        if L <= 0:
            continue
        mask = np.triu(np.ones((L, L), dtype=bool), 1) if is_causal else None
        for h in range(Hq):
            kh = h // G
            dot = _imatmul(q[st : st + L, h], k[st : st + L, kh].T).astype(np.int32)
            scores = mul_shift(dot, cm, score_shift)
            p = softmax_q0_15(scores, mask)
            acc = _imatmul(p, v[st : st + L, kh])
            out[st : st + L, h] = mul_shift(acc, v_mul, v_shift - 1)
    return out


def q15_to_bf16_bits(out_q15: np.ndarray) -> np.ndarray:
    """bf16(float32(out) / 65536) as raw int16 bit patterns (round-to-nearest-even)."""
    f = out_q15.astype(np.float32) / np.float32(65536.0)
    u = f.view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16).view(np.int16)


def quantize_per_tensor_int8_ms(x_bf16_bits: np.ndarray):
    """quantize_per_tensor_int8_ms (int8_attention_kernels.py:41-53) for a bf16 tensor given as raw uint16 bits.

    The maximum, its clamp at 1e-8 and log2 / ceil / 31 - e are bf16 operations in the reference (the tensor's
    dtype), the multiplier and the codes fp32.  Returns (codes int8, multiplier int, shift int).
    """
    bits = np.asarray(x_bf16_bits).view(np.uint16)
    x = (bits.astype(np.uint32) << 16).view(np.float32)

    def bf16(v):
        u = np.float32(v).reshape(1).view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        return r.astype(np.uint32).view(np.float32)[0]
    max_abs = max(np.float32(np.abs(x).max()) if x.size else np.float32(0), bf16(1e-8))
    e = np.ceil(bf16(np.log2(np.float32(max_abs))))
    shift = int(bf16(np.float32(31.0) - e))
    mult_f = np.float32(max_abs) * np.float32(2.0) ** np.float32(shift)
    multiplier = int(min(mult_f, np.float32(2**31 - 1)))
    multiplier = min(multiplier, 2**31 - 1)
    q = np.clip(np.rint((x / np.float32(max_abs)) * np.float32(127.0)), -128, 127).astype(np.int8)
    return q, multiplier, shift + 7


# --------------------------------------------------------------------------- paged pool
def absmax_to_mul_shift(m):
    """Fixed-point form of the per-row int8 scale m / (127 * 65536) (build-defined).

    Returns (mul, shift) with mul in [2**30, 2**31) and mul / 2**shift ~= m / (127*65536):
      p = msb(m); k = 37 - p; mul = ((m << k) + 63) // 127
      if mul >= 2**31: k -= 1 and recompute;  shift = k + 16
    """
    from .fixed_point import msb

    m = np.maximum(np.asarray(m, dtype=np.int64), 1)
    p = msb(m).astype(np.int64)
    k = 37 - p
    mul = ((m << k) + 63) // 127
    over = mul >= (1 << 31)
    k = np.where(over, k - 1, k)
    mul = np.where(over, ((m << k) + 63) // 127, mul)
    return mul.astype(np.int32), (k + 16).astype(np.int32)


def v_chunk_offset(d, tok):
    """Byte offset of (d, tok) inside a page's 2 KB V chunk (build-defined layout).

    Four 512-byte quarters, each one 16-byte vector per "lane"; lane = (d % 8) * 4 + tok // 4
    owns, as word (d // 16) * 2 + (d % 16) // 8, the four tokens tok & ~3 .. of row d.
    """
    wi = ((d >> 4) << 1) | ((d >> 3) & 1)
    lane = ((d & 7) << 2) | (tok >> 2)
    return ((wi >> 2) << 9) + (lane << 4) + ((wi & 3) << 2) + (tok & 3)


V_OFFSETS = np.array([[v_chunk_offset(d, t) for t in range(PAGE)] for d in range(128)], dtype=np.int64)
assert sorted(V_OFFSETS.reshape(-1).tolist()) == list(range(2048))


class PagedKV:
    """An int8 KV pool for ONE layer in the physical layout the CUDA kernels read.

      k_codes int8  [P, Hkv, 16, D]   token-major rows inside a page
      v_codes int8  [P, Hkv, 2048]    the 16 x 128 bytes of a page in tensor-core operand order:
                                      byte (d, tok) sits at ``v_chunk_offset(d, tok)``
      meta    int32 [P, Hkv, 40]      words 0-15 k_mul, 16-31 v_mul,
                                      32-35 k_shift (16 int8), 36-39 v_shift (16 int8)
    A token location is ``page * 16 + offset``.
    """

    def __init__(self, num_pages: int, num_kv_heads: int, head_dim: int = 128):
        self.P, self.H, self.D = num_pages, num_kv_heads, head_dim
        self.k_codes = np.zeros((num_pages, num_kv_heads, PAGE, head_dim), dtype=np.int8)
        self.v_codes = np.zeros((num_pages, num_kv_heads, head_dim * PAGE), dtype=np.int8)
        self.meta = np.zeros((num_pages, num_kv_heads, 40), dtype=np.int32)

    def _shift_view(self, which: int) -> np.ndarray:
        lo = 32 if which == 0 else 36
        return self.meta[:, :, lo : lo + 4].view(np.int8)  # [P, H, 16]

    def store_codes(self, loc, k8, v8, k_mul, k_shift, v_mul, v_shift):
        """Scatter already-quantised tokens. k8/v8 int8 [T, Hkv, D]; scales [T, Hkv]."""
        loc = np.asarray(loc, dtype=np.int64)
        pg, off = loc // PAGE, loc % PAGE
        ks, vs = self._shift_view(0), self._shift_view(1)
        for t in range(len(loc)):
            self.k_codes[pg[t], :, off[t], :] = k8[t]
            self.v_codes[pg[t], :, V_OFFSETS[:, off[t]]] = np.asarray(v8[t]).T
            self.meta[pg[t], :, off[t]] = k_mul[t]
            self.meta[pg[t], :, 16 + off[t]] = v_mul[t]
            ks[pg[t], :, off[t]] = k_shift[t]
            vs[pg[t], :, off[t]] = v_shift[t]

    def store_q15(self, loc, k_q15, v_q15):
        """Quantise Q15.16 rows per token and KV head, then scatter (build-defined).

        codes follow per_token_quant_from_q15 on each 128-wide head row; the
        (mul, shift) pair is ``absmax_to_mul_shift`` of that row's absmax.
        """
        T = len(loc)
        k3 = np.asarray(k_q15, dtype=np.int32).reshape(T, self.H, self.D)
        v3 = np.asarray(v_q15, dtype=np.int32).reshape(T, self.H, self.D)
        k8, _, km = per_token_quant_from_q15(k3)
        v8, _, vm = per_token_quant_from_q15(v3)
        kmul, ksh = absmax_to_mul_shift(km[..., 0])
        vmul, vsh = absmax_to_mul_shift(vm[..., 0])
        self.store_codes(loc, k8, v8, kmul, ksh, vmul, vsh)

    def gather(self, pages, length: int):
        """Logical view of one sequence: k,v int8 [L,Hkv,D]; muls/shifts int64 [L,Hkv]."""
        pages = np.asarray(pages, dtype=np.int64)
        n = (length + PAGE - 1) // PAGE
        pg = pages[:n]
        k = self.k_codes[pg].transpose(0, 2, 1, 3).reshape(n * PAGE, self.H, self.D)[:length]
        v = self.v_codes[pg][:, :, V_OFFSETS]  # [n, H, D, 16]
        v = v.transpose(0, 3, 1, 2).reshape(n * PAGE, self.H, self.D)[:length]
        km = self.meta[pg, :, 0:16].transpose(0, 2, 1).reshape(n * PAGE, self.H)[:length]
        vm = self.meta[pg, :, 16:32].transpose(0, 2, 1).reshape(n * PAGE, self.H)[:length]
        ks = self._shift_view(0)[pg].transpose(0, 2, 1).reshape(n * PAGE, self.H)[:length]
        vs = self._shift_view(1)[pg].transpose(0, 2, 1).reshape(n * PAGE, self.H)[:length]
        return k, v, km.astype(np.int64), ks.astype(np.int64), vm.astype(np.int64), vs.astype(np.int64)


def v_reference_scale(v_mul: np.ndarray, v_shift: np.ndarray):
    """Smallest shift, then largest multiplier, over the keys of one (sequence, KV head)."""
    s_ref = int(v_shift.min())
    m_ref = int(v_mul[v_shift == s_ref].max())
    return m_ref, s_ref


def v_relative_q15(v_mul, v_shift, m_ref: int, s_ref: int) -> np.ndarray:
    d = (v_shift - s_ref).astype(np.int64)
    if m_ref <= 0:
        return np.zeros_like(d)
    ratio = (v_mul.astype(np.int64) << 15) // m_ref
    return np.minimum(np.where(d >= 32, 0, ratio >> np.minimum(d, 31)), 65535)


def sequence_attention(q, q_mul, q_shift, k, v, k_mul, k_shift, v_mul, v_shift):
    """The definition in the module docstring for ONE sequence.

    q int8 [n_q, Hq, D] (the last n_q positions of the sequence); q_mul/q_shift [n_q, Hq];
    k, v int8 [L, Hkv, D]; k_mul.. [L, Hkv].  Returns int32 [n_q, Hq, D] (Q15.16).
    """
    n_q, Hq, D = q.shape
    L, Hk, _ = k.shape
    G = Hq // Hk
    out = np.zeros((n_q, Hq, D), dtype=np.int32)
    if L == 0:
        return out
    kpos = np.arange(L)[None, :]
    limit = (L - n_q + np.arange(n_q))[:, None]
    mask = kpos > limit  # True = not visible
    for kh in range(Hk):
        m_ref, s_ref = v_reference_scale(v_mul[:, kh], v_shift[:, kh])
        rel = v_relative_q15(v_mul[:, kh], v_shift[:, kh], m_ref, s_ref)
        for g in range(G):
            h = kh * G + g
            dot = _imatmul(q[:, h], k[:, kh].T)  # [n_q, L]
            cm = (q_mul[:, h].astype(np.int64)[:, None] * k_mul[:, kh][None, :]) >> 32
            sh = q_shift[:, h].astype(np.int64)[:, None] + k_shift[:, kh][None, :] - 48
            scores = np.clip(mul_shift(dot, cm, sh), I32_MIN, I32_MAX)
            p = softmax_q0_15(scores, mask).astype(np.int64)
            w = (p * rel[None, :] + (1 << 14)) >> 15
            acc = _imatmul(w, v[:, kh])
            out[:, h] = sat32(mul_shift(acc, m_ref, s_ref - 1))
    return out


def paged_attention(q, q_mul, q_shift, pool: PagedKV, page_table, kv_lens, q_lens):
    """Batch of sequences over a paged pool (decode: every q_len == 1; extend: >= 1).

    q int8 [sum(q_lens), Hq, D] with sequences back to back; ``page_table`` is a
    list of per-sequence page-id arrays; kv_lens include the new tokens (which
    must already be stored in the pool).  Returns int32 [sum(q_lens), Hq, D].
    """
    q = np.asarray(q, dtype=np.int8)
    out = np.zeros(q.shape, dtype=np.int32)
    st = 0
    for b, (L, n) in enumerate(zip(kv_lens, q_lens)):
        L, n = int(L), int(n)
        if n == 0:
            continue
        k, v, km, ks, vm, vs = pool.gather(page_table[b], L)
        out[st : st + n] = sequence_attention(
            q[st : st + n], np.asarray(q_mul)[st : st + n], np.asarray(q_shift)[st : st + n],
            k, v, km, ks, vm, vs,
        )
        st += n
    return out


def quant_heads_int8(out_q15: np.ndarray):
    """int8 form of an attention output: per (token, head) row quant of the Q15.16 values.

    Codes follow per_token_quant_from_q15 on each head row; returns (codes, absmax[T,Hq]).
    """
    codes, _, m = per_token_quant_from_q15(out_q15)
    return codes, m[..., 0]
