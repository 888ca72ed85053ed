"""Generate the golden fixtures from the reference's own Python implementation.

Run on a CPU host that has the reference checked out:

    python tests/golden/make_golden.py --reference /path/to/mini-sgl-integer

The script imports ``minisgl`` from ``<reference>/python`` and runs each op of the
integer path on CPU: torch-CPU branches directly, the Triton kernels (RMSNorm v2,
SiLU-and-mul) under ``TRITON_INTERPRET=1``, and ``int8_context_attention_fwd`` with
``python -O`` (its only CUDA dependency is an ``assert``).  It writes

    tests/golden/ref_vectors.npz   inputs and reference outputs, one key per array
    tests/golden/ref_hashes.json   sha256[:16] of selected outputs
    oracle/luts.npz                the three look-up tables, dumped from the reference

Nothing here is imported by the tests; they only read the files it wrote.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def _reexec_optimised() -> None:
    if sys.flags.optimize < 1 or os.environ.get("TRITON_INTERPRET") != "1":
        env = dict(os.environ, TRITON_INTERPRET="1", PYTHONOPTIMIZE="1")
        os.execve(sys.executable, [sys.executable, "-O"] + sys.argv, env)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    _reexec_optimised()
    sys.path.insert(0, os.path.join(args.reference, "python"))

    import numpy as np
    import torch

    from minisgl.kernel.fixed_point import (
        from_fixed, fused_add_rmsnorm_int_only_v2, fwht_int_q15, rmsnorm_int_only_v2,
        rope_fwht_int_q15, rope_int_q15, silu_and_mul_int_only, to_fixed,
    )
    from minisgl.kernel.fixed_point.rmsnorm_int_only_v2 import _get_lut_tables
    from minisgl.kernel.fixed_point.silu_and_mul_int_only import _get_exp2_lut
    from minisgl.kernel.triton.int8_attention_kernels import (
        _exp2_lut_i32, int8_context_attention_fwd, quantize_per_tensor_int8_ms,
    )
    from minisgl.layers.quantization.w8a8_int8 import per_tensor_quant_int8_static, per_token_quant_int8_from_q15
    from minisgl.layers.rotary_integer import RotaryEmbeddingInteger
    from minisgl.models.utils_integer import apply_blockwise_fwht_q15

    def h(t):
        a = t.contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
        return hashlib.sha256(a.tobytes()).hexdigest()[:16]

    vec: dict[str, np.ndarray] = {}
    hashes: dict[str, str] = {}

    def put(name, t):
        a = t.contiguous().numpy() if isinstance(t, torch.Tensor) else np.asarray(t)
        if a.dtype == np.dtype("V2"):
            raise TypeError(name)
        vec[name] = a

    # ---- look-up tables
    inv_sqrt = _get_lut_tables()[0]
    e_silu = _get_exp2_lut()
    e_attn = _exp2_lut_i32(torch.device("cpu"))
    np.savez(os.path.join(ROOT, "oracle", "luts.npz"),
             inv_sqrt=inv_sqrt.numpy(), exp2_silu=e_silu.numpy(), exp2_attn=e_attn.numpy())
    hashes["lut_inv_sqrt"], hashes["lut_exp2_silu"], hashes["lut_exp2_attn"] = h(inv_sqrt), h(e_silu), h(e_attn)

    g = torch.Generator().manual_seed(0)

    def ri(lo, hi, shape, dt=torch.int32):
        return torch.randint(lo, hi, shape, generator=g, dtype=dt)

    # ---- the seeded chain whose hashes the survey of the reference recorded
    x = ri(-(2**20), 2**20, (8, 1024)); r = ri(-(2**20), 2**20, (8, 1024)); w = ri(2**13, 2**15 + 1, (1024,))
    put("norm_x", x); put("norm_r", r); put("norm_w", w)
    o = rmsnorm_int_only_v2(x, w); put("norm_out", o); hashes["A_rmsnorm"] = h(o)
    o, ro = fused_add_rmsnorm_int_only_v2(r, x, w)
    put("fused_out", o); put("fused_res", ro); hashes["B_fused_out"], hashes["B_fused_res"] = h(o), h(ro)
    gu = ri(-(2**19), 2**19, (8, 6144)); put("silu_in", gu)
    s = silu_and_mul_int_only(gu); put("silu_out", s); hashes["C_silu"] = h(s)
    f = apply_blockwise_fwht_q15(s, 128); put("bfwht_out", f); hashes["D_bfwht"] = h(f)
    q8, sc = per_token_quant_int8_from_q15(f); put("quant_codes", q8); put("quant_scale", sc)
    hashes["E_quant_codes"], hashes["E_quant_scale"] = h(q8), h(sc)
    rot = RotaryEmbeddingInteger(128, 128, 4096, 1000000.0)
    cache = rot._cos_sin_cache_q15
    hashes["rope_cache"] = h(cache)
    pos = ri(0, 4096, (8,)); qq = ri(-(2**18), 2**18, (8, 16, 128)); kk = ri(-(2**18), 2**18, (8, 8, 128))
    put("rope_pos", pos); put("rope_q", qq); put("rope_k", kk); put("rope_cache_rows", cache[pos.long()])
    a, b = rope_int_q15(pos, qq, kk, cache); put("rope_q_out", a); put("rope_k_out", b)
    hashes["F_rope_q"], hashes["F_rope_k"] = h(a), h(b)
    a, b = rope_fwht_int_q15(pos, qq, kk, cache); put("ropefwht_q_out", a); put("ropefwht_k_out", b)
    hashes["G_ropefwht_q"], hashes["G_ropefwht_k"] = h(a), h(b)
    qi = ri(-127, 128, (48, 4, 128), torch.int8); ki = ri(-127, 128, (48, 2, 128), torch.int8)
    vi = ri(-127, 128, (48, 2, 128), torch.int8)
    ms = dict(q=(1399068544, 44), k=(2062117504, 36), v=(1224789248, 35))
    t32 = lambda v: torch.tensor(v, dtype=torch.int32)
    out = torch.zeros(48, 4, 128, dtype=torch.bfloat16)
    int8_context_attention_fwd(qi, ki, vi, out, t32(ms["q"][0]), t32(ms["q"][1]), t32(ms["k"][0]), t32(ms["k"][1]),
                               t32(ms["v"][0]), t32(ms["v"][1]), torch.tensor([0, 16], dtype=torch.int32),
                               torch.tensor([16, 32], dtype=torch.int32), 32, True)
    put("attn_q", qi); put("attn_k", ki); put("attn_v", vi)
    put("attn_ms", np.array([ms["q"], ms["k"], ms["v"]], dtype=np.int64))
    put("attn_out_bf16_bits", out.view(torch.int16)); hashes["H_attn_bf16"] = h(out.view(torch.int16))
    out_nc = torch.zeros(48, 4, 128, dtype=torch.bfloat16)
    int8_context_attention_fwd(qi, ki, vi, out_nc, t32(ms["q"][0]), t32(ms["q"][1]), t32(ms["k"][0]), t32(ms["k"][1]),
                               t32(ms["v"][0]), t32(ms["v"][1]), torch.tensor([0, 16], dtype=torch.int32),
                               torch.tensor([16, 32], dtype=torch.int32), 32, False)
    put("attn_out_noncausal_bf16_bits", out_nc.view(torch.int16))

    # ---- edge cases (second generator so the chain above keeps its draw order)
    g2 = torch.Generator().manual_seed(1)
    rj = lambda lo, hi, shape, dt=torch.int32: torch.randint(lo, hi, shape, generator=g2, dtype=dt)

    # RMSNorm: zero row, one-hot rows, tiny rows, huge rows, mixed signs near int32 limits
    H = 256
    e = rj(-(2**22), 2**22, (12, H))
    e[0] = 0
    e[1] = 0; e[1, 7] = 1
    e[2] = 0; e[2, 3] = -1
    e[3] = rj(-3, 4, (H,))
    e[4] = rj(-(2**30), 2**30, (H,))
    e[5] = rj(-(2**31) + 1, 2**31 - 1, (H,), torch.int64).to(torch.int32)
    e[6] = 2**31 - 1
    e[7] = -(2**31) + 1
    e[8] = 0; e[8, 0] = 2**30
    e[9] = rj(-(2**8), 2**8, (H,))
    ew = rj(-(2**17), 2**17, (H,))
    put("norm_edge_x", e); put("norm_edge_w", ew)
    put("norm_edge_out", rmsnorm_int_only_v2(e, ew))
    er = rj(-(2**31) + 1, 2**31 - 1, (12, H), torch.int64).to(torch.int32)
    o, ro = fused_add_rmsnorm_int_only_v2(er, e, ew)
    put("fused_edge_r", er); put("fused_edge_out", o); put("fused_edge_res", ro)
    # packed per-head norm (q_norm / k_norm use): rows of 4 heads x 128
    ph = rj(-(2**21), 2**21, (6, 4 * 128)); pw = rj(2**12, 2**16, (128,))
    put("norm_packed_x", ph); put("norm_packed_w", pw); put("norm_packed_out", rmsnorm_int_only_v2(ph, pw))
    # a Qwen3-14B-wide row
    wx = torch.clamp(torch.round(torch.randn(2, 5120, generator=g2) * 4096.0), -(2**23), 2**23).to(torch.int32)
    wr = torch.clamp(torch.round(torch.randn(2, 5120, generator=g2) * 4096.0), -(2**23), 2**23).to(torch.int32)
    ww = rj(2**13, 2**15 + 1, (5120,))
    o, ro = fused_add_rmsnorm_int_only_v2(wr, wx, ww)
    put("fused_wide_x", wx); put("fused_wide_r", wr); put("fused_wide_w", ww)
    put("fused_wide_out", o); put("fused_wide_res", ro)

    # SiLU: special gates against assorted ups
    sg = torch.tensor([0, 1, -1, 2, -2, 65536, -65536, 65535, -65537, 3 * 65536, -3 * 65536, 20 * 65536,
                       -20 * 65536, -35 * 65536, -36 * 65536, -40 * 65536, -1000 * 65536, 1000 * 65536,
                       2**31 - 1, -(2**31), -(2**31) + 1, 2**30, -(2**30), 12345, -54321, 7, -7, 100000,
                       -100000, 9 * 65536 + 17, -(9 * 65536 + 17), 45426], dtype=torch.int32)
    su = torch.tensor([65536, -65536, 2**31 - 1, -(2**31), 1, -1, 0, 3 * 65536], dtype=torch.int32)
    gate = sg.repeat(8); up = su.repeat_interleave(32)
    sin = torch.cat([gate, up]).view(1, -1).repeat(2, 1).contiguous()
    sin[1] = torch.cat([rj(-(2**23), 2**23, (256,)), rj(-(2**23), 2**23, (256,))])
    put("silu_edge_in", sin); put("silu_edge_out", silu_and_mul_int_only(sin))

    # FWHT: sizes 64/128/256, saturating inputs, un-normalised
    for n in (64, 128, 256):
        fx = rj(-(2**20), 2**20, (4, n))
        put(f"fwht{n}_in", fx); put(f"fwht{n}_out", fwht_int_q15(fx, normalize=True))
    fs = rj(-(2**31) + 1, 2**31 - 1, (6, 128), torch.int64).to(torch.int32)
    fs[0] = 2**31 - 1
    fs[1] = -(2**31)
    fs[2, ::2] = 2**30
    put("fwht_sat_in", fs); put("fwht_sat_out", fwht_int_q15(fs, normalize=True))
    put("fwht_sat_raw", fwht_int_q15(fs, normalize=False))
    fneg = torch.tensor([[-1, 0, 1, -2] * 32, [5, -5, 11, -11] * 32], dtype=torch.int32)
    put("fwht_small_in", fneg); put("fwht_small_out", fwht_int_q15(fneg, normalize=True))

    # RoPE: large magnitudes that saturate
    rq = rj(-(2**31) + 1, 2**31 - 1, (3, 2, 128), torch.int64).to(torch.int32)
    rk = rj(-(2**31) + 1, 2**31 - 1, (3, 1, 128), torch.int64).to(torch.int32)
    rp = torch.tensor([0, 1, 4095], dtype=torch.int32)
    a, b = rope_int_q15(rp, rq, rk, cache)
    put("rope_edge_pos", rp); put("rope_edge_q", rq); put("rope_edge_k", rk)
    put("rope_edge_cache_rows", cache[rp.long()]); put("rope_edge_q_out", a); put("rope_edge_k_out", b)

    # per-token quant: ties, zero row, absmax 1, int32 extremes
    qe = rj(-(2**20), 2**20, (8, 64))
    qe[0] = 0
    qe[1] = 0; qe[1, 5] = 1
    qe[2] = torch.arange(-32, 32, dtype=torch.int32) * 2
    qe[2, 0] = 254   # ratios k/2 -> half-way cases
    qe[3] = rj(-(2**31) + 1, 2**31 - 1, (64,), torch.int64).to(torch.int32)
    qe[4] = torch.arange(64, dtype=torch.int32) - 31
    qe[4, 0] = 127
    q8, sc = per_token_quant_int8_from_q15(qe)
    put("quant_edge_in", qe); put("quant_edge_codes", q8); put("quant_edge_scale", sc)

    # to_fixed / from_fixed
    tf = torch.randn(4, 257, generator=g2) * 37.0
    tf[0, :8] = torch.tensor([0.0, 0.5 / 65536, 1.5 / 65536, -0.5 / 65536, 2.5 / 65536, 32767.5, -32768.0, 1e-9])
    put("tofixed_in", tf); put("tofixed_out", to_fixed(tf))
    put("tofixed_bf16_in_bits", tf.to(torch.bfloat16).view(torch.int16))
    put("tofixed_bf16_out", to_fixed(tf.to(torch.bfloat16)))
    ff = rj(-(2**31) + 1, 2**31 - 1, (4, 257), torch.int64).to(torch.int32)
    put("fromfixed_in", ff); put("fromfixed_f32", from_fixed(ff, torch.float32))
    put("fromfixed_bf16_bits", from_fixed(ff, torch.bfloat16).view(torch.int16))

    # per-tensor quantiser used by the reference backend (for the uniform-scale reduction test)
    kq = torch.randn(40, 2, 128, generator=g2).to(torch.bfloat16)
    k8, kmul, ksh = quantize_per_tensor_int8_ms(kq)
    put("ptq_in_bf16_bits", kq.view(torch.int16)); put("ptq_codes", k8)
    put("ptq_ms", np.array([int(kmul), int(ksh)], dtype=np.int64))

    # static (checkpoint-provided) input scale: from_fixed(x) / scale, rounded and clamped (w8a8_int8.py:75-92, :251-254)
    sq = rj(-(2**20), 2**20, (6, 384))
    sq[0, :6] = torch.tensor([0, 1, -1, 2**31 - 1, -(2**31), 32768], dtype=torch.int32)
    for i, scale in enumerate((0.013671875, 0.05, 1e-3)):
        c8, sc = per_tensor_quant_int8_static(from_fixed(sq, torch.float32), torch.tensor([scale], dtype=torch.float32))
        put(f"static_codes_{i}", c8)
    put("static_in", sq); put("static_scales", np.array([0.013671875, 0.05, 1e-3], dtype=np.float32))

    # per-token quant of rows that hold -2^31 (its |x| wraps, so it never enters the absmax and its code clamps
    # to -128) next to mid-size values: row absmax below 2^22, above it, and just below 2^31
    g3 = torch.Generator().manual_seed(3)
    qi = torch.randint(-(2**20), 2**20, (4, 64), generator=g3, dtype=torch.int32)
    qi[1] = torch.randint(-(2**27), 2**27, (64,), generator=g3, dtype=torch.int32)
    qi[2] = torch.randint(-(2**31) + 1, 2**31 - 1, (64,), generator=g3, dtype=torch.int64).to(torch.int32)
    qi[3] = 0
    for r in range(4):
        qi[r, 7 + r] = -(2**31)
    qi[0, 40] = -(2**31)
    i8, isc = per_token_quant_int8_from_q15(qi)
    put("quant_intmin_in", qi); put("quant_intmin_codes", i8); put("quant_intmin_scale", isc)

    # the same quantiser at other magnitudes: a maximum just above a power of two (its bf16 log2 rounds down to the
    # integer, and the multiplier then exceeds int32: the x86 conversion stored here wraps to -2^31 where a CUDA
    # device saturates at 2^31 - 1), a small one, a large one, and an all-zero tensor (clamped at 1e-8)
    g4 = torch.Generator().manual_seed(4)
    for i, (mult, peak) in enumerate(((1.0, 16.125), (1.0 / 300.0, None), (1000.0, None), (0.0, None))):
        t = (torch.randn(33, 128, generator=g4) * mult).to(torch.bfloat16)
        if peak is not None:
            t = t.clamp(-8, 8); t[3, 5] = peak
        c8, cm, cs = quantize_per_tensor_int8_ms(t)
        put(f"ptq{i}_in_bf16_bits", t.view(torch.int16)); put(f"ptq{i}_codes", c8)
        put(f"ptq{i}_ms", np.array([int(cm), int(cs)], dtype=np.int64))

    # rotary table with the "llama3" frequency re-scaling (layers/rotary_integer.py:152-187): a few rows
    from minisgl.layers.rotary_integer import _get_rope_integer
    l3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 64}
    rot3 = _get_rope_integer(128, 128, 512, 500000.0, l3)
    put("rope_llama3_rows", rot3._cos_sin_cache_q15[[0, 1, 7, 63, 300, 511]])
    l3b = dict(l3, low_freq_factor=2.0, high_freq_factor=2.0)
    put("rope_llama3_step_rows", _get_rope_integer(128, 128, 512, 500000.0, l3b)._cos_sin_cache_q15[[1, 63, 511]])

    np.savez_compressed(os.path.join(HERE, "ref_vectors.npz"), **vec)
    with open(os.path.join(HERE, "ref_hashes.json"), "w") as fjs:
        json.dump(hashes, fjs, indent=1, sort_keys=True)
    print("wrote", len(vec), "arrays;", json.dumps(hashes))


if __name__ == "__main__":
    main()
