"""Look-up tables of the integer path (oracle side; test infrastructure only).

The three 1024-entry tables are held as data in ``luts.npz`` beside this file.
They were dumped from the reference's own generators on a CPU host by
``tests/golden/make_golden.py``; the oracle never regenerates them at run time
because two of them depend on the host's libm / vector-math library.

  inv_sqrt   kernel/fixed_point/rmsnorm_int_only_v2.py:31-43   (Q0.16 of 1/sqrt(4i/1023))
  exp2_silu  kernel/fixed_point/silu_and_mul_int_only.py:35-46 (Q0.29 of 2^(i/1023), numpy)
  exp2_attn  kernel/triton/int8_attention_kernels.py:27-29     (Q0.29 of 2^(i/1023), torch fp32)

``recompute_*`` restate the generators; the CPU test-suite checks that they give
the stored tables on the machine the tests run on.
"""
from __future__ import annotations

import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_CACHE: dict[str, np.ndarray] = {}


def _load() -> dict[str, np.ndarray]:
    if not _CACHE:
        with np.load(os.path.join(_HERE, "luts.npz")) as z:
            for k in ("inv_sqrt", "exp2_silu", "exp2_attn"):
                a = z[k].astype(np.int32)
                assert a.shape == (1024,)
                _CACHE[k] = a
    return _CACHE


def inv_sqrt() -> np.ndarray:
    return _load()["inv_sqrt"]


def exp2_silu() -> np.ndarray:
    return _load()["exp2_silu"]


def exp2_attn() -> np.ndarray:
    return _load()["exp2_attn"]


def recompute_inv_sqrt() -> np.ndarray:
    """rmsnorm_int_only_v2.py:36-43: fp64 formula, truncated to int32, entry 0 = 0."""
    lut = np.zeros(1024, dtype=np.int32)
    v = np.linspace(0.0, 4.0, 1024)
    lut[1:] = np.clip((1.0 / np.sqrt(v[1:])) * (1 << 16) + 0.5, 0, (1 << 16) - 1).astype(np.int64)
    return lut


def recompute_exp2_silu() -> np.ndarray:
    """silu_and_mul_int_only.py:42-46: fp64 exp2 rounded to fp32, scaled in fp32, truncated."""
    e = np.exp2(np.linspace(0.0, 1.0, 1024)).astype(np.float32)
    f = np.clip(e * np.float32(1 << 29) + np.float32(0.5), 0, (1 << 32) - 1)
    return f.astype(np.int64).astype(np.int32)


def recompute_exp2_attn() -> np.ndarray:
    """int8_attention_kernels.py:27-29: torch fp32 linspace/exp2, scaled in fp32, truncated."""
    import torch

    lut = torch.exp2(torch.linspace(0, 1, 1024, dtype=torch.float32))
    return (lut * (1 << 29) + 0.5).to(torch.int32).numpy()
