"""The arithmetic shortcuts of the CUDA row kernels, restated in numpy and checked against the oracle on the CPU.

The kernels do not evaluate the reference's formulas literally everywhere: the sigmoid term comes from a direct
table, one form serves both signs of the gate, the n = 128 Hadamard scale is one wide multiply-add, and the per-token
quantisation estimates the quotient with a reciprocal and only divides near a rounding tie.  Each of these rests on an
identity that holds for every input of its stated range; the parity tests on the GPU show the kernels' bits, these
show the identities themselves (and that the generated table and its constants are the ones in the tree).
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

import numpy as np

from oracle import fixed_point as ofp

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "mini_sgl_integer_b200", "csrc")
ENTRIES = 19457                     # kSnegEntries
FIRST_A = -863090                   # kSnegFirstA


def _table() -> np.ndarray:
    src = open(os.path.join(CSRC, "silu_sneg.inc")).read()
    vals = [int(v) for v in re.findall(r"-?\d+", src.split("\\\n", 1)[1])]
    assert len(vals) == ENTRIES
    return np.asarray(vals, dtype=np.int64)


def test_sigmoid_table_is_what_its_generator_writes(tmp_path):
    """make_silu_table.py reproduces silu_sneg.inc from luts.inc, and silu.cuh carries the table's size and the
    argument of its first key."""
    work = tmp_path / "csrc"
    work.mkdir()
    for name in ("make_silu_table.py", "luts.inc"):
        (work / name).write_bytes(open(os.path.join(CSRC, name), "rb").read())
    subprocess.run([sys.executable, str(work / "make_silu_table.py")], check=True, capture_output=True)
    assert (work / "silu_sneg.inc").read_bytes() == open(os.path.join(CSRC, "silu_sneg.inc"), "rb").read()
    hdr = open(os.path.join(CSRC, "silu.cuh")).read()
    assert f"constexpr int kSnegEntries = {ENTRIES};" in hdr
    assert f"constexpr int kSnegFirstA = {FIRST_A};" in hdr
    tab = _table()
    assert tab[0] == 0 and tab[-1] == 32768 and np.all(np.diff(tab) >= 0)
    assert (FIRST_A * 94549) >> 22 == -(ENTRIES - 1) and ((FIRST_A - 1) * 94549) >> 22 == -ENTRIES


def _silu_small(g: np.ndarray, u: np.ndarray, tab: np.ndarray) -> np.ndarray:
    """silu_mul_elem_table_small: a = max(-|g|, FIRST_A); s = table[(a * 94549 >> 22) + ENTRIES - 1];
    t = (a * s >> 16) + max(g, 0); result = t * u >> 16 (no saturation in its range)."""
    a = np.maximum(np.minimum(g, -g), FIRST_A)
    s = tab[((a * 94549) >> 22) + (ENTRIES - 1)]
    t = ((a * s) >> 16) + np.maximum(g, 0)
    return (t * u) >> 16


def test_small_magnitude_silu_form_equals_the_reference_arithmetic():
    """Every gate and up in [-2**20, 2**20): the clamped-argument table lookup and the single form for both signs give
    silu_and_mul_int_only's result, and the result stays below 2**24 in magnitude (so that neither the products nor
    the seven butterfly stages behind them can saturate)."""
    rng = np.random.default_rng(1)
    n = 1_500_000
    g = np.concatenate([rng.integers(-(2**20), 2**20, n), np.rint(rng.normal(0, 2**17, n)).clip(-(2**20), 2**20 - 1).astype(np.int64),
                        np.arange(-70000, 70000), np.array([-(2**20), 2**20 - 1, FIRST_A - 1, FIRST_A, FIRST_A + 1, 0, 1, -1])])
    u = rng.integers(-(2**20), 2**20, len(g))
    u[:8] = [-(2**20), 2**20 - 1, 0, 1, -1, 2**19, -(2**19), 3]
    got = _silu_small(g, u, _table())
    want = ofp.silu_and_mul(np.concatenate([g, u]).astype(np.int32)[None, :])[0]
    np.testing.assert_array_equal(got, want)
    assert np.abs(got).max() < 2**24
    # the range check itself: v + 2**20 has a bit above bit 20 exactly when v is outside [-2**20, 2**20)
    v = np.array([-(2**20) - 1, -(2**20), -1, 0, 2**20 - 1, 2**20, 2**31 - 1, -(2**31)], dtype=np.int64)
    outside = ((v + 2**20) & 0xFFFFFFFF) >= 2**21
    np.testing.assert_array_equal(outside, (v < -(2**20)) | (v >= 2**20))


def test_hadamard_scale_as_one_wide_multiply_add():
    """rsr15(y * 2896) == ((y * 181 + 1024) >> 11) + (y >> 31) for every int32 y (2896 = 16 * 181; for y < 0 the
    sign-dependent rounding subtracts the bias, which is one less after the shift)."""
    rng = np.random.default_rng(0)
    y = np.concatenate([rng.integers(-(2**31), 2**31, 2_000_000), np.arange(-5000, 5000),
                        np.array([-(2**31), 2**31 - 1])]).astype(np.int64)
    want = ofp.rsr(y * 2896, 15)
    got = ((y * 181 + 1024) >> 11) + (y >> 31)
    np.testing.assert_array_equal(got, want)
    assert np.abs(got).max() < 2**31


def test_quant_estimate_only_differs_from_the_division_inside_the_tie_band():
    """code = rint(fp32(x) * 127 / absmax) in fp32 (per_token_quant_int8_from_q15).  Both estimates used by the kernels
    (x * (127 * rcp(absmax)) for absmax < 2**22, (x * 127) * rcp(absmax) otherwise) round to the same integer as the
    division whenever they are farther than 2**-13 from a half-integer - the rows where the kernels skip the division.
    Inputs include the nearest integers to every half-integer quotient."""
    f = np.float32
    magic, band = f(12582912.0), f(0.4998779296875)
    rng = np.random.default_rng(5)
    checked = 0
    for trial in range(300):
        m = int(rng.integers(1, 2**22)) if trial % 3 else int(rng.integers(1, 5000))
        mf = f(m)
        y = f(1) / mf
        y127 = f(y * f(127))
        ks = rng.integers(-127, 127, 4000)
        near = np.rint((ks + 0.5) * m / 127.0).astype(np.int64)
        xs = np.clip(np.concatenate([near - 1, near, near + 1, rng.integers(-m, m + 1, 4000)]), -m, m).astype(np.float32)
        exact = np.rint((xs * f(127)) / mf)
        for q in (xs * y127, (xs * f(127)) * y):
            r = (q + magic) - magic                     # round to nearest even integer, as the kernels do
            far = np.abs(q - r) <= band
            np.testing.assert_array_equal(r[far], exact[far])
            checked += int(far.sum())
    assert checked > 1_000_000
