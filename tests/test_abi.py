"""CPU-only checks of the C-ABI library: it loads, exports what the header declares, holds the
reference's tables, and rejects bad arguments before touching the GPU."""
from __future__ import annotations

import ctypes
import os
import re

import numpy as np
import pytest

from mini_sgl_integer_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "b200int.h")).read()
    return sorted(set(re.findall(r"B200_API\s+[\w\s\*]+?\b(b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 16
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names  # the ctypes table covers the whole header


def test_version():
    assert _lib.load().b200_version() >= 100


def test_compiled_in_luts_equal_reference_tables():
    from oracle import luts
    buf = (ctypes.c_int32 * 1024)()
    for which, ref in ((0, luts.inv_sqrt()), (1, luts.exp2_silu()), (2, luts.exp2_attn())):
        _lib.call("b200_get_lut", which, ctypes.cast(buf, ctypes.c_void_p))
        assert np.array_equal(np.frombuffer(buf, dtype=np.int32), ref)
    with pytest.raises(_lib.B200Error):
        _lib.call("b200_get_lut", 7, ctypes.cast(buf, ctypes.c_void_p))


def test_bad_arguments_are_rejected_before_launch():
    one = ctypes.c_void_p(16)  # never dereferenced: every call below fails validation first
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_rmsnorm_q15", None, None, one, None, one, None, None, None, 4, 128, None)
    assert e.value.code == -1
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_rmsnorm_q15", one, None, one, None, one, None, None, None, 4, 130, None)
    assert e.value.code == -4 and "multiple of 4" in str(e.value)
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_rmsnorm_q15", ctypes.c_void_p(20), None, one, None, one, None, None, None, 4, 128, None)
    assert e.value.code == -3
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_fwht_q15", one, one, 4, 96, 1, None)
    assert e.value.code == -2
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_silu_mul_q15", one, one, None, None, None, 4, 200, 128, None)
    assert e.value.code == -4
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_attn_decode", one, one, one, one, one, one, one, 4, one, None, one, None, None,
                  2, 12, 5, 10, 64, 0, None)
    assert e.value.code == -2  # q_heads not a multiple of kv_heads
    with pytest.raises(_lib.B200Error) as e:
        _lib.call("b200_attn_decode", one, one, one, one, one, one, one, 1, one, None, one, None, None,
                  2, 8, 2, 10, 640, 0, None)
    assert e.value.code == -2 and "table_pitch" in str(e.value)


def test_ops_refuse_cpu_tensors():
    import torch
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    x = torch.zeros(2, 128, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fp.fwht_int_q15(x)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        fp.rmsnorm_int_only_v2(x, torch.ones(128, dtype=torch.int32))


def test_argument_errors_mirror_reference():
    import torch
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    with pytest.raises(TypeError):
        fp.fwht_int_q15(torch.zeros(2, 128))
    with pytest.raises(ValueError):
        fp.fwht_int_q15(torch.zeros(128, dtype=torch.int32))
    with pytest.raises(ValueError):
        fp.fwht_int_q15(torch.zeros(2, 96, dtype=torch.int32))
    with pytest.raises(ValueError):
        fp.rmsnorm_int_only_v2(torch.zeros(2, 100, dtype=torch.int32), torch.ones(64, dtype=torch.int32))
    with pytest.raises(ValueError):
        fp.fused_add_rmsnorm_int_only_v2(torch.zeros(2, 64, dtype=torch.int32), torch.zeros(3, 64, dtype=torch.int32),
                                         torch.ones(64, dtype=torch.int32))
    with pytest.raises(TypeError):
        fp.rope_int_q15(torch.zeros(2), torch.zeros(2, 4, 128), torch.zeros(2, 2, 128, dtype=torch.int32),
                        torch.zeros(8, 128, dtype=torch.int32))
    with pytest.raises(TypeError):
        fp.apply_blockwise_fwht_q15(torch.zeros(2, 256), 128)
    with pytest.raises(ValueError):
        fp.apply_blockwise_fwht_q15(torch.zeros(2, 200, dtype=torch.int32), 128)
    with pytest.raises(TypeError):
        fp.assert_q15(torch.zeros(2))
