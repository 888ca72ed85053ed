"""The attention entry point that brings its own scratch area (b200_attn_paged_static), called through the C ABI.

Collected last on purpose (the file name sorts after the others): the area is shared by every call on the
device, so the checks below also cover calls made after everything else in the suite has run.
"""
import numpy as np
import pytest
import torch

from attn_util import device_pool, make_case
from oracle import attention as oattn

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 16 << 20


def d(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _args(case, pool, max_kv_len):
    from mini_sgl_integer_b200._lib import ptr
    need = (max_kv_len + 15) // 16
    table = case["table"]
    if table.shape[1] < need:
        table = np.pad(table, ((0, 0), (0, need - table.shape[1])))
    t = dict(q8=d(case["q8"]), qm=d(case["qm"]), qs=d(case["qs"]), table=d(table), lens=d(case["kv_lens"]))
    batch, q_heads, _ = case["q8"].shape
    head = [ptr(t["q8"]), ptr(t["qm"]), ptr(t["qs"]), ptr(pool.k_cache(0)), ptr(pool.v_cache(0)), ptr(pool.meta(0)),
            ptr(t["table"]), t["table"].stride(0), ptr(t["lens"]), None, None]
    tail = [batch, q_heads, pool.kv_heads, pool.num_pages, int(max_kv_len)]
    return t, head, tail, (batch, q_heads)


def _outputs(batch, q_heads):
    return (torch.full((batch, q_heads, 128), 0x5A5A5A5A, dtype=torch.int32, device="cuda"),
            torch.full((batch, q_heads, 128), 0x5A, dtype=torch.int8, device="cuda"),
            torch.full((batch, q_heads), 0x5A5A5A5A, dtype=torch.int32, device="cuda"))


def _both(case, pool, max_kv_len):
    """(outputs of the caller-workspace entry point, outputs of the built-in-scratch entry point)."""
    from mini_sgl_integer_b200._lib import call, load, ptr, stream
    keep, head, tail, (batch, q_heads) = _args(case, pool, max_kv_len)
    need = load().b200_attn_workspace_bytes(batch, q_heads, pool.kv_heads, int(max_kv_len))
    assert 0 < need <= SCRATCH_BYTES
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    want, got = _outputs(batch, q_heads), _outputs(batch, q_heads)
    call("b200_attn_paged_ws", *head, ptr(want[0]), ptr(want[1]), ptr(want[2]), *tail, ptr(ws), ws.numel(), stream())
    call("b200_attn_paged_static", *head, ptr(got[0]), ptr(got[1]), ptr(got[2]), *tail, stream())
    torch.cuda.synchronize()
    del keep
    return [w.cpu().numpy() for w in want], [g.cpu().numpy() for g in got]


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    # Two different batches back to back: the second call finds the area full of the first call's data.
    first = make_case(71, [700, 33, 1, 256, 2049], 8, 2, 256)
    second = make_case(72, [16, 1500, 300], 16, 2, 160)
    pool1, pool2 = device_pool(first, 256, 2), device_pool(second, 160, 2)
    for case, pool, longest in ((first, pool1, 2049), (second, pool2, 1500), (first, pool1, 2049)):
        want, got = _both(case, pool, longest)
        for w, g in zip(want, got):
            np.testing.assert_array_equal(g, w)


def test_matches_the_oracle_and_leaves_device_memory_alone():
    """One batch against the CPU oracle (Q15.16 output, int8 codes and their absmax), and the amount of free device
    memory before and after a call that is not the first one on the device: the call allocates nothing."""
    from mini_sgl_integer_b200._lib import call, ptr, stream
    case = make_case(75, [130, 17, 1, 640], 8, 2, 64)
    pool = device_pool(case, 64, 2)
    keep, head, tail, (batch, q_heads) = _args(case, pool, 640)
    out = _outputs(batch, q_heads)
    call("b200_attn_paged_static", *head, ptr(out[0]), ptr(out[1]), ptr(out[2]), *tail, stream())   # set-up call
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    call("b200_attn_paged_static", *head, ptr(out[0]), ptr(out[1]), ptr(out[2]), *tail, stream())
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    want = oattn.paged_attention(case["q8"], case["qm"], case["qs"], case["pool"], case["tables"], case["kv_lens"], [1] * batch)
    codes, absmax = oattn.quant_heads_int8(want)
    np.testing.assert_array_equal(out[0].cpu().numpy(), want)
    np.testing.assert_array_equal(out[1].cpu().numpy(), codes)
    np.testing.assert_array_equal(out[2].cpu().numpy(), absmax)


def test_same_call_twice_gives_the_same_answer():
    case = make_case(73, [900, 901, 5], 4, 1, 128)
    pool = device_pool(case, 128, 1)
    a = _both(case, pool, 901)[1]
    b = _both(case, pool, 901)[1]
    for x, y in zip(a, b):
        np.testing.assert_array_equal(x, y)


def test_request_beyond_the_built_in_area_is_refused():
    from mini_sgl_integer_b200._lib import B200Error, call, load, ptr, stream
    case = make_case(74, [64, 64], 32, 8, 16)
    pool = device_pool(case, 16, 8)
    too_long = 70000                      # 2 rows x 32 heads x 70000 keys x 4 bytes > 16 MiB
    assert load().b200_attn_workspace_bytes(2, 32, 8, too_long) > SCRATCH_BYTES
    keep, head, tail, (batch, q_heads) = _args(case, pool, too_long)
    out = _outputs(batch, q_heads)
    with pytest.raises(B200Error, match="scratch"):
        call("b200_attn_paged_static", *head, ptr(out[0]), ptr(out[1]), ptr(out[2]), *tail, stream())
    torch.cuda.synchronize()
    assert int(out[0][0, 0, 0]) == 0x5A5A5A5A          # nothing was launched
