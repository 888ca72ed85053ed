"""Host logic of the attention plug-in: metadata built from a batch's requests (no GPU needed)."""
from types import SimpleNamespace

import pytest
import torch

from mini_sgl_integer_b200.attention.backend import B200Int8Backend, Int8Metadata, token_locations


def req(table_idx, cached_len, device_len):
    return SimpleNamespace(table_idx=table_idx, cached_len=cached_len, device_len=device_len,
                           extend_len=device_len - cached_len)


def batch_of(reqs, phase):
    return SimpleNamespace(reqs=reqs, padded_reqs=reqs, phase=phase, is_prefill=phase == "prefill",
                           is_decode=phase == "decode", size=len(reqs), padded_size=len(reqs))


def backend(max_req=8, max_pages=6):
    table = torch.arange(max_req * max_pages, dtype=torch.int32).reshape(max_req, max_pages) * 3 % 50
    return B200Int8Backend.from_heads(16, 8, SimpleNamespace(device=torch.device("cpu")), table), table


def test_prefill_metadata_with_cached_prefixes():
    be, table = backend()
    b = batch_of([req(5, 0, 20), req(2, 16, 40), req(7, 3, 4)], "prefill")
    be.prepare_metadata(b)
    md = b.attn_metadata
    assert isinstance(md, Int8Metadata)
    assert md.kv_lens.tolist() == [20, 40, 4] and md.q_lens.tolist() == [20, 24, 1]
    assert md.qo_indptr.tolist() == [0, 20, 44, 45] and md.max_seqlen_q == 24 and md.max_seqlen_k == 40
    assert torch.equal(md.page_table, table[[5, 2, 7]])
    assert md.get_last_indices(3).tolist() == [19, 43, 44]


def test_decode_metadata_and_capture_buffers():
    be, table = backend()
    b = batch_of([req(1, 9, 10), req(4, 30, 31)], "decode")
    be.prepare_metadata(b)
    md = b.attn_metadata
    assert md.q_lens is None and md.qo_indptr is None and md.kv_lens.tolist() == [10, 31]
    assert md.get_last_indices(2).tolist() == [0, 1]
    be.init_capture_graph(64, [1, 2, 4])
    with pytest.raises(RuntimeError):
        be.init_capture_graph(64, [2])
    cap = batch_of(b.reqs, "decode")
    be.prepare_for_capture(cap)
    assert cap.attn_metadata.page_table.shape == (2, 4) and cap.attn_metadata.max_seqlen_k == 64
    be.prepare_for_replay(b)                      # copies the live metadata into the captured buffers
    assert cap.attn_metadata.kv_lens.tolist() == [10, 31]
    assert torch.equal(cap.attn_metadata.page_table, table[[1, 4], :4])
    with pytest.raises(RuntimeError):
        be.prepare_for_capture(batch_of([req(0, 0, 1)] * 3, "decode"))      # 3 is not a registered size


def test_token_locations():
    _, table = backend()
    rows = table[[5, 2]]
    pos = torch.tensor([0, 15, 16, 39])
    row = torch.tensor([0, 0, 1, 1])
    want = [int(rows[0, 0]) * 16, int(rows[0, 0]) * 16 + 15, int(rows[1, 1]) * 16, int(rows[1, 2]) * 16 + 7]
    assert token_locations(rows, pos, row).tolist() == want


def test_merge_sharded_argmax_prefers_value_then_lowest_id():
    from mini_sgl_integer_b200.models import merge_sharded_argmax
    vals = torch.tensor([[5, -7, 2**31 - 1, -2**31], [5, -3, 2**31 - 1, -2**31], [4, -3, 0, -2**31]], dtype=torch.int32)
    ids = torch.tensor([[10, 11, 12, 13], [110, 111, 112, 113], [210, 211, 212, 213]], dtype=torch.int32)
    assert merge_sharded_argmax(vals, ids).tolist() == [10, 111, 12, 13]
