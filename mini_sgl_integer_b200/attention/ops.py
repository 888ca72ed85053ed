"""Functional entry points of the int8 paged attention kernels."""
from __future__ import annotations

import torch

from .. import _lib
from .._lib import call, ptr, require_cuda, stream
from .kv_pool import HEAD_DIM, Int8PagedKVCache

_WORKSPACES: dict = {}


def attention_workspace(rows: int, q_heads: int, kv_heads: int, max_kv_len: int, device) -> torch.Tensor:
    """A cached uint8 workspace for the workspace-based attention passes (one per device and stream)."""
    need = int(_lib.load().b200_attn_workspace_bytes(rows, q_heads, kv_heads, int(max_kv_len)))
    key = (torch.device(device).index, torch.cuda.current_stream().cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def _cluster_fits(group: int, max_kv_len: int) -> bool:
    """Shared memory of the cluster kernel with eight CTAs per (sequence, KV head): ring + per-key state."""
    pages = (int(max_kv_len) + 15) // 16
    s_max = (((pages + 7) // 8) * 16 + 31) // 32 * 32
    smem = 8 * 4480 + group * s_max * 4 + (s_max // 16) * 4 + 8 * 2 * group * 32
    return smem <= 200 * 1024


def _paged_ws(q8, q_mul, q_shift, pool, layer_id, page_table, kv_lens, row_seq, row_limit, o32, o8, om, rows, q_heads,
              max_kv_len, workspace):
    ws = workspace if workspace is not None else attention_workspace(rows, q_heads, pool.kv_heads, max_kv_len, q8.device)
    call("b200_attn_paged_ws", ptr(q8), ptr(q_mul), ptr(q_shift), ptr(pool.k_cache(layer_id)),
         ptr(pool.v_cache(layer_id)), ptr(pool.meta(layer_id)), ptr(page_table), page_table.stride(0),
         ptr(kv_lens), ptr(row_seq), ptr(row_limit), ptr(o32), ptr(o8), ptr(om), rows, q_heads, pool.kv_heads,
         pool.num_pages, int(max_kv_len), ptr(ws), ws.numel(), stream())


def decode_attention_int8_paged(q8: torch.Tensor, q_mul: torch.Tensor, q_shift: torch.Tensor,
                                pool: Int8PagedKVCache, layer_id: int, page_table: torch.Tensor,
                                kv_lens: torch.Tensor, max_kv_len: int, *, out_q15: bool = True,
                                out_int8: bool = False, cluster: int = 0, impl: str = "auto",
                                workspace: torch.Tensor | None = None, row_order: torch.Tensor | None = None):
    """One decode step of integer attention over the int8 paged pool.

    ``row_order`` (optional int32 [batch]): the batch rows sorted by descending length, e.g.
    ``torch.argsort(kv_lens, descending=True)``, computed once per step by whoever schedules the batch; the
    kernel takes the rows in that order (the result does not depend on it, the run time does).

    ``impl``: "cluster" = one kernel whose CTAs exchange the softmax statistics inside thread-block clusters
    (fastest; a slice's scores must fit in shared memory, which bounds the context at roughly 50k keys for
    four query heads per KV head); "split" = grid-wide passes over a workspace (any context length; the
    workspace is cached per device and stream unless given); "auto" = cluster when it fits, else split.

    q8 int8 [batch, q_heads, 128]; q_mul / q_shift int32 [batch, q_heads]; page_table int32
    [batch, pitch] of page ids; kv_lens int32 [batch].  Returns the Q15.16 output int32
    [batch, q_heads, 128] and/or (int8 codes, int32 absmax [batch, q_heads]) per the flags.

    The arithmetic is int8_context_attention_fwd's (kernel/triton/int8_attention_kernels.py:278-383)
    with one (multiplier, shift) per key; it stands in for Int8Backend._forward_decode
    (attention/triton_int8.py:155-176).
    """
    if q8.dtype != torch.int8:
        raise TypeError(f"q8 must be int8, got {q8.dtype}")
    if q8.ndim != 3 or q8.shape[-1] != HEAD_DIM:
        raise ValueError(f"q8 must be [batch, q_heads, {HEAD_DIM}], got shape {tuple(q8.shape)}")
    require_cuda(q8, q_mul, q_shift, page_table, kv_lens)
    batch, q_heads, _ = q8.shape
    c = lambda t: t.to(torch.int32).contiguous()
    q8 = q8.contiguous()
    q_mul, q_shift, page_table, kv_lens = c(q_mul), c(q_shift), c(page_table), c(kv_lens)
    if page_table.ndim != 2 or page_table.shape[0] != batch:
        raise ValueError(f"page_table must be [batch, pitch], got shape {tuple(page_table.shape)}")
    o32 = torch.empty((batch, q_heads, HEAD_DIM), dtype=torch.int32, device=q8.device) if out_q15 else None
    o8 = torch.empty((batch, q_heads, HEAD_DIM), dtype=torch.int8, device=q8.device) if out_int8 else None
    om = torch.empty((batch, q_heads), dtype=torch.int32, device=q8.device) if out_int8 else None
    if impl == "auto":
        impl = "cluster" if _cluster_fits(q_heads // pool.kv_heads, max_kv_len) else "split"
    if batch == 0:
        pass
    elif impl == "split":
        _paged_ws(q8, q_mul, q_shift, pool, layer_id, page_table, kv_lens, None, None, o32, o8, om, batch, q_heads,
                  max_kv_len, workspace)
    else:
        call("b200_attn_decode", ptr(q8), ptr(q_mul), ptr(q_shift), ptr(pool.k_cache(layer_id)),
             ptr(pool.v_cache(layer_id)), ptr(pool.meta(layer_id)), ptr(page_table), page_table.stride(0),
             ptr(kv_lens), ptr(None if row_order is None else row_order.to(torch.int32).contiguous()), ptr(o32), ptr(o8),
             ptr(om), batch, q_heads, pool.kv_heads, pool.num_pages, int(max_kv_len), int(cluster), stream())
    if out_q15 and out_int8:
        return o32, o8, om
    return o32 if out_q15 else (o8, om)


def prefill_attention_int8_paged(q8: torch.Tensor, q_mul: torch.Tensor, q_shift: torch.Tensor, pool: Int8PagedKVCache,
                                 layer_id: int, page_table: torch.Tensor, kv_lens: torch.Tensor, q_lens: torch.Tensor,
                                 max_kv_len: int, max_q_len: int, *, out_q15: bool = True, out_int8: bool = False,
                                 q_start: torch.Tensor | None = None):
    """Causal attention of newly appended tokens over the cached prefix plus themselves, tiled: one CTA per
    (sequence, KV head, tile of new tokens) streams the keys once per pass instead of once per query row.

    q8 int8 [sum(q_lens), q_heads, 128] with the sequences back to back; kv_lens int32 [batch] count the new
    tokens too (they must already be stored in the pool); q_lens int32 [batch]; ``max_q_len`` bounds every
    q_lens[i] and ``max_kv_len`` every kv_lens[i] (host integers: they size the grid and shared memory, nothing is
    read back from the device).  ``q_start`` (optional int32 [batch]): the row of each sequence's first new token,
    by default the exclusive prefix sum of q_lens.  The i-th of the n new tokens of a sequence with L keys sees
    keys 0 .. L-n+i.  Stands in for Int8Backend._forward_prefill (attention/triton_int8.py:178-212) ->
    int8_context_attention_fwd (kernel/triton/int8_attention_kernels.py:229-383); unlike the reference it attends
    the cached prefix.
    """
    if q8.dtype != torch.int8:
        raise TypeError(f"q8 must be int8, got {q8.dtype}")
    if q8.ndim != 3 or q8.shape[-1] != HEAD_DIM:
        raise ValueError(f"q8 must be [tokens, q_heads, {HEAD_DIM}], got shape {tuple(q8.shape)}")
    require_cuda(q8, q_mul, q_shift, page_table, kv_lens, q_lens, q_start)
    rows, q_heads, _ = q8.shape
    c = lambda t: t.to(torch.int32).contiguous()
    q8 = q8.contiguous()
    q_mul, q_shift, page_table, kv_lens, q_lens = c(q_mul), c(q_shift), c(page_table), c(kv_lens), c(q_lens)
    batch = kv_lens.shape[0]
    if page_table.ndim != 2 or page_table.shape[0] != batch or q_lens.shape[0] != batch:
        raise ValueError(f"page_table [batch, pitch], kv_lens and q_lens [batch] expected, got {tuple(page_table.shape)}, "
                         f"{tuple(kv_lens.shape)}, {tuple(q_lens.shape)}")
    if q_start is None:
        q_start = torch.cumsum(q_lens, 0, dtype=torch.int32) - q_lens
    q_start = c(q_start)
    o32 = torch.empty((rows, q_heads, HEAD_DIM), dtype=torch.int32, device=q8.device) if out_q15 else None
    o8 = torch.empty((rows, q_heads, HEAD_DIM), dtype=torch.int8, device=q8.device) if out_int8 else None
    om = torch.empty((rows, q_heads), dtype=torch.int32, device=q8.device) if out_int8 else None
    if rows > 0 and batch > 0:
        call("b200_attn_prefill", ptr(q8), ptr(q_mul), ptr(q_shift), ptr(pool.k_cache(layer_id)), ptr(pool.v_cache(layer_id)),
             ptr(pool.meta(layer_id)), ptr(page_table), page_table.stride(0), ptr(kv_lens), ptr(q_lens), ptr(q_start),
             ptr(o32), ptr(o8), ptr(om), batch, int(min(max_q_len, rows)), q_heads, pool.kv_heads, pool.num_pages,
             int(max_kv_len), stream())
    if out_q15 and out_int8:
        return o32, o8, om
    return o32 if out_q15 else (o8, om)


def extend_attention_int8_paged(q8: torch.Tensor, q_mul: torch.Tensor, q_shift: torch.Tensor,
                                pool: Int8PagedKVCache, layer_id: int, page_table: torch.Tensor,
                                kv_lens: torch.Tensor, q_lens: torch.Tensor, max_kv_len: int, *,
                                out_q15: bool = True, out_int8: bool = False, cluster: int = 0,
                                impl: str = "auto", workspace: torch.Tensor | None = None):
    """Causal attention of newly appended tokens over the cached prefix plus themselves.

    q8 int8 [sum(q_lens), q_heads, 128] with the sequences back to back; kv_lens int32 [batch] count the
    new tokens too (they must already be stored in the pool); q_lens int32 [batch].  The i-th of the n new
    tokens of a sequence with L keys sees keys 0 .. L-n+i.  Stands in for Int8Backend._forward_prefill
    (attention/triton_int8.py:178-212) -> int8_context_attention_fwd
    (kernel/triton/int8_attention_kernels.py:229-383); unlike the reference it attends the cached prefix.

    ``impl``: "tiled" = `prefill_attention_int8_paged` (the default: keys are streamed once per tile of new
    tokens); "cluster" = the decode kernel launched once per query row, "split" = its workspace passes (each row
    re-reads its keys: only for a handful of new tokens per sequence).  All three give the same bits.
    """
    if q8.dtype != torch.int8:
        raise TypeError(f"q8 must be int8, got {q8.dtype}")
    if q8.ndim != 3 or q8.shape[-1] != HEAD_DIM:
        raise ValueError(f"q8 must be [tokens, q_heads, {HEAD_DIM}], got shape {tuple(q8.shape)}")
    require_cuda(q8, q_mul, q_shift, page_table, kv_lens, q_lens)
    rows, q_heads, _ = q8.shape
    c = lambda t: t.to(torch.int32).contiguous()
    q8 = q8.contiguous()
    q_mul, q_shift, page_table, kv_lens, q_lens = c(q_mul), c(q_shift), c(page_table), c(kv_lens), c(q_lens)
    total, longest = (int(v) for v in torch.stack((q_lens.sum(), q_lens.max() if q_lens.numel() else q_lens.sum())).tolist())
    if total != rows:
        raise ValueError(f"sum(q_lens)={total} does not match the {rows} query rows")
    if impl in ("auto", "tiled"):
        return prefill_attention_int8_paged(q8, q_mul, q_shift, pool, layer_id, page_table, kv_lens, q_lens, max_kv_len,
                                            longest, out_q15=out_q15, out_int8=out_int8)
    batch = kv_lens.shape[0]
    seq_ids = torch.arange(batch, device=q8.device, dtype=torch.int32)
    row_seq = torch.repeat_interleave(seq_ids, q_lens.to(torch.int64)).to(torch.int32).contiguous()
    starts = torch.cumsum(q_lens, 0, dtype=torch.int32) - q_lens
    rs = row_seq.to(torch.int64)
    within = torch.arange(rows, device=q8.device, dtype=torch.int32) - starts[rs]
    row_limit = (kv_lens[rs] - q_lens[rs] + within + 1).to(torch.int32).contiguous()
    o32 = torch.empty((rows, q_heads, HEAD_DIM), dtype=torch.int32, device=q8.device) if out_q15 else None
    o8 = torch.empty((rows, q_heads, HEAD_DIM), dtype=torch.int8, device=q8.device) if out_int8 else None
    om = torch.empty((rows, q_heads), dtype=torch.int32, device=q8.device) if out_int8 else None
    step = 65535                                            # rows per launch of the row kernels (a grid dimension)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        sl = lambda t: None if t is None else t[r0:r1]
        if impl == "split":
            _paged_ws(q8[r0:r1], q_mul[r0:r1], q_shift[r0:r1], pool, layer_id, page_table, kv_lens, row_seq[r0:r1], row_limit[r0:r1],
                      sl(o32), sl(o8), sl(om), r1 - r0, q_heads, max_kv_len, workspace)
        else:
            call("b200_attn_extend", ptr(q8[r0:r1]), ptr(q_mul[r0:r1]), ptr(q_shift[r0:r1]), ptr(pool.k_cache(layer_id)),
                 ptr(pool.v_cache(layer_id)), ptr(pool.meta(layer_id)), ptr(page_table), page_table.stride(0),
                 ptr(kv_lens), ptr(row_seq[r0:r1]), ptr(row_limit[r0:r1]), ptr(sl(o32)), ptr(sl(o8)), ptr(sl(om)), r1 - r0, q_heads,
                 pool.kv_heads, pool.num_pages, int(max_kv_len), int(cluster), stream())
    if out_q15 and out_int8:
        return o32, o8, om
    return o32 if out_q15 else (o8, om)


def qkv_rope_quant_store(positions: torch.Tensor, qkv_q15: torch.Tensor, q_heads: int, pool: Int8PagedKVCache,
                         layer_id: int, out_loc: torch.Tensor, cos_sin_cache_q15: torch.Tensor,
                         q_norm_weight: torch.Tensor | None = None, k_norm_weight: torch.Tensor | None = None,
                         with_fwht: bool = True):
    """One launch for everything between the qkv projection and attention: q/k-norm + RoPE + Hadamard rotation,
    the new K/V rows quantised into the pool at ``out_loc``, q quantised per (token, head).

    ``qkv_q15``: int32 [tokens, (q_heads + 2*kv_heads)*128] as the qkv projection leaves it (q | k | v blocks).
    Returns (q8 int8 [tokens, q_heads, 128], q_mul, q_shift int32 [tokens, q_heads]).  Same bits as
    qk_norm_rope_fwht -> pool.store_kv -> per_token_quant_int8_from_q15 -> absmax_to_mul_shift
    (models/utils_integer.py:209-227, attention/triton_int8.py:125)."""
    from ..kernel.pending import PendingLinear
    hk = pool.kv_heads
    if isinstance(qkv_q15, PendingLinear):
        # the qkv linear's accumulators: requantised by the kernel while it loads them (and zeroed behind it)
        pl = qkv_q15
        tokens = pl.acc.shape[0]
        if pl.acc.shape[1] != (q_heads + 2 * hk) * HEAD_DIM:
            raise ValueError(f"qkv width {pl.acc.shape[1]} != (q_heads + 2*kv_heads)*{HEAD_DIM}")
        require_cuda(positions, pl.acc, out_loc, cos_sin_cache_q15, q_norm_weight, k_norm_weight)
        c = lambda t: None if t is None else t.to(torch.int32).contiguous()
        q8 = torch.empty((tokens, q_heads, HEAD_DIM), dtype=torch.int8, device=pl.acc.device)
        q_mul = torch.empty((tokens, q_heads), dtype=torch.int32, device=pl.acc.device)
        q_shift = torch.empty_like(q_mul)
        cache = c(cos_sin_cache_q15)
        if tokens:
            call("b200_qkv_prepare_pending", ptr(c(positions)), ptr(pl.acc), ptr(pl.x_absmax), ptr(pl.weight_mul),
                 ptr(pl.weight_shift), ptr(cache), cache.shape[0], ptr(c(q_norm_weight)), ptr(c(k_norm_weight)),
                 ptr(c(out_loc)), ptr(pool.k_cache(layer_id)), ptr(pool.v_cache(layer_id)), ptr(pool.meta(layer_id)),
                 ptr(q8), ptr(q_mul), ptr(q_shift), tokens, q_heads, hk, pool.num_pages, int(with_fwht), stream())
        return q8, q_mul, q_shift
    if qkv_q15.dtype != torch.int32 or qkv_q15.ndim != 2:
        raise TypeError(f"qkv_q15 must be int32 [tokens, width], got {qkv_q15.dtype} {tuple(qkv_q15.shape)}")
    if qkv_q15.shape[1] != (q_heads + 2 * hk) * HEAD_DIM:
        raise ValueError(f"qkv width {qkv_q15.shape[1]} != (q_heads + 2*kv_heads)*{HEAD_DIM}")
    require_cuda(positions, qkv_q15, out_loc, cos_sin_cache_q15, q_norm_weight, k_norm_weight)
    if qkv_q15.stride(1) != 1 or qkv_q15.stride(0) % 4 or qkv_q15.data_ptr() % 16:
        qkv_q15 = qkv_q15.contiguous()
    tokens, pitch = qkv_q15.shape[0], qkv_q15.stride(0)
    qd, kd = q_heads * HEAD_DIM, hk * HEAD_DIM
    q, k, v = qkv_q15[:, :qd], qkv_q15[:, qd:qd + kd], qkv_q15[:, qd + kd:]
    c = lambda t: None if t is None else t.to(torch.int32).contiguous()
    q8 = torch.empty((tokens, q_heads, HEAD_DIM), dtype=torch.int8, device=qkv_q15.device)
    q_mul = torch.empty((tokens, q_heads), dtype=torch.int32, device=qkv_q15.device)
    q_shift = torch.empty_like(q_mul)
    cache = c(cos_sin_cache_q15)
    if tokens:
        call("b200_qkv_prepare_q15", ptr(c(positions)), ptr(q), pitch, ptr(k), pitch, ptr(v), pitch, ptr(cache),
             cache.shape[0], ptr(c(q_norm_weight)), ptr(c(k_norm_weight)), ptr(c(out_loc)), ptr(pool.k_cache(layer_id)),
             ptr(pool.v_cache(layer_id)), ptr(pool.meta(layer_id)), ptr(q8), ptr(q_mul), ptr(q_shift), tokens, q_heads, hk,
             pool.num_pages, int(with_fwht), stream())
    return q8, q_mul, q_shift


def quantize_per_tensor_int8_ms(x: torch.Tensor):
    """Per-tensor int8 quantisation with a (multiplier, shift) scale: same name, arguments and results as the
    reference's quantiser of the prefill path (kernel/triton/int8_attention_kernels.py:41-53): returns
    (int8 codes of x's shape, multiplier, shift) with 0-dim int32 tensors, value ~ code * multiplier / 2**shift.
    ``x`` must be bfloat16 (what the reference's backend passes, attention/triton_int8.py:139-140)."""
    if x.dtype != torch.bfloat16:
        raise TypeError(f"x must be bfloat16, got {x.dtype}")
    require_cuda(x)
    xc = x.contiguous()
    codes = torch.empty(xc.shape, dtype=torch.int8, device=xc.device)
    ms = torch.empty(2, dtype=torch.int32, device=xc.device)
    word = torch.empty(1, dtype=torch.int32, device=xc.device)
    if xc.numel():
        call("b200_quantize_per_tensor_int8_ms", ptr(xc), xc.numel(), ptr(codes), ptr(ms), ptr(word), stream())
    return codes, ms[0], ms[1]
