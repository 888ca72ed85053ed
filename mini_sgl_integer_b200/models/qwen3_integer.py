"""Integer-only Qwen3 model on the sm_100a kernels: embedding -> decoder layers -> final norm -> lm_head -> arg-max.

Same composition as ``Qwen3ModelInteger`` / ``Qwen3ForCausalLMInteger`` (models/integer/qwen3_integer.py:83-143):
the embedding row is converted with ``to_fixed`` at the entry (:115-118), the layers pass (x, residual) in Q15.16
(:119-121), the final norm is the fused add + RMSNorm (:122).  The reference leaves the integer domain there
(bf16 ``F.linear`` lm_head, layers/embedding.py:88-110, and a float arg-max, engine/sample.py:74); here the
lm_head is one more W8A8 linear (int8 weights, exact int32 accumulators, fixed-point epilogue) and the greedy
token is an integer arg-max with the lowest index winning ties, so token ids are reproducible bit for bit.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .._lib import call, ptr, require_cuda, stream
from ..attention import Int8PagedKVCache
from ..distributed import DistributedCommunicator
from ..kernel import fixed_point as fp
from ..layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger, _Linear
from ..layers.tp_linear import TpExchange
from ..layers.w8a8_int8 import W8A8Int8LinearMethod


@dataclass
class Qwen3IntegerConfig:
    num_layers: int
    hidden: int
    num_qo_heads: int
    num_kv_heads: int
    inter: int
    vocab: int
    head_dim: int = 128
    rope_base: float = 1000000.0
    max_pos: int = 4096
    hadamard_block: int = 128


def rope_cache_q15(max_pos: int, base: float = 1000000.0, head_dim: int = 128) -> torch.Tensor:
    """cos | sin table in Q1.15, int32 [max_pos, head_dim], built on the host in fp32 like
    RotaryEmbeddingInteger (layers/rotary_integer.py:25-38)."""
    inv = 1.0 / (base ** (torch.arange(0, head_dim, 2, dtype=torch.float) / head_dim))
    fr = torch.einsum("i,j -> ij", torch.arange(max_pos, dtype=torch.float), inv)
    c = torch.cat((fr.cos(), fr.sin()), dim=-1)
    return torch.clamp(torch.round(c * 32768), -32768, 32767).to(torch.int32)


def embedding_to_fixed(table_bf16: torch.Tensor, input_ids: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """to_fixed(embedding(input_ids)) in one pass; ids outside this shard's rows give zeros."""
    if table_bf16.dtype != torch.bfloat16:
        raise TypeError(f"the embedding table must be bfloat16, got {table_bf16.dtype}")
    if input_ids.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"input_ids must be int32 or int64, got {input_ids.dtype}")
    require_cuda(table_bf16, input_ids)
    ids = input_ids.reshape(-1).to(torch.int32).contiguous()
    table = table_bf16.contiguous()
    rows, hidden = ids.numel(), table.shape[1]
    out = torch.empty((rows, hidden), dtype=torch.int32, device=table.device)
    if rows:
        call("b200_embedding_bf16_q15", ptr(table), ptr(ids), ptr(out), rows, hidden, int(vocab_start), table.shape[0], stream())
    return out


def argmax_int32(logits: torch.Tensor, index_offset: int = 0, return_values: bool = False):
    """Row-wise arg-max of int32 logits [rows, n]; the lowest index wins ties."""
    if logits.dtype != torch.int32 or logits.ndim != 2:
        raise TypeError(f"logits must be int32 [rows, n], got {logits.dtype} {tuple(logits.shape)}")
    require_cuda(logits)
    if logits.stride(1) != 1 or logits.stride(0) % 4 or logits.data_ptr() % 16:
        logits = logits.contiguous()
    rows, n = logits.shape
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    val = torch.empty(rows, dtype=torch.int32, device=logits.device) if return_values else None
    if rows:
        call("b200_argmax_i32", ptr(logits), rows, n, logits.stride(0), int(index_offset), ptr(idx), ptr(val), stream())
    return (idx, val) if return_values else idx


def merge_sharded_argmax(values: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """Global arg-max from per-shard results: ``values`` / ``indices`` int32 [shards, rows], the shards' local
    maxima and their GLOBAL vocabulary ids.  The largest value wins, the lowest id among equal values - the
    same token a single arg-max over the whole vocabulary picks."""
    v64 = values.to(torch.int64)
    best = v64.max(dim=0, keepdim=True).values
    ids = torch.where(v64 == best, indices.to(torch.int64), torch.full_like(v64, 2**62))
    return ids.min(dim=0).values.to(torch.int32)


def check_device_status() -> None:
    """Raises if a bounded wait inside a GEMM kernel (operand / accumulator hand-over) or inside a tensor-parallel
    exchange kernel (a peer's signal) has expired since the last check.  Both reads synchronise with the device:
    call it where the step's tokens have just been copied to the host anyway."""
    import ctypes
    st = ctypes.c_int(0)
    call("b200_gemm_status", ctypes.byref(st), 1)
    if st.value:
        raise RuntimeError(f"a wait inside a W8A8 GEMM kernel expired (code {st.value}: 1 loader, 2 MMA issuer, "
                           "3 epilogue, 4 accumulator hand-back); the step's results are not valid")
    call("b200_tp_status", ctypes.byref(st), 1)
    if st.value:
        raise RuntimeError(f"a tensor-parallel wait expired on channel {st.value - 1} (0 absmax, 1 sums, 2 gather): "
                           "a peer rank did not arrive; the step's results are not valid")


class DecodeBatch:
    """Device-resident state of a decode batch: page table, lengths and the per-step views derived from them.

    ``advance()`` runs one small kernel (no host round trip), so a whole decode step - bookkeeping, the layers,
    the arg-max and feeding the token back - can be captured once in a CUDA graph and replayed; this replaces the
    per-request Python loops and ``torch.cat`` of Int8Backend.prepare_metadata (attention/triton_int8.py:214-253).
    """

    def __init__(self, page_table: torch.Tensor, seq_lens: torch.Tensor, max_len: int, first_wave_rows: int = 37):
        require_cuda(page_table, seq_lens)
        self.page_table = page_table.to(torch.int32).contiguous()
        self.seq_lens = seq_lens.to(torch.int32).contiguous().clone()
        self.batch = self.seq_lens.numel()
        self.max_len = int(max_len)
        dev = self.page_table.device
        self.positions = torch.zeros(self.batch, dtype=torch.int32, device=dev)
        self.out_loc = torch.zeros(self.batch, dtype=torch.int32, device=dev)
        self.kv_lens = torch.zeros(self.batch, dtype=torch.int32, device=dev)
        # Every sequence grows by one token per step, so the order by length never changes.  Longest first keeps the
        # tail of the attention launch short; but the CTAs of the FIRST wave start together, and rows of similar
        # length then move through their streaming and scalar phases in lock-step, leaving HBM idle in between.
        # So the first wave (`first_wave_rows`: about 296 CTA slots / KV heads of this rank, 37 rows for 8 heads) is a
        # sample across the whole length range (every batch / first_wave_rows-th row of the sorted list), and the other
        # rows follow longest first (145 -> 139 us on the 8B shape at batch 256).
        desc = torch.argsort(self.seq_lens, descending=True, stable=True)
        step = self.batch // max(first_wave_rows, 1)
        if step >= 2:
            head = desc[0::step][:first_wave_rows]
            keep = torch.ones(self.batch, dtype=torch.bool, device=dev)
            keep[head] = False
            desc = torch.cat((head, desc[keep[desc]]))
        self.row_order = desc.to(torch.int32)

    def advance(self) -> AttnBatch:
        call("b200_decode_prepare", ptr(self.page_table), self.page_table.stride(0), ptr(self.seq_lens), ptr(self.positions),
             ptr(self.out_loc), ptr(self.kv_lens), self.batch, self.max_len, stream())
        return AttnBatch(self.positions, self.out_loc, self.page_table, self.kv_lens, None, self.max_len, self.row_order)


class Qwen3ModelInteger:
    """embed_tokens -> layers -> final norm, activations in Q15.16 / int8 codes."""

    def __init__(self, cfg: Qwen3IntegerConfig, weights: dict, pool: Int8PagedKVCache,
                 comm: Optional[DistributedCommunicator] = None, exchange: Optional[TpExchange] = None):
        """``weights``: "embed" bf16 [vocab, hidden]; "layers": list of per-layer dicts (see
        Qwen3DecoderLayerInteger); "final_norm" int32 [hidden] (Q15.16).

        Under tensor parallelism ``cfg`` carries this rank's head counts and intermediate size, the layer
        weights are this rank's shards, and "embed" holds this rank's block of vocabulary rows starting at
        ``weights["vocab_start"]`` (VocabParallelEmbedding, layers/embedding.py:14-42): ids of other ranks give
        zero rows and the sum over ranks restores the embedding.  With ``weights["embed_replicated"]`` every
        rank holds the whole table and no sum is needed (a decode step then has no collective call when the
        layers run on an ``exchange``)."""
        self.cfg, self.w, self.pool = cfg, weights, pool
        self.comm = comm if comm is not None else DistributedCommunicator()
        self.exchange = exchange
        self.embed_replicated = bool(weights.get("embed_replicated", False))
        self.vocab_start = 0 if self.embed_replicated else int(weights.get("vocab_start", 0))
        self.cache = rope_cache_q15(cfg.max_pos, cfg.rope_base, cfg.head_dim).to(pool.device)
        self.layers = [
            Qwen3DecoderLayerInteger(i, cfg.num_qo_heads, cfg.num_kv_heads, cfg.hidden, cfg.inter, weights["layers"][i],
                                     self.cache, pool, cfg.hadamard_block, comm, exchange=exchange)
            for i in range(cfg.num_layers)
        ]

    def forward(self, input_ids: torch.Tensor, batch: AttnBatch):
        """Returns the final norm's output as int8 codes [tokens, hidden] with the per-token absmax [tokens]."""
        x = embedding_to_fixed(self.w["embed"], input_ids, self.vocab_start)
        if self.comm.size > 1 and not self.embed_replicated:
            x = self.comm.all_reduce(x)
        T = x.shape[0]
        if self.exchange is not None and self.exchange.size > 1 and self.exchange.fits(T, self.cfg.hidden) and self.layers:
            # tensor parallel on an exchange block: the rows of the residual stream have owners, and every row-split
            # linear is finished together with the norm that follows it (Qwen3DecoderLayerInteger.forward_codes)
            codes, _, absmax, _, _ = fp.fused_add_rmsnorm_quant(x, None, self.layers[0].w["input_norm"])
            absmax = absmax.reshape(-1)
            residual = x.contiguous()                       # layer 0's residual is its input; updated in place from here on
            for i, layer in enumerate(self.layers):
                nw = self.layers[i + 1].w["input_norm"] if i + 1 < len(self.layers) else self.w["final_norm"]
                codes, absmax = layer.forward_codes(codes, absmax, residual, batch, nw)
            return codes, absmax
        residual = None
        for layer in self.layers:
            x, residual = layer.forward_q15(x, residual, batch, defer_down=True)
        codes, _, absmax, _, _ = fp.fused_add_rmsnorm_quant(x, residual, self.w["final_norm"])
        return codes, absmax


class Qwen3ForCausalLMInteger:
    def __init__(self, cfg: Qwen3IntegerConfig, weights: dict, pool: Int8PagedKVCache,
                 comm: Optional[DistributedCommunicator] = None, exchange: Optional[TpExchange] = None):
        """``weights`` additionally holds "lm_head": _Linear with int8 [vocab, hidden] and its channel scales
        (under tensor parallelism this rank's vocabulary rows, ParallelLMHead, layers/embedding.py:46-110)."""
        self.model = Qwen3ModelInteger(cfg, weights, pool, comm, exchange)
        self.comm = self.model.comm
        self.exchange = exchange
        self.vocab_start = int(weights.get("vocab_start", 0))          # of the lm_head rows
        self.lm_head = weights["lm_head"]
        self.method = W8A8Int8LinearMethod()

    def forward(self, input_ids: torch.Tensor, batch: AttnBatch, last_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Q15.16 logits int32 [rows, vocab]; ``last_indices`` selects the token rows that need logits
        (the last token of every sequence in a prefill batch, BaseAttnMetadata.get_last_indices)."""
        codes, absmax = self.model.forward(input_ids, batch)
        if last_indices is not None:
            idx = last_indices.to(torch.int64)
            codes, absmax = codes.index_select(0, idx), absmax.index_select(0, idx)
        return self.method.apply_quantised(self.lm_head, codes, absmax)

    check_status = staticmethod(check_device_status)

    def greedy(self, input_ids: torch.Tensor, batch: AttnBatch, last_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Next token ids int32 [rows] (integer arg-max, lowest index on ties).  With a sharded vocabulary every
        rank takes the arg-max of its rows and the (value, id) pairs are merged - two tiny all-gathers instead
        of the reference's all-gather of the full logits (layers/embedding.py:100-110)."""
        logits = self.forward(input_ids, batch, last_indices)
        ranks = self.exchange.size if self.exchange is not None else self.comm.size
        if ranks == 1:
            return argmax_int32(logits)
        idx, val = argmax_int32(logits, index_offset=self.vocab_start, return_values=True)
        rows = idx.shape[0]
        if self.exchange is not None and 2 * rows <= 2 * self.exchange.m_max:
            both = self.exchange.all_gather(torch.stack((val, idx))).view(ranks, 2, rows)   # over peer memory
        else:
            both = self.comm.all_gather(torch.stack((val, idx)).reshape(1, 2, rows))        # [ranks, 2, rows]
        return merge_sharded_argmax(both[:, 0], both[:, 1])


def shard_layer_weights(lw: dict, rank: int, size: int, num_qo_heads: int, num_kv_heads: int, inter: int,
                        head_dim: int = 128) -> dict:
    """Rank ``rank``'s tensor-parallel shard of one layer's weight dict (see Qwen3DecoderLayerInteger): the q | k | v
    and gate | up output channels of the local heads / columns, the input features of o / down, as the reference
    shards and merges them at load time (models/weight.py:12-52)."""
    hq, hk, il = num_qo_heads // size, num_kv_heads // size, inter // size
    dev = lw["qkv"].weight.device
    ar = lambda a, b: torch.arange(a, b, device=dev)

    def rows(l, idx):
        return _Linear(l.weight[idx].contiguous(), weight_mul=l.weight_mul[idx].contiguous(),
                       weight_shift=l.weight_shift[idx].contiguous())

    def cols(l, per):
        return _Linear(l.weight[:, rank * per:(rank + 1) * per].contiguous(), weight_mul=l.weight_mul, weight_shift=l.weight_shift)
    k0, v0 = num_qo_heads * head_dim, (num_qo_heads + num_kv_heads) * head_dim
    out = dict(lw)
    out["qkv"] = rows(lw["qkv"], torch.cat([ar(rank * hq * head_dim, (rank + 1) * hq * head_dim),
                                            ar(k0 + rank * hk * head_dim, k0 + (rank + 1) * hk * head_dim),
                                            ar(v0 + rank * hk * head_dim, v0 + (rank + 1) * hk * head_dim)]))
    out["gate_up"] = rows(lw["gate_up"], torch.cat([ar(rank * il, (rank + 1) * il), inter + ar(rank * il, (rank + 1) * il)]))
    out["o"], out["down"] = cols(lw["o"], hq * head_dim), cols(lw["down"], il)
    return out


def random_weights(cfg: Qwen3IntegerConfig, seed: int, device="cuda", qk_norm: bool = True,
                   generate_on_device: bool = False) -> dict:
    """Seeded random-init weights of the architecture: int8 uniform in [-127, 127], per-channel multipliers in
    [2^29, 2^30) with shift 31, small norm gains so that activations stay inside Q15.16.

    The draw is made on the host (the same values on every machine) unless ``generate_on_device`` is set,
    which is much faster for multi-gigabyte models."""
    dev = torch.device(device)
    gdev = dev if generate_on_device else torch.device("cpu")
    g = torch.Generator(device=gdev).manual_seed(seed)

    def lin(n, k):
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g, device=gdev).to(dev)
        mul = torch.randint(2**29, 2**30, (n,), dtype=torch.int32, generator=g, device=gdev).to(dev)
        return _Linear(w, weight_mul=mul, weight_shift=torch.full((n,), 31, dtype=torch.int32, device=dev))

    ri = lambda lo, hi, n: torch.randint(lo, hi, (n,), dtype=torch.int32, generator=g, device=gdev).to(dev)
    hq, hk, hd = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    layers = []
    for _ in range(cfg.num_layers):
        layers.append({
            "qkv": lin((hq + 2 * hk) * hd, cfg.hidden), "o": lin(cfg.hidden, hq * hd),
            "gate_up": lin(2 * cfg.inter, cfg.hidden), "down": lin(cfg.hidden, cfg.inter),
            "input_norm": ri(2**5, 2**7, cfg.hidden), "post_norm": ri(2**5, 2**7, cfg.hidden),
            "q_norm": ri(2**11, 2**13, hd) if qk_norm else None, "k_norm": ri(2**12, 2**14, hd) if qk_norm else None,
        })
    embed = (torch.randn((cfg.vocab, cfg.hidden), generator=g, device=gdev) * 0.5).to(torch.bfloat16).to(dev)
    return {"embed": embed, "layers": layers, "final_norm": ri(2**5, 2**7, cfg.hidden), "lm_head": lin(cfg.vocab, cfg.hidden)}
