"""Tensor parallelism on real GPUs: a decoder layer split over two ranks (NCCL) must give the bits of one GPU.
Needs two visible GPUs; skipped otherwise."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

HQ, HK, HID, INTER = 16, 8, 1024, 3072


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs():
    from tests.layer_util import build, make_weights, rope_cache
    rng = np.random.default_rng(0)
    kv_lens, q_lens = [16, 32, 64, 128], [1, 1, 1, 1]
    w = make_weights(rng)
    cache = rope_cache()
    ref_pool, pre, tables, table, positions, out_loc = build(rng, kv_lens, q_lens, 32)
    T = sum(q_lens)
    x = np.clip(np.rint(rng.normal(0, 2**15, (T, HID))), -(2**23), 2**23).astype(np.int32)
    res = np.clip(np.rint(rng.normal(0, 2**15, (T, HID))), -(2**23), 2**23).astype(np.int32)
    return w, cache, pre, table, positions, out_loc, kv_lens, x, res


def _run_layer(rank, world, comm, mode="nccl"):
    """Build this rank's shard of the layer and run one decode step; world == 1 is the single-GPU layer.
    ``mode``: "nccl" = all-reduce after the GEMM; "fused" = the row-parallel GEMMs sum their accumulators over
    peer memory inside the kernel (symmetric-memory barrier); "exchange" = no collective call at all."""
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger
    from tests.layer_util import device_layer_weights, shard_layer_weights
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    w, cache, pre, table, positions, out_loc, kv_lens, x, res = _inputs()
    hq, hk, inter = HQ // world, HK // world, INTER // world
    weights = shard_layer_weights(w, rank, world) if world > 1 else device_layer_weights(w)
    pool = Int8PagedKVCache(hk, 1, 128, 32, "cuda")
    for b, (k8, v8, km, ks, vm, vs, l) in pre.items():
        sl = slice(rank * hk, (rank + 1) * hk)
        pool.store_codes(d(k8[:, sl]), d(v8[:, sl]), d(km[:, sl]), d(ks[:, sl]), d(vm[:, sl]), d(vs[:, sl]), d(l), 0)
    bufs = exch = None
    if mode == "fused":
        from mini_sgl_integer_b200.layers.tp_linear import PeerReduceBuffers
        bufs = PeerReduceBuffers(comm, 8, HID, "cuda")
    if mode == "exchange":
        from mini_sgl_integer_b200.layers.tp_linear import TpExchange
        exch = TpExchange(comm, 8, HID, "cuda")
    layer = Qwen3DecoderLayerInteger(0, hq, hk, HID, inter, weights, d(cache), pool, comm=comm, peer_buffers=bufs, exchange=exch)
    batch = AttnBatch(d(positions), d(out_loc), d(table), d(np.asarray(kv_lens, np.int32)), None, 128)
    out, resid = layer.forward_q15(d(x), d(res), batch)
    if mode != "nccl":                          # more rounds on the same inputs: both halves of the buffers get reused
        for _ in range(3):
            out2, _ = layer.forward_q15(d(x), d(res), batch)
            assert torch.equal(out2, out)
    torch.cuda.synchronize()
    if exch is not None:
        assert exch.status() == 0, "a cross-rank wait ran out"
    return out.cpu().numpy(), resid.cpu().numpy()


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    out, resid = _run_layer(rank, world, DistributedCommunicator())
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), out=out, resid=resid)
    dist.barrier()
    out, resid = _run_layer(rank, world, DistributedCommunicator(), mode="fused")
    np.savez(os.path.join(out_dir, f"f{rank}.npz"), out=out, resid=resid)
    dist.barrier()
    out, resid = _run_layer(rank, world, DistributedCommunicator(), mode="exchange")
    np.savez(os.path.join(out_dir, f"x{rank}.npz"), out=out, resid=resid)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_layer_equals_one_gpu(tmp_path):
    """NCCL all-reduce after the GEMM, the sum done by the GEMM kernel over peer memory, and the exchange without any
    collective call: all give one GPU's bits."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    want_out, want_res = _run_layer(0, 1, None)
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for kind in "rfx":
        for r in range(2):
            z = np.load(tmp_path / f"{kind}{r}.npz")
            assert np.array_equal(z["out"], want_out), f"{kind} rank {r}: layer output differs from one GPU"
            assert np.array_equal(z["resid"], want_res)


# ---------------------------------------------------------------------------------------------- whole model
M_L, M_HID, M_HQ, M_HK, M_INTER, M_VOCAB = 2, 256, 4, 2, 512, 1000


def _model_case():
    rng = np.random.default_rng(8)
    prompt_lens = [7, 20]
    table = rng.permutation(8).astype(np.int32).reshape(2, 4)
    ids = rng.integers(0, M_VOCAB, sum(prompt_lens)).astype(np.int32)
    positions = np.concatenate([np.arange(n) for n in prompt_lens]).astype(np.int32)
    out_loc = np.concatenate([table[b][np.arange(n) // 16] * 16 + np.arange(n) % 16 for b, n in enumerate(prompt_lens)]).astype(np.int32)
    return prompt_lens, table, ids, positions, out_loc


def _run_model(rank, world, comm, steps=3, exchange=False, graph=False):
    """Prefill two prompts and decode `steps` tokens greedily; this rank's shard of every weight.  ``exchange``: the
    decode steps run without any collective call (replicated embedding, exchange block); ``graph``: they are
    replayed from a CUDA graph captured on every rank."""
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.distributed import shard_cols, shard_rows
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, _Linear
    from mini_sgl_integer_b200.models import DecodeBatch, Qwen3ForCausalLMInteger, Qwen3IntegerConfig, random_weights
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    full = Qwen3IntegerConfig(M_L, M_HID, M_HQ, M_HK, M_INTER, M_VOCAB, max_pos=128)
    w = random_weights(full, seed=21)                          # the same full weights on every rank
    hq, hk, inter, vs = M_HQ // world, M_HK // world, M_INTER // world, M_VOCAB // world
    if world > 1:
        def rows(l, idx):
            return _Linear(l.weight[idx].contiguous(), weight_mul=l.weight_mul[idx].contiguous(), weight_shift=l.weight_shift[idx].contiguous())

        def cols(l, per):
            return _Linear(l.weight[:, rank * per:(rank + 1) * per].contiguous(), weight_mul=l.weight_mul, weight_shift=l.weight_shift)
        ar = lambda a, b: torch.arange(a, b, device="cuda")
        for lw in w["layers"]:
            q0, k0, v0 = 0, M_HQ * 128, (M_HQ + M_HK) * 128
            lw["qkv"] = rows(lw["qkv"], torch.cat([ar(q0 + rank * hq * 128, q0 + (rank + 1) * hq * 128),
                                                   ar(k0 + rank * hk * 128, k0 + (rank + 1) * hk * 128),
                                                   ar(v0 + rank * hk * 128, v0 + (rank + 1) * hk * 128)]))
            lw["gate_up"] = rows(lw["gate_up"], torch.cat([ar(rank * inter, (rank + 1) * inter), M_INTER + ar(rank * inter, (rank + 1) * inter)]))
            lw["o"], lw["down"] = cols(lw["o"], hq * 128), cols(lw["down"], inter)
        if exchange:
            w["embed_replicated"] = True
        else:
            w["embed"] = w["embed"][rank * vs:(rank + 1) * vs].contiguous()
        w["lm_head"] = rows(w["lm_head"], ar(rank * vs, (rank + 1) * vs))
        w["vocab_start"] = rank * vs
    cfg = Qwen3IntegerConfig(M_L, M_HID, hq, hk, inter, M_VOCAB, max_pos=128)
    prompt_lens, table, ids, positions, out_loc = _model_case()
    pool = Int8PagedKVCache(hk, M_L, 128, 8, "cuda")
    exch = None
    if exchange and world > 1:
        from mini_sgl_integer_b200.layers.tp_linear import TpExchange
        exch = TpExchange(comm, 8, M_HID, "cuda")
    lm = Qwen3ForCausalLMInteger(cfg, w, pool, comm, exch)
    pl = d(np.asarray(prompt_lens, np.int32))
    pre = AttnBatch(d(positions), d(out_loc), d(table), pl, pl, 64)
    toks = [lm.greedy(d(ids), pre, d((np.cumsum(prompt_lens) - 1).astype(np.int32)))]
    state = DecodeBatch(d(table), pl, 64)
    if not graph:
        for _ in range(steps):
            toks.append(lm.greedy(toks[-1], state.advance()))
    else:
        cur = toks[0].clone()

        def step():
            cur.copy_(lm.greedy(cur, state.advance()))
        snap = state.seq_lens.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()                                          # warm-up outside the capture (writes the KV slot the replay rewrites)
        torch.cuda.current_stream().wait_stream(side)
        state.seq_lens.copy_(snap); cur.copy_(toks[0])
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        state.seq_lens.copy_(snap); cur.copy_(toks[0])
        for _ in range(steps):
            g.replay()
            toks.append(cur.clone())
    torch.cuda.synchronize()
    if exch is not None:
        assert exch.status() == 0, "a cross-rank wait ran out"
    return np.stack([t.cpu().numpy() for t in toks])


def _model_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    toks = _run_model(rank, world, DistributedCommunicator())
    np.save(os.path.join(out_dir, f"m{rank}.npy"), toks)
    dist.barrier()
    toks = _run_model(rank, world, DistributedCommunicator(), exchange=True)
    np.save(os.path.join(out_dir, f"e{rank}.npy"), toks)
    dist.barrier()
    toks = _run_model(rank, world, DistributedCommunicator(), exchange=True, graph=True)
    np.save(os.path.join(out_dir, f"g{rank}.npy"), toks)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_model_tokens_equal_one_gpu(tmp_path):
    """Vocabulary-parallel embedding and lm_head, head / column / row split layers: same greedy tokens as one GPU."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    want = _run_model(0, 1, None)
    mp.spawn(_model_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for kind in "meg":                                   # NCCL; exchange blocks, eager; exchange blocks, CUDA graph
        for r in range(2):
            assert np.array_equal(np.load(tmp_path / f"{kind}{r}.npy"), want), f"{kind} rank {r}: tokens differ from one GPU"
