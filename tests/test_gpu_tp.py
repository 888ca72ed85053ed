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
    import types
    here = os.path.dirname(os.path.abspath(__file__))
    src = open(os.path.join(here, "test_gpu_layer.py")).read().replace("pytestmark = pytest.mark.gpu", "")
    mod = types.ModuleType("layer_case")
    exec(compile(src, "layer_case", "exec"), mod.__dict__)
    rng = np.random.default_rng(0)
    kv_lens, q_lens = [16, 32, 64, 128], [1, 1, 1, 1]
    w = mod.make_weights(rng)
    cache = mod.rope_cache()
    ref_pool, pre, tables, table, positions, out_loc = mod.build(rng, kv_lens, q_lens, 32)
    T = sum(q_lens)
    x = np.clip(np.rint(rng.normal(0, 2**15, (T, HID))), -(2**23), 2**23).astype(np.int32)
    res = np.clip(np.rint(rng.normal(0, 2**15, (T, HID))), -(2**23), 2**23).astype(np.int32)
    return w, cache, pre, table, positions, out_loc, kv_lens, x, res


def _run_layer(rank, world, comm):
    """Build this rank's shard of the layer and run one decode step; world == 1 is the single-GPU layer."""
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger, _Linear
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    w, cache, pre, table, positions, out_loc, kv_lens, x, res = _inputs()
    hq, hk, inter = HQ // world, HK // world, INTER // world
    rows = lambda a, lo, hi: a[lo:hi]

    def qkv_shard(t):
        wq, wm, ws = t
        q0, k0, v0 = 0, HQ * 128, (HQ + HK) * 128
        idx = np.concatenate([np.arange(q0 + rank * hq * 128, q0 + (rank + 1) * hq * 128),
                              np.arange(k0 + rank * hk * 128, k0 + (rank + 1) * hk * 128),
                              np.arange(v0 + rank * hk * 128, v0 + (rank + 1) * hk * 128)])
        return _Linear(d(wq[idx]), weight_mul=d(wm[idx]), weight_shift=d(ws[idx]))

    def gate_up_shard(t):
        wq, wm, ws = t
        idx = np.concatenate([np.arange(rank * inter, (rank + 1) * inter), INTER + np.arange(rank * inter, (rank + 1) * inter)])
        return _Linear(d(wq[idx]), weight_mul=d(wm[idx]), weight_shift=d(ws[idx]))

    def col_shard(t, per):   # input features
        wq, wm, ws = t
        return _Linear(d(wq[:, rank * per:(rank + 1) * per]), weight_mul=d(wm), weight_shift=d(ws))

    weights = {"qkv": qkv_shard(w["qkv"]), "o": col_shard(w["o"], hq * 128), "gate_up": gate_up_shard(w["gate_up"]),
               "down": col_shard(w["down"], inter), "input_norm": d(w["input_norm"]), "post_norm": d(w["post_norm"]),
               "q_norm": d(w["q_norm"]), "k_norm": d(w["k_norm"])}
    pool = Int8PagedKVCache(hk, 1, 128, 32, "cuda")
    for b, (k8, v8, km, ks, vm, vs, l) in pre.items():
        sl = slice(rank * hk, (rank + 1) * hk)
        pool.store_codes(d(k8[:, sl]), d(v8[:, sl]), d(km[:, sl]), d(ks[:, sl]), d(vm[:, sl]), d(vs[:, sl]), d(l), 0)
    layer = Qwen3DecoderLayerInteger(0, hq, hk, HID, inter, weights, d(cache), pool, comm=comm)
    batch = AttnBatch(d(positions), d(out_loc), d(table), d(np.asarray(kv_lens, np.int32)), None, 128)
    out, resid = layer.forward_q15(d(x), d(res), batch)
    torch.cuda.synchronize()
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
    dist.destroy_process_group()


def test_two_gpu_layer_equals_one_gpu(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    want_out, want_res = _run_layer(0, 1, None)
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        z = np.load(tmp_path / f"r{r}.npz")
        assert np.array_equal(z["out"], want_out), f"rank {r}: layer output differs from one GPU"
        assert np.array_equal(z["resid"], want_res)
