"""Tensor-parallel host logic on CPU: two gloo ranks run the row-split / column-split recipe with the
oracle's arithmetic and must reproduce the single-rank result bit for bit."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention as oattn
from oracle import fixed_point as ofp
from oracle import linear as olin


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case():
    rng = np.random.default_rng(5)
    T, K, N = 12, 512, 96
    x = rng.integers(-(2**22), 2**22, (T, K)).astype(np.int32)
    w8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    w_mul = rng.integers(2**29, 2**30, N).astype(np.int32)
    w_shift = rng.integers(31, 36, N).astype(np.int32)
    return x, w8, w_mul, w_shift


def _single_rank(x, w8, w_mul, w_shift):
    codes, _, absmax = ofp.per_token_quant_from_q15(x)
    x_mul, x_shift = oattn.absmax_to_mul_shift(absmax[:, 0])
    return olin.requant_q15(olin.int32_accumulate(codes, w8), x_mul, x_shift, w_mul, w_shift)


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from mini_sgl_integer_b200.distributed import (DistributedCommunicator, _reset_tp_info_for_tests, get_tp_info,
                                                    set_tp_info, shard_cols, shard_rows)
    _reset_tp_info_for_tests()
    set_tp_info(rank, world)
    assert get_tp_info().rank == rank and get_tp_info().size == world and get_tp_info().is_primary() == (rank == 0)
    comm = DistributedCommunicator()
    x, w8, w_mul, w_shift = _case()
    # row-parallel: input features split, absmax agreed by a max all-reduce, int32 partial sums added
    xs = shard_cols(torch.from_numpy(x), rank, world).numpy()
    ws = shard_cols(torch.from_numpy(w8), rank, world).numpy()
    _, _, local_absmax = ofp.per_token_quant_from_q15(xs)
    absmax = comm.all_reduce_max(torch.from_numpy(local_absmax[:, 0].copy())).numpy()
    codes = np.clip(np.rint((xs.astype(np.float32) * np.float32(127.0)) / absmax[:, None].astype(np.float32)), -128, 127).astype(np.int8)
    acc = comm.all_reduce(torch.from_numpy(olin.int32_accumulate(codes, ws))).numpy()
    x_mul, x_shift = oattn.absmax_to_mul_shift(absmax)
    row_out = olin.requant_q15(acc, x_mul, x_shift, w_mul, w_shift)
    # column-parallel: output channels split, results gathered
    wr = shard_rows(torch.from_numpy(w8), rank, world).numpy()
    sl = slice(rank * (len(w_mul) // world), (rank + 1) * (len(w_mul) // world))
    col_local = _single_rank(x, wr, w_mul[sl], w_shift[sl])
    col_out = comm.all_gather(torch.from_numpy(np.ascontiguousarray(col_local.T))).numpy().T
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), row=row_out, col=col_out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tp_equals_single_rank(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    want = _single_rank(*_case())
    for r in range(world):
        z = np.load(tmp_path / f"r{r}.npz")
        assert np.array_equal(z["row"], want), f"rank {r}: row-parallel differs from a single rank"
        assert np.array_equal(z["col"], want), f"rank {r}: column-parallel differs from a single rank"


def test_tp_info_guards():
    from mini_sgl_integer_b200.distributed import _reset_tp_info_for_tests, get_tp_info, set_tp_info
    _reset_tp_info_for_tests()
    with pytest.raises(RuntimeError):
        get_tp_info()
    set_tp_info(0, 1)
    with pytest.raises(RuntimeError):
        set_tp_info(0, 1)
    _reset_tp_info_for_tests()


def test_single_process_communicator_is_identity():
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    c = DistributedCommunicator()
    t = torch.arange(6, dtype=torch.int32).reshape(2, 3)
    assert c.all_reduce(t) is t and c.all_gather(t) is t and c.all_reduce_max(t) is t
