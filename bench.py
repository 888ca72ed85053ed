#!/usr/bin/env python
"""Benchmark of the integer-only W8A8 forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

Default workload ("model"): one greedy DECODE STEP of a Qwen3-8B-shaped integer model (36 layers, hidden 4096,
32 q / 8 kv heads, intermediate 12288, vocabulary 151936; random-init int8 weights) for a batch of 256 sequences
whose contexts are drawn from U[100, 2048] (the spread of prompt + generated lengths of the offline run that
the model configuration names), 16-token int8 KV pages.  One step = bookkeeping on the device, embedding,
36 layers, final norm, integer lm_head, arg-max, the token fed back; captured once in a CUDA graph and replayed.
With N > 1 (torchrun, one rank per GPU) the SAME step is split tensor-parallel over the N ranks - attention by
KV head, qkv / gate_up by output channel, o / down by input feature with the int32 partial sums added over
NVLink peer memory inside the GEMM kernel, lm_head by vocabulary rows - so N measures strong scaling, and a
parity check inside the run compares a tensor-parallel layer with the unsplit layer bit for bit.

The script prints ONE JSON line:
  value        decode tokens/s of the whole job (batch / step time; CUDA events over K graph replays, max over ranks)
  e2e          the same through the public model API with the step's token ids coming from pinned host memory and
               the new ids copied back to it, every step
  roofline     weights + KV bytes a rank must stream per step / step time, against the measured HBM copy peak;
               `dominant_kernel` is the decode attention timed alone on the same batch
  kernels      (N = 1) the other metric components: decode attention GB/s on the attention configuration,
               W8A8 GEMM int8 TOPS at M = 4096 with the library's int8 GEMM beside it, the fused row kernels
  tp_parity    (N > 1) "ok" when the tensor-parallel layer equals the unsplit layer on every rank
  tp32b        (N > 1) one Qwen3-32B-shaped layer, batch 256, contexts U[1024, 8192], split over the same ranks
  cpu_baseline (N = 1) the numpy oracle port of one decoder layer timed on the host cores, scaled to 36 layers

`--impl reference` times only that CPU port (the reference's Python/torch code cannot travel with this
repository; its arithmetic is restated in oracle/).  Other workloads (`--workload attn|gemm|rowops|prefill|
tp_layer|tp_linear`) print the same kind of line for one component.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ATTN_CFG = dict(batch=64, q_heads=32, kv_heads=8, head_dim=128, page=16, ctx_lo=512, ctx_hi=4096, pool_pages=200_000)
MODEL_CFG = dict(layers=36, hidden=4096, q_heads=32, kv_heads=8, inter=12288, vocab=151936, batch=256, ctx_lo=100, ctx_hi=2048)
TP32B_CFG = dict(hidden=5120, q_heads=64, kv_heads=8, inter=25600, layers=64, batch=256, ctx_lo=1024, ctx_hi=8192)
METRIC = "decode tokens/s, integer-only W8A8 Qwen3-8B-shaped model (tensor-parallel over the GPUs)"
# DRAM bytes (read + write) of ONE launch of the decode-attention kernel on the attention configuration, from an
# ncu capture of that kernel; a constant, not measured by this script - see `traffic_source` in the line
ATTN_NCU_TRAFFIC = {"bytes": 334636800, "source": "ncu capture of attn_decode_kernel<4,1> on this workload (dram__bytes_read.sum + dram__bytes_write.sum), not re-measured by this run"}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def env_ranks():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


# ----------------------------------------------------------------------------- clocks sampler
class ClockSampler:
    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.samples = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [s for (t, s) in self.samples if t0 <= t <= t1] or [s for (_, s) in self.samples]
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            parts = [p.strip() for p in r.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ----------------------------------------------------------------------------- CPU oracle legs
def blas_threads() -> int:
    try:
        from threadpoolctl import threadpool_info
        n = [int(i.get("num_threads", 1)) for i in threadpool_info() if i.get("user_api") == "blas"]
        return max(n) if n else 1
    except Exception:
        return 1


def cpu_layer_sample(n_tok: int, seed: int = 0):
    """One decoder layer of the 8B shape through the numpy oracle on `n_tok` decode tokens (contexts drawn like the
    GPU batch).  Returns the seconds of the layer pass."""
    from oracle import layer as olayer
    from tests.layer_util import build, make_weights, rope_cache
    c = MODEL_CFG
    rng = np.random.default_rng(seed)
    kv_lens = [int(v) for v in rng.integers(c["ctx_lo"], c["ctx_hi"] + 1, n_tok)]
    q_lens = [1] * n_tok
    pages = sum((l + 15) // 16 for l in kv_lens) + 4
    key = (n_tok, seed)
    st = _CPU_CACHE.get(key)
    if st is None:
        w = make_weights(rng, c["q_heads"], c["kv_heads"], c["hidden"], c["inter"], wide=True)
        ref_pool, pre, tables, table, positions, out_loc = build(rng, kv_lens, q_lens, pages, c["kv_heads"])
        x = np.clip(np.rint(rng.normal(0, 2**15, (n_tok, c["hidden"]))), -(2**23), 2**23).astype(np.int32)
        res = np.clip(np.rint(rng.normal(0, 2**15, (n_tok, c["hidden"]))), -(2**23), 2**23).astype(np.int32)
        st = (w, rope_cache(c["ctx_hi"] + 16), ref_pool, tables, positions, out_loc, kv_lens, q_lens, x, res)
        _CPU_CACHE[key] = st
    w, cache, ref_pool, tables, positions, out_loc, kv_lens, q_lens, x, res = st
    t0 = time.perf_counter()
    olayer.decoder_layer(x, res, w, cache, ref_pool, positions, out_loc, tables, kv_lens, q_lens, c["q_heads"], c["kv_heads"])
    return time.perf_counter() - t0


_CPU_CACHE: dict = {}
CPU_SAMPLE_TOKENS = 4


def cpu_sample_text(n_tok):
    return (f"one decoder layer of the 8B shape on {n_tok} of the 256 decode tokens (contexts U[100,2048]) through the numpy "
            f"oracle port, scaled to {MODEL_CFG['layers']} layers; embedding, final norm and lm_head not counted")


def run_reference(args) -> None:
    rank, world, _ = env_ranks()
    if rank != 0:
        return
    n_tok = CPU_SAMPLE_TOKENS
    t_wall = time.perf_counter()
    for _ in range(args.warmup):
        cpu_layer_sample(n_tok)
    total = 0.0
    for _ in range(args.steps):
        total += cpu_layer_sample(n_tok)
    per_layer = total / max(args.steps, 1)
    rate = n_tok / (MODEL_CFG["layers"] * per_layer)
    threads = blas_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * per_layer, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": model_config_dict(1, args),
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": threads, "threads_effective": threads,
                         "host_cpus": os.cpu_count(), "kind": "port",
                         "sample": cpu_sample_text(n_tok) + "; one step = one such layer pass"},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_wall,
    }
    print(json.dumps(line))


def model_config_dict(world: int, args) -> dict:
    c = MODEL_CFG
    return {"workload": "Qwen3-8B-shaped integer-only W8A8 model, greedy decode step, batch %d, ctx U[%d,%d], page 16, "
                        "random-init int8 weights" % (args.batch, c["ctx_lo"], c["ctx_hi"]),
            "layers": args.model_layers, "hidden": c["hidden"], "q_heads": c["q_heads"], "kv_heads": c["kv_heads"],
            "inter": c["inter"], "vocab": c["vocab"], "global_batch": args.batch}


# ----------------------------------------------------------------------------- timing helpers
def time_launches(fn, launches: int, warmup: int = 3):
    """Mean and median milliseconds of one call of `fn` on the current stream: CUDA events around the whole run of
    `launches` back-to-back calls (mean) and around every call (median)."""
    import torch
    st = torch.cuda.current_stream()
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(st)
    for _ in range(launches):
        fn()
    e1.record(st)
    torch.cuda.synchronize()
    mean = e0.elapsed_time(e1) / launches
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(min(launches, 100))]
    for a, b in evs:
        a.record(st); fn(); b.record(st)
    torch.cuda.synchronize()
    return mean, float(np.median([a.elapsed_time(b) for a, b in evs]))


def fill_pool_random(pool, layers, gen, v_shift=(33, 38)):
    import torch
    dev = pool.device
    for i in range(layers):
        pool.k_cache(i).copy_(torch.randint(-127, 128, pool.k_cache(i).shape, dtype=torch.int8, device=dev, generator=gen))
        pool.v_cache(i).copy_(torch.randint(-127, 128, pool.v_cache(i).shape, dtype=torch.int8, device=dev, generator=gen))
        meta = pool.meta(i)
        P, H = meta.shape[0], meta.shape[1]
        meta[:, :, 0:32] = torch.randint(2**30, 2**31, (P, H, 32), dtype=torch.int64, device=dev, generator=gen).to(torch.int32)
        meta[:, :, 32:36] = torch.randint(35, 39, (P, H, 16), dtype=torch.int8, device=dev, generator=gen).view(torch.int32)
        meta[:, :, 36:40] = torch.randint(v_shift[0], v_shift[1], (P, H, 16), dtype=torch.int8, device=dev, generator=gen).view(torch.int32)


def page_tables(rng, lens, pitch, extra_pages=0):
    """Disjoint page-id runs out of a random permutation of the pool: (table [B, pitch] int32, pool pages)."""
    n_pg = (np.asarray(lens) + 15) // 16 + extra_pages
    P = int(n_pg.sum()) + 8
    perm = rng.permutation(P)
    table = np.zeros((len(lens), pitch), dtype=np.int32)
    off = 0
    for b, n in enumerate(n_pg):
        table[b, :n] = perm[off:off + n]; off += n
    return table, P


# ----------------------------------------------------------------------------- component benchmarks (return dicts)
def attn_micro(dev, launches=200, pool_pages=None, cluster=0, seed=0):
    """The attention configuration: batch 64, 32 q / 8 kv heads, ctx U[512, 4096], 200k-page pool."""
    import torch
    from mini_sgl_integer_b200 import _lib
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    w = ATTN_CFG
    B, Hq, Hkv, D = w["batch"], w["q_heads"], w["kv_heads"], w["head_dim"]
    P = pool_pages or w["pool_pages"]
    lens = np.random.default_rng(seed).integers(w["ctx_lo"], w["ctx_hi"] + 1, B)
    g = torch.Generator(device=dev).manual_seed(1000 + seed)
    pool = Int8PagedKVCache(Hkv, 1, D, P, dev)
    fill_pool_random(pool, 1, g)
    rng = np.random.default_rng(2000 + seed)
    perm = rng.permutation(P)
    n_pg = (lens + 15) // 16
    pitch = (w["ctx_hi"] + 15) // 16
    table = np.zeros((B, pitch), dtype=np.int32)
    off = 0
    for b in range(B):
        table[b, : n_pg[b]] = perm[off:off + n_pg[b]]; off += n_pg[b]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    q = t(rng.integers(-127, 128, (B, Hq, D), dtype=np.int8))
    qm, qs = t(rng.integers(2**30, 2**31, (B, Hq)).astype(np.int32)), t(rng.integers(43, 46, (B, Hq)).astype(np.int32))
    d_table, d_lens = t(table), t(lens.astype(np.int32))
    order = t(np.argsort(-lens, kind="stable").astype(np.int32))
    out = torch.empty((B, Hq, D), dtype=torch.int8, device=dev)
    absmax = torch.empty((B, Hq), dtype=torch.int32, device=dev)
    p, sp = _lib.ptr, _lib.stream()

    def launch():
        _lib.call("b200_attn_decode", p(q), p(qm), p(qs), p(pool.k_cache(0)), p(pool.v_cache(0)), p(pool.meta(0)), p(d_table),
                  pitch, p(d_lens), p(order), None, p(out), p(absmax), B, Hq, Hkv, P, w["ctx_hi"], cluster, sp)
    mean, median = time_launches(launch, launches)
    alg = int((lens.astype(np.int64) * Hkv * D * 2 + lens.astype(np.int64) * Hkv * 10 + n_pg.astype(np.int64) * 4).sum() + B * Hq * D * 2)
    peak, how = measured_peak()
    gbs = alg / (mean * 1e-3) / 1e9
    return {"workload": "batch 64, 32q/8kv heads, head_dim 128, page 16, ctx U[512,4096], %d-page pool" % P,
            "kernel_ms": mean, "kernel_ms_median": median, "launches_timed": launches, "GBs": gbs, "frac": gbs / peak,
            "frac_of_8TBs": gbs / 8000.0, "peak": peak, "peak_source": how, "algorithmic_bytes": alg,
            "tok_s": B / (mean * 1e-3), "traffic": ATTN_NCU_TRAFFIC["bytes"] if P == w["pool_pages"] else None,
            "traffic_source": ATTN_NCU_TRAFFIC["source"], "sum_ctx": int(lens.sum())}


def gemm_micro(dev, M=4096, launches=20):
    """The four linears of the 8B-shaped layer at the given M: int8 TOPS, and the library's int8 GEMM beside them."""
    import torch
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    out = {}
    g = torch.Generator(device=dev).manual_seed(3)
    for name, (N, K) in {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}.items():
        x8 = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
        w8 = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
        xm = torch.randint(2**30, 2**31 - 1, (M,), dtype=torch.int64, device=dev, generator=g).to(torch.int32)
        xs = torch.full((M,), 40, dtype=torch.int32, device=dev)
        wm = torch.randint(2**29, 2**30, (N,), dtype=torch.int32, device=dev, generator=g)
        ms, _ = time_launches(lambda: int8_gemm_q15(x8, xm, xs, w8, wm), launches)
        lib = float("nan")
        if M > 16:
            lib, _ = time_launches(lambda: torch._int_mm(x8, w8.t()), launches)
        out[name] = {"N": N, "K": K, "ms": ms, "TOPS": 2 * M * N * K / ms / 1e9,
                     "library_int_mm_TOPS": 2 * M * N * K / lib / 1e9, "weight_GBs": N * K / ms / 1e6}
    tot_ops = sum(2 * M * v["N"] * v["K"] for v in out.values())
    tot_ms = sum(v["ms"] for v in out.values())
    tops = tot_ops / tot_ms / 1e9
    lib_ms = sum(2 * M * v["N"] * v["K"] / v["library_int_mm_TOPS"] / 1e9 for v in out.values())
    return {"M": M, "TOPS": tops, "frac_nominal": tops / 4500.0, "nominal_peak_TOPS": 4500.0,
            "frac_of_int_mm": lib_ms / tot_ms if lib_ms == lib_ms else None, "ms": tot_ms, "shapes": out,
            "note": "int8 tensor peak is not in MEASURED_PEAKS.json: nominal dense 4.5 POPS and torch._int_mm on the same box"}


def rowops_micro(dev, rows=16384, launches=20):
    """The row-kernel configuration: add+RMSNorm+quant (A) on [rows, 5120], SiLU*up+FWHT128+quant (B) on [rows, 2*17408]."""
    import torch
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    T, H, I = rows, 5120, 17408
    g = torch.Generator(device=dev).manual_seed(0)
    clip = lambda t: t.round().clamp(-(2**23), 2**23).to(torch.int32)
    x = clip(torch.randn(T, H, device=dev, generator=g) * 4096.0)
    r = clip(torch.randn(T, H, device=dev, generator=g) * 4096.0)
    w = torch.randint(2**13, 2**15 + 1, (H,), device=dev, dtype=torch.int32, generator=g)
    gu = (torch.randn(T, 2 * I, device=dev, generator=g) * 2.0**17).round().to(torch.int32)
    ms_a, _ = time_launches(lambda: fp.fused_add_rmsnorm_quant(x, r, w), launches)
    ms_b, _ = time_launches(lambda: fp.silu_mul_fwht_quant(gu, 128), launches)
    bytes_a, bytes_b = T * (13 * H + 8), T * (9 * I + 8)
    peak, how = measured_peak()
    tot = ms_a + ms_b
    rec = {"rows": T, "A_add_rmsnorm_quant": {"ms": ms_a, "GBs": bytes_a / ms_a / 1e6, "frac": bytes_a / ms_a / 1e6 / peak, "bytes": bytes_a},
           "B_silu_fwht_quant": {"ms": ms_b, "GBs": bytes_b / ms_b / 1e6, "frac": bytes_b / ms_b / 1e6 / peak, "bytes": bytes_b},
           "A_plus_B": {"ms": tot, "GBs": (bytes_a + bytes_b) / tot / 1e6, "frac": (bytes_a + bytes_b) / tot / 1e6 / peak},
           "peak": peak, "peak_source": how}
    return rec, (x, r, w, gu)


PREFILL_NCU_TRAFFIC_BYTES = 52994560 + 80477696      # one launch of the prefill workload below, from its ncu capture


def prefill_micro(dev, launches=5):
    """Prefill attention on prompts of the offline run's shape: 16 prompts of U[100, 1024] tokens, 32 q / 8 kv heads."""
    import torch
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.attention import ops as aops
    if not hasattr(aops, "prefill_attention_int8_paged"):
        return None
    rng = np.random.default_rng(5)
    B, Hq, Hkv = 16, 32, 8
    lens = rng.integers(100, 1025, B)
    table, P = page_tables(rng, lens, 64)
    pool = Int8PagedKVCache(Hkv, 1, 128, P, dev)
    fill_pool_random(pool, 1, torch.Generator(device=dev).manual_seed(6))
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    T = int(lens.sum())
    q = t(rng.integers(-127, 128, (T, Hq, 128), dtype=np.int8))
    qm, qs = t(rng.integers(2**30, 2**31, (T, Hq)).astype(np.int32)), t(rng.integers(43, 46, (T, Hq)).astype(np.int32))
    d_table, d_lens = t(table), t(lens.astype(np.int32))
    fn = lambda: aops.prefill_attention_int8_paged(q, qm, qs, pool, 0, d_table, d_lens, d_lens, 1024, int(lens.max()))
    ms, med = time_launches(fn, launches)
    pairs = float((lens.astype(np.float64) * (lens + 1) / 2).sum()) * Hq
    ops = pairs * 128 * 2 * 2                                   # QK^T and PV, causal half
    kv_bytes = float(lens.sum()) * Hkv * 266
    algo_bytes = kv_bytes + T * Hq * 128 * (1 + 4) + T * Hq * 8          # K/V once, int8 queries in, Q15.16 rows out, scales
    return {"workload": "16 prompts of U[100,1024] tokens, 32q/8kv heads, causal, no cached prefix", "tokens": T, "ms": ms,
            "ms_median": med, "tok_s": T / (ms * 1e-3), "int8_TOPS_algorithmic": ops / ms / 1e9,
            "kv_bytes_once": kv_bytes, "score_elements": pairs, "algorithmic_bytes": algo_bytes,
            "traffic": PREFILL_NCU_TRAFFIC_BYTES, "traffic_over_algorithmic": PREFILL_NCU_TRAFFIC_BYTES / algo_bytes,
            "traffic_source": "ncu capture of attn_prefill_kernel<4> on this workload (dram__bytes_read.sum + dram__bytes_write.sum), "
                              "not re-measured by this run"}


# ----------------------------------------------------------------------------- the model step (default workload)
def build_parity_case(dev, comm, exch, full_layer0, cache, rank, world):
    """A tensor-parallel layer against the unsplit layer on 8 decode tokens: identical seeded inputs on every rank,
    KV pools that hold the same codes (this rank's heads), outputs compared bit for bit.  Returns True / False."""
    import torch
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger
    from mini_sgl_integer_b200.models import shard_layer_weights
    c = MODEL_CFG
    HID, HQ, HK, INTER = c["hidden"], c["q_heads"], c["kv_heads"], c["inter"]
    rng = np.random.default_rng(77)
    T = 8
    lens = rng.integers(20, 200, T)
    table, P = page_tables(rng, lens, 16)
    g = torch.Generator(device=dev).manual_seed(78)
    pool_full = Int8PagedKVCache(HK, 1, 128, P, dev)
    fill_pool_random(pool_full, 1, g)
    hk = HK // world
    pool_tp = Int8PagedKVCache(hk, 1, 128, P, dev)
    sl = slice(rank * hk, (rank + 1) * hk)
    pool_tp.k_cache(0).copy_(pool_full.k_cache(0)[:, sl]); pool_tp.v_cache(0).copy_(pool_full.v_cache(0)[:, sl])
    pool_tp.meta(0).copy_(pool_full.meta(0)[:, sl])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    out_loc = np.array([table[b, (lens[b] - 1) // 16] * 16 + (lens[b] - 1) % 16 for b in range(T)], dtype=np.int32)
    batch = AttnBatch(t((lens - 1).astype(np.int32)), t(out_loc), t(table), t(lens.astype(np.int32)), None, 256)
    x = (torch.randn(T, HID, device=dev, generator=g) * 30000.0).round().to(torch.int32)
    res = (torch.randn(T, HID, device=dev, generator=g) * 30000.0).round().to(torch.int32)
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    full = Qwen3DecoderLayerInteger(0, HQ, HK, HID, INTER, full_layer0, cache, pool_full, comm=DistributedCommunicator(single=True))
    want, want_res = full.forward_q15(x, res, batch)
    tp = Qwen3DecoderLayerInteger(0, HQ // world, hk, HID, INTER // world, shard_layer_weights(full_layer0, rank, world, HQ, HK, INTER),
                                  cache, pool_tp, comm=comm, exchange=exch)
    ok = True
    for _ in range(3):                                       # three rounds: both halves of the exchange blocks
        got, got_res = tp.forward_q15(x, res, batch)
        ok = ok and bool(torch.equal(got, want)) and bool(torch.equal(got_res, want_res))
    # the form the model step uses: codes in, codes out, every row finished and normalised by its owner
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    next_w = full_layer0["post_norm"]                        # any norm weight will do for the norm after the layer
    w_codes, _, w_absmax, w_res3, _ = fp.fused_add_rmsnorm_quant(want, want_res, next_w)
    in_codes, _, in_absmax, res1, _ = fp.fused_add_rmsnorm_quant(x, res, full_layer0["input_norm"])
    own = exch.owner_rows(T)
    for _ in range(3):
        resid = res1.clone()
        g_codes, g_absmax = tp.forward_codes(in_codes, in_absmax.reshape(-1), resid, batch, next_w)
        ok = ok and bool(torch.equal(g_codes, w_codes)) and bool(torch.equal(g_absmax, w_absmax.reshape(-1)))
        ok = ok and bool(torch.equal(resid[own], w_res3[own]))
    return ok and int(want.abs().max()) > 0


def run_model(args) -> None:
    import torch
    import torch.distributed as dist
    from mini_sgl_integer_b200 import _lib
    from mini_sgl_integer_b200.attention import Int8PagedKVCache, decode_attention_int8_paged
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    from mini_sgl_integer_b200.models import (DecodeBatch, Qwen3ForCausalLMInteger, Qwen3IntegerConfig, check_device_status,
                                              random_weights, rope_cache_q15, shard_layer_weights)

    rank, world, local = env_ranks()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    c = MODEL_CFG
    HID, HQ, HK, INTER, VOCAB, L = c["hidden"], c["q_heads"], c["kv_heads"], c["inter"], c["vocab"], args.model_layers
    if HK % world or VOCAB % world:
        raise SystemExit(f"the model splits over 1, 2, 4 or 8 ranks, not {world}")
    B = args.batch
    comm = DistributedCommunicator()
    exch = TpExchange(comm, max(B, 8), HID, dev) if world > 1 else None
    hq, hk, inter, vs = HQ // world, HK // world, INTER // world, VOCAB // world

    # ---- weights: layer 0, the embedding and the lm_head are drawn at full size with one seed on every rank and
    # sliced (so that the parity check can run the unsplit layer); the other layers are drawn at shard size
    wf = random_weights(Qwen3IntegerConfig(1, HID, HQ, HK, INTER, VOCAB), seed=4, device=dev, generate_on_device=True)
    cache = rope_cache_q15(4096).to(dev)
    tp_parity = None
    if world > 1:
        ok = build_parity_case(dev, comm, exch, wf["layers"][0], cache, rank, world)
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        tp_parity = "ok" if int(flag) == 1 else "mismatch"
        check_device_status()   # a peer that never arrived: every later wait would run out too, so stop at once
    wl = random_weights(Qwen3IntegerConfig(max(L - 1, 0), HID, hq, hk, inter, 128), seed=1000 + rank, device=dev,
                        generate_on_device=True)
    weights = {"embed": wf["embed"], "embed_replicated": True, "final_norm": wf["final_norm"],
               "layers": [shard_layer_weights(wf["layers"][0], rank, world, HQ, HK, INTER)] + wl["layers"]}
    lmh = wf["lm_head"]
    from mini_sgl_integer_b200.layers.decoder_layer import _Linear
    weights["lm_head"] = _Linear(lmh.weight[rank * vs:(rank + 1) * vs].contiguous(), weight_mul=lmh.weight_mul[rank * vs:(rank + 1) * vs].contiguous(),
                                 weight_shift=lmh.weight_shift[rank * vs:(rank + 1) * vs].contiguous())
    weights["vocab_start"] = rank * vs
    del wf, wl, lmh
    torch.cuda.empty_cache()

    # ---- batch and KV pool (same lengths and page ids on every rank; each rank holds its KV heads)
    rng = np.random.default_rng(21)
    lens = rng.integers(c["ctx_lo"], c["ctx_hi"] + 1, B)
    total_steps = 2 * args.warmup + 2 * args.steps + 16
    max_len = int(-(-(int(lens.max()) + total_steps + 1) // 16) * 16)
    table, P = page_tables(rng, lens + total_steps, max_len // 16)
    cfg = Qwen3IntegerConfig(L, HID, hq, hk, inter, VOCAB, max_pos=4096)
    pool = Int8PagedKVCache(hk, L, 128, P, dev)
    fill_pool_random(pool, L, torch.Generator(device=dev).manual_seed(5 + rank), v_shift=(36, 40))
    state = DecodeBatch(torch.from_numpy(table).to(dev), torch.from_numpy(lens.astype(np.int32)).to(dev), max_len,
                        first_wave_rows=max(1, 296 // hk))
    lm = Qwen3ForCausalLMInteger(cfg, weights, pool, comm, exch)
    h_in = torch.from_numpy(rng.integers(0, VOCAB, B).astype(np.int32)).pin_memory()
    h_out = torch.empty(B, dtype=torch.int32).pin_memory()
    cur = h_in.to(dev)

    def step():
        cur.copy_(lm.greedy(cur, state.advance()))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                              # loads modules, sizes attributes (outside the capture)
    torch.cuda.current_stream().wait_stream(side)
    barrier()
    check_device_status()       # a tensor-parallel wait that ran out in the very first step: stop here, not after the run
    calls0 = _lib.CALLS
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    calls_per_step = _lib.CALLS - calls0
    barrier()
    for _ in range(args.warmup):
        graph.replay()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    t_wall0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    t_wall1 = time.perf_counter()
    ms = e0.elapsed_time(e1) / args.steps
    check_device_status()

    # ---- end to end: token ids in from pinned host memory, new ids back to it, every step
    def e2e_step():
        cur.copy_(h_in, non_blocking=True)
        graph.replay()
        h_out.copy_(cur, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h_in.copy_(h_out)
    for _ in range(min(args.warmup, 3)):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_step()
    f1.record()
    barrier()
    e2e_ms = f0.elapsed_time(f1) / args.steps
    check_device_status()
    clocks = sampler.stop(t_wall0, time.perf_counter()) if sampler else None
    lens_after = state.seq_lens.cpu().numpy().astype(np.int64)

    # ---- the dominant kernel on its own: the decode attention of one layer over this batch
    q8 = torch.randint(-127, 128, (B, hq, 128), dtype=torch.int8, device=dev)
    qm = torch.randint(2**30, 2**31, (B, hq), dtype=torch.int64, device=dev).to(torch.int32)
    qs = torch.full((B, hq), 44, dtype=torch.int32, device=dev)
    kv_lens = state.seq_lens.clone()
    rot = [0]

    def attn_launch():
        rot[0] = (rot[0] + 1) % L                            # a different layer's pages every launch: nothing stays in L2
        decode_attention_int8_paged(q8, qm, qs, pool, rot[0], state.page_table, kv_lens, max_len, row_order=state.row_order)
    attn_ms, attn_med = time_launches(attn_launch, 200)
    attn_bytes = int((lens_after * hk * 266 + ((lens_after + 15) // 16) * 4).sum() + B * hq * 128 * 5)

    t = torch.tensor([ms, e2e_ms, attn_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, attn_ms = (float(v) for v in t.tolist())

    per_layer_w = (HQ + 2 * HK) * 128 * HID + HID * HQ * 128 + 2 * INTER * HID + HID * INTER
    w_bytes = (L * per_layer_w + VOCAB * HID) / world
    kv_bytes = float(lens_after.sum()) * hk * 266 * L
    peak, how = measured_peak()
    ach = (w_bytes + kv_bytes) / (ms * 1e-3) / 1e9
    line = None
    if rank == 0:
        line = {
            "metric": METRIC, "value": B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": {**model_config_dict(world, args), "parallelism": f"tp{world}", "per_gpu_tok_s": B / (ms * 1e-3) / world,
                       "mean_ctx": float(lens_after.mean()), "cuda_graph": True,
                       "row_parallel_sum": "in the GEMM kernel over NVLink peer memory; no collective call in the step" if world > 1 else "none (one GPU)",
                       "l2": "weights + KV streamed per step (%.1f GB per GPU) exceed L2" % ((w_bytes + kv_bytes) / 1e9)},
            "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": 4 * B,
                    "d2h_bytes_per_step": 4 * B},
            "gpu_launches": calls_per_step * args.steps,
            "gpu_launches_note": "entry-point calls of libb200int.so captured in one step x steps (a split-K GEMM call is three graph nodes)",
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "traffic_source": "not captured for the whole step; the decode-attention kernel's capture is under kernels.attn_cfg2",
                         "peak_source": how, "weight_bytes_per_gpu": w_bytes, "kv_bytes_per_gpu": kv_bytes,
                         "dominant_kernel": {"name": "attn_decode_kernel", "kernel_ms": attn_ms, "kernel_ms_median": attn_med,
                                             "launches_timed": 200, "algorithmic_bytes": attn_bytes,
                                             "achieved": attn_bytes / attn_ms / 1e6, "frac": attn_bytes / attn_ms / 1e6 / peak,
                                             "share_of_step": attn_ms * L / ms}},
            "clocks": clocks, "wall_s": t_wall1 - t_wall0,
        }
        if tp_parity is not None:
            line["tp_parity"] = tp_parity
    # ---- free the model before the component runs
    del lm, pool, weights, state, graph
    torch.cuda.empty_cache()
    if world > 1 and not args.no_tp32b:
        rec = tp32b_layer(dev, comm, rank, world, args)
        if rank == 0:
            line["tp32b"] = rec
    if world == 1 and not args.no_kernels:
        kern = {}
        kern["attn_cfg2"] = attn_micro(dev, 200)
        kern["gemm_m4096"] = gemm_micro(dev, 4096, 20)
        rec, tensors = rowops_micro(dev, 16384, 20)
        kern["rowops_cfg3"] = rec
        del tensors
        torch.cuda.empty_cache()
        pre = prefill_micro(dev)
        if pre is not None:
            kern["prefill_attn"] = pre
        line["kernels"] = kern
        n_tok = CPU_SAMPLE_TOKENS
        cpu_layer_sample(n_tok)
        dt = min(cpu_layer_sample(n_tok), cpu_layer_sample(n_tok))
        threads = blas_threads()
        line["cpu_baseline"] = {"value": n_tok / (L * dt), "unit": "tokens/s", "cores": threads, "threads_effective": threads,
                                "host_cpus": os.cpu_count(), "kind": "port",
                                "sample": cpu_sample_text(n_tok) + " (%.2f s per layer pass, best of two)" % dt}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def tp32b_layer(dev, comm, rank, world, args):
    """One Qwen3-32B-shaped decoder layer, decode batch 256, contexts U[1024, 8192], split over the ranks; replayed
    from a CUDA graph.  tokens/s are quoted for the 64-layer model (64 x this layer)."""
    import torch
    import torch.distributed as dist
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange
    from mini_sgl_integer_b200.models import Qwen3IntegerConfig, check_device_status, random_weights, rope_cache_q15
    c = TP32B_CFG
    HID, HQ, HK, INTER, LAYERS, B = c["hidden"], c["q_heads"], c["kv_heads"], c["inter"], c["layers"], c["batch"]
    hq, hk, inter = HQ // world, HK // world, INTER // world
    w = random_weights(Qwen3IntegerConfig(1, HID, hq, hk, inter, 128), seed=9, device=dev, generate_on_device=True)["layers"][0]
    rng = np.random.default_rng(11)
    lens = rng.integers(c["ctx_lo"], c["ctx_hi"] + 1, B)
    table, P = page_tables(rng, lens, 512)
    pool = Int8PagedKVCache(hk, 1, 128, P, dev)
    fill_pool_random(pool, 1, torch.Generator(device=dev).manual_seed(12), v_shift=(36, 40))
    out_loc = np.array([table[b, (lens[b] - 1) // 16] * 16 + (lens[b] - 1) % 16 for b in range(B)], dtype=np.int32)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    exch = TpExchange(comm, B, HID, dev) if world > 1 else None
    layer = Qwen3DecoderLayerInteger(0, hq, hk, HID, inter, w, rope_cache_q15(8192).to(dev), pool, comm=comm, exchange=exch)
    batch = AttnBatch(d((lens - 1).astype(np.int32)), d(out_loc), d(table), d(lens.astype(np.int32)), None, 8192,
                      d(np.argsort(-lens, kind="stable").astype(np.int32)))
    g = torch.Generator(device=dev).manual_seed(13)
    x = (torch.randn(B, HID, device=dev, generator=g) * 4096.0).round().to(torch.int32)
    res = (torch.randn(B, HID, device=dev, generator=g) * 4096.0).round().to(torch.int32)
    if world > 1:
        # the form the model step uses between two norms: codes in, codes out, rows finished by their owners
        from mini_sgl_integer_b200.kernel import fixed_point as fp
        codes_in, _, absmax_in, resid, _ = fp.fused_add_rmsnorm_quant(x, res, w["input_norm"])
        absmax_in = absmax_in.reshape(-1)
        run = lambda: layer.forward_codes(codes_in, absmax_in, resid, batch, w["input_norm"])
    else:
        run = lambda: layer.forward_q15(x, res, batch)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
    torch.cuda.current_stream().wait_stream(side)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(5):
        graph.replay()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    n = 30
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    check_device_status()
    ms = torch.tensor([e0.elapsed_time(e1) / n], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    w_bytes = ((HQ + 2 * HK) * 128 * HID + HID * HQ * 128 + 2 * INTER * HID + HID * INTER) / world
    kv_bytes = float(lens.sum()) * hk * 266
    peak, _ = measured_peak()
    ach = (w_bytes + kv_bytes) / (ms * 1e-3) / 1e9
    return {"workload": "one Qwen3-32B-shaped decoder layer, decode batch %d, ctx U[1024,8192], TP=%d, CUDA graph" % (B, world),
            "ms_per_layer": ms, "tok_s": B / (LAYERS * ms * 1e-3), "per_gpu_tok_s": B / (LAYERS * ms * 1e-3) / world,
            "GBs_per_gpu": ach, "frac": ach / peak, "bytes_per_gpu": w_bytes + kv_bytes}


# ----------------------------------------------------------------------------- single-component lines
def component_line(metric, value, unit, ms, args, config, roofline, extra=None):
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
            "data": "synthetic", "config": config, "roofline": roofline}
    line.update(extra or {})
    print(json.dumps(line))


def run_attn(args) -> None:
    import torch
    torch.cuda.set_device(0)
    sampler = ClockSampler(0)
    t0 = time.perf_counter()
    r = attn_micro(torch.device("cuda", 0), max(args.steps, 200), args.pool_pages, args.cluster)
    clocks = sampler.stop(t0, time.perf_counter())
    component_line("int8 paged decode attention throughput (decode tokens/s; HBM GB/s in roofline)", r["tok_s"], "tokens/s",
                   r["kernel_ms"], args, {"workload": "int8 paged decode attention, " + r["workload"], **ATTN_CFG, "sum_ctx": r["sum_ctx"],
                                          "l2": "inputs larger than L2 (about 314 MB of KV touched per launch vs 126 MB)"},
                   {"bound": "hbm", "achieved": r["GBs"], "peak": r["peak"], "unit": "GB/s", "frac": r["frac"], "traffic": r["traffic"],
                    "traffic_source": r["traffic_source"], "peak_source": r["peak_source"], "algorithmic_bytes": r["algorithmic_bytes"],
                    "kernel_ms": r["kernel_ms"], "kernel_ms_median": r["kernel_ms_median"], "frac_of_8TBs": r["frac_of_8TBs"]},
                   {"gpu_launches": r["launches_timed"], "clocks": clocks})


def run_rowops(args) -> None:
    import torch
    from oracle import fixed_point as ofp
    torch.cuda.set_device(0)
    rec, (x, r, w, gu) = rowops_micro(torch.device("cuda", 0), args.rows, args.steps)
    n_cpu = 64
    t0 = time.perf_counter()
    xo, ro, wo, go = (t[:n_cpu].cpu().numpy() if t.ndim == 2 else t.cpu().numpy() for t in (x, r, w, gu))
    eo, _ = ofp.fused_add_rmsnorm_v2(ro, xo, wo); ofp.per_token_quant_from_q15(eo)
    ofp.per_token_quant_from_q15(ofp.blockwise_fwht_q15(ofp.silu_and_mul(go), 128))
    cpu_dt = time.perf_counter() - t0
    ab = rec["A_plus_B"]
    component_line("fused fixed-point row kernels A+B (tokens/s; HBM GB/s in roofline)", args.rows / (ab["ms"] * 1e-3), "tokens/s",
                   ab["ms"], args, {"workload": f"add+RMSNorm+quant on [{args.rows},5120] and SiLU*up+FWHT128+quant on [{args.rows},2*17408]",
                                    "l2": "inputs larger than L2"},
                   {"bound": "hbm", "achieved": ab["GBs"], "peak": rec["peak"], "unit": "GB/s", "frac": ab["frac"], "traffic": None,
                    "peak_source": rec["peak_source"]},
                   {"gpu_launches": 2 * args.steps, "kernels": rec,
                    "cpu_baseline": {"value": n_cpu / cpu_dt, "unit": "tokens/s", "cores": blas_threads(), "kind": "port",
                                     "sample": f"{n_cpu} of the {args.rows} rows through the vectorised numpy oracle ({cpu_dt:.2f} s)"}})


def run_gemm(args) -> None:
    import torch
    torch.cuda.set_device(0)
    r = gemm_micro(torch.device("cuda", 0), args.m, args.steps)
    component_line("W8A8 GEMM with fixed-point epilogue (int8 TOPS)", r["TOPS"], "TOPS", r["ms"], args,
                   {"workload": f"four linears of the 8B-shaped layer at M={args.m}", "M": args.m},
                   {"bound": "tensor", "achieved": r["TOPS"], "peak": 4500.0, "unit": "TOPS", "frac": r["frac_nominal"], "traffic": None,
                    "peak_source": "nominal dense int8 (no measured int8 figure in MEASURED_PEAKS.json)", "frac_of_int_mm": r["frac_of_int_mm"]},
                   {"gpu_launches": 4 * args.steps, "kernels": r["shapes"]})


def run_prefill(args) -> None:
    import torch
    torch.cuda.set_device(0)
    r = prefill_micro(torch.device("cuda", 0), max(args.steps, 5))
    if r is None:
        raise SystemExit("the prefill attention kernel is not in this build")
    component_line("int8 paged prefill attention (prompt tokens/s)", r["tok_s"], "tokens/s", r["ms"], args,
                   {"workload": r["workload"]},
                   {"bound": "tensor", "achieved": r["int8_TOPS_algorithmic"], "peak": 4500.0, "unit": "TOPS",
                    "frac": r["int8_TOPS_algorithmic"] / 4500.0, "traffic": None, "peak_source": "nominal dense int8"},
                   {"gpu_launches": args.steps, "kernels": {"prefill_attn": r}})


def run_offline(args) -> None:
    """Configuration 4 as a run: R requests with prompts U[100, 1024] are prefilled for real (tiled prefill attention over
    their own pages, chunks of at most `--chunk-tokens` prompt tokens per forward), then decoded greedily together for
    `--decode-steps` steps from a CUDA graph.  Reports prefill, decode and overall tokens/s of the 8B-shaped model on one
    GPU and checks batch invariance: the first requests run again on their own must generate the same token ids, bit
    for bit (integer arithmetic with per-token scales has no cross-request term)."""
    import torch
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch
    from mini_sgl_integer_b200.models import (DecodeBatch, Qwen3ForCausalLMInteger, Qwen3IntegerConfig, argmax_int32,
                                              check_device_status, random_weights)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    c = MODEL_CFG
    HID, HQ, HK, INTER, VOCAB, L = c["hidden"], c["q_heads"], c["kv_heads"], c["inter"], c["vocab"], args.model_layers
    R, D = args.batch, args.decode_steps
    rng = np.random.default_rng(33)
    prompt_lens = rng.integers(100, 1025, R)
    ids = rng.integers(0, VOCAB, int(prompt_lens.sum())).astype(np.int32)
    starts = np.concatenate([[0], np.cumsum(prompt_lens)])
    max_len = int(-(-(int(prompt_lens.max()) + D + 1) // 16) * 16)
    table, P = page_tables(rng, prompt_lens + D + 1, max_len // 16)
    cfg = Qwen3IntegerConfig(L, HID, HQ, HK, INTER, VOCAB, max_pos=4096)
    weights = random_weights(cfg, seed=4, device=dev, generate_on_device=True)
    d_table = torch.from_numpy(table).to(dev)

    def run(req, pool):
        """Prefill + D decode steps of the requests `req` (indices); returns generated ids [D + 1, len(req)] and times."""
        lm = Qwen3ForCausalLMInteger(cfg, weights, pool)
        first = torch.empty(len(req), dtype=torch.int32, device=dev)
        chunks, cur, tok = [], [], 0
        for j, r in enumerate(req):                          # whole prompts per chunk, up to chunk_tokens tokens
            if cur and tok + prompt_lens[r] > args.chunk_tokens:
                chunks.append(cur); cur, tok = [], 0
            cur.append(j); tok += int(prompt_lens[r])
        chunks.append(cur)
        batches = []
        for ch in chunks:
            rr = [req[j] for j in ch]
            lens = prompt_lens[rr].astype(np.int32)
            pos = np.concatenate([np.arange(n) for n in lens]).astype(np.int32)
            loc = np.concatenate([table[r][np.arange(n) // 16] * 16 + np.arange(n) % 16 for r, n in zip(rr, lens)]).astype(np.int32)
            tok_ids = np.concatenate([ids[starts[r]:starts[r + 1]] for r in rr])
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
            batches.append((torch.tensor(ch, device=dev), t(tok_ids), AttnBatch(t(pos), t(loc), d_table[rr].contiguous(), t(lens), t(lens), max_len),
                            t((np.cumsum(lens) - 1).astype(np.int32))))
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        for slot, tok_ids, ab, last in batches:
            first[slot] = lm.greedy(tok_ids, ab, last)
        e[1].record()
        state = DecodeBatch(d_table[req].contiguous(), torch.from_numpy(prompt_lens[req].astype(np.int32)).to(dev), max_len)
        out = torch.empty((D + 1, len(req)), dtype=torch.int32, device=dev)
        out[0] = first
        cur_t = first.clone()
        step_no = torch.zeros(1, dtype=torch.int64, device=dev)

        def step():
            cur_t.copy_(lm.greedy(cur_t, state.advance()))
            step_no.add_(1)
            out.index_copy_(0, step_no, cur_t.view(1, -1))
        step()                                               # eager; counts as the first decode step
        ea, eb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ea.record()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):                        # host work only (nothing runs): left out of the decode time
            step()
        eb.record()
        for _ in range(D - 1):
            graph.replay()
        e[2].record()
        torch.cuda.synchronize()
        check_device_status()
        # decode time per step from the D - 1 graph replays (the eager first step is bound by the host's launch rate)
        return out.cpu().numpy(), e[0].elapsed_time(e[1]), eb.elapsed_time(e[2]) * D / max(D - 1, 1)

    pool = Int8PagedKVCache(HK, L, 128, P, dev)
    sub = list(range(min(4, R)))
    ids_sub, _, _ = run(sub, pool)                           # also the warm-up of every kernel shape class
    sampler = ClockSampler(0)
    t0 = time.perf_counter()
    ids_all, pre_ms, dec_ms = run(list(range(R)), pool)
    clocks = sampler.stop(t0, time.perf_counter())
    invariant = bool(np.array_equal(ids_all[:, :len(sub)], ids_sub))
    n_prompt, n_gen = int(prompt_lens.sum()), R * D
    total_ms = pre_ms + dec_ms
    per_layer_w = (HQ + 2 * HK) * 128 * HID + HID * HQ * 128 + 2 * INTER * HID + HID * INTER
    lens_dec = prompt_lens + D / 2.0
    dec_bytes = (L * per_layer_w + VOCAB * HID) + float(lens_dec.sum()) * HK * 266 * L
    peak, how = measured_peak()
    ach = dec_bytes / (dec_ms / D * 1e-3) / 1e9
    gemm_ops = 2.0 * n_prompt * (L * per_layer_w)
    component_line("offline run, prompts U[100,1024] + greedy decode, integer-only W8A8 Qwen3-8B-shaped model (tokens/s, prompt + generated)",
                   (n_prompt + n_gen) / (total_ms * 1e-3), "tokens/s", total_ms, args,
                   {"workload": f"{R} requests, prompts U[100,1024] ({n_prompt} tokens) prefilled in chunks of <= {args.chunk_tokens} tokens, "
                                f"then {D} greedy decode steps of all requests (CUDA graph); Qwen3-8B shape, {L} layers, one GPU",
                    "prefill_tok_s": n_prompt / (pre_ms * 1e-3), "prefill_ms": pre_ms, "prefill_gemm_TOPS": gemm_ops / (pre_ms * 1e-3) / 1e12,
                    "decode_tok_s": n_gen / (dec_ms * 1e-3), "decode_ms_per_step": dec_ms / D,
                    "batch_invariance": "ok" if invariant else "mismatch",
                    "batch_invariance_note": f"requests 0..{len(sub) - 1} run alone generate the ids they generate inside the batch of {R}",
                    "l2": "weights + KV per decode step exceed L2; prefill chunks stream the weights once per chunk"},
                   {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                    "peak_source": how, "note": "decode phase: weights + KV bytes per step over the mean decode step time"},
                   {"clocks": clocks, "gpu_launches": None, "data": "synthetic (seeded prompts and random-init weights)"})
    if not invariant:
        raise SystemExit("offline run: token ids depend on the batch composition")


def run_tp_layer(args) -> None:
    import torch
    import torch.distributed as dist
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    rank, world, local = env_ranks()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rec = tp32b_layer(dev, DistributedCommunicator(), rank, world, args)
    if rank == 0:
        peak, how = measured_peak()
        line = {"metric": "decode tok/s of a 64-layer 32B-shaped integer model, from one tensor-parallel layer step", "value": rec["tok_s"],
                "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": rec["ms_per_layer"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": rec["workload"], "per_gpu_tok_s": rec["per_gpu_tok_s"]},
                "roofline": {"bound": "hbm", "achieved": rec["GBs_per_gpu"], "peak": peak, "unit": "GB/s", "frac": rec["frac"],
                             "traffic": None, "peak_source": how, "bytes_per_rank": rec["bytes_per_gpu"]}}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_tp_linear(args) -> None:
    """One row-split linear of the 8B shape (M = batch, N 4096, K 4096 or 12288 split over the ranks) in its
    pieces, each replayed from a CUDA graph of 20 repetitions: microseconds per call for the exchange-block form, its
    steps alone, the same work on one GPU without any exchange, and the NCCL form (eager)."""
    import torch
    import torch.distributed as dist
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    from mini_sgl_integer_b200.kernel.fixed_point import absmax_to_mul_shift
    from mini_sgl_integer_b200.layers.decoder_layer import _Linear
    from mini_sgl_integer_b200.layers.tp_linear import TpExchange, quant_given_absmax, requant_q15, row_absmax_q15, row_parallel_q15
    from mini_sgl_integer_b200.layers.w8a8_int8 import W8A8Int8LinearMethod, int8_gemm_q15
    rank, world, local = env_ranks()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    comm, method = DistributedCommunicator(), W8A8Int8LinearMethod()
    M, N = args.batch, MODEL_CFG["hidden"]
    res = {}
    for name, K in (("o", MODEL_CFG["hidden"] // world), ("down", MODEL_CFG["inter"] // world)):
        ex = TpExchange(comm, M, N, dev) if world > 1 else TpExchange.emulated(1, M, N, dev)[0]
        g = torch.Generator(device=dev).manual_seed(1)
        x = (torch.randn(M, K, device=dev, generator=g) * 30000).round().to(torch.int32)
        w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
        wm = torch.randint(2**29, 2**30, (N,), dtype=torch.int32, device=dev, generator=g)
        layer = _Linear(w, weight_mul=wm, weight_shift=torch.full((N,), 31, dtype=torch.int32, device=dev))
        c0, a0 = ex.absmax_quant(x)

        def finish():
            if ex.direct:
                return ex.requant_direct(a0, wm, None)
            ex.requant_scatter(a0, wm, None)
            return ex.collect(M, dev)

        def local_linear():
            a = row_absmax_q15(x); c = quant_given_absmax(x, a)
            acc = int8_gemm_q15(c, None, None, w, None, want_q15=False, want_acc=True)
            xm, xs = absmax_to_mul_shift(a)
            return requant_q15(acc, xm, xs, wm, None)
        cases = [("exchange", lambda: ex.row_parallel_q15(method, layer, x), True), ("absmax+quant", lambda: ex.absmax_quant(x), True),
                 ("gemm", lambda: ex.gemm_add(c0, w), True), ("gemm+finish", lambda: (ex.gemm_add(c0, w), finish()), True),
                 ("one_gpu_same_work", local_linear, True)]
        if world > 1:
            cases.append(("nccl_eager", lambda: row_parallel_q15(method, layer, x, comm), False))
        for label, fn, graphable in cases:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            reps = 20
            if graphable:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    fn()
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for _ in range(reps):
                        fn()
                run = graph.replay
            else:
                def run():
                    for _ in range(reps):
                        fn()
            run()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                run()
            e1.record()
            torch.cuda.synchronize()
            res[f"{name}.{label}"] = round(e0.elapsed_time(e1) / (5 * reps) * 1e3, 1)
        if TpExchange.status() != 0:
            raise SystemExit("a cross-rank wait ran out")
    if rank == 0:
        print(json.dumps({"metric": "microseconds per row-split linear (8B shape)", "n_gpus": world, "unit": "us", "M": M, "N": N,
                          "value": res["o.exchange"], "higher_is_better": False, "phases_us": res}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    # NCCL only sets up the process group and runs the barriers / timing reductions around the step (the step itself
    # has no collective call), so it does not need in-switch reduction; the multi-GPU runs were validated with it off
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="model", choices=["model", "attn", "rowops", "gemm", "prefill", "offline", "tp_layer", "tp_linear"],
                    help="model = the decode step of the 8B-shaped model, tensor-parallel over the launched ranks (default); "
                         "the others time one component")
    ap.add_argument("--batch", type=int, default=MODEL_CFG["batch"], help="decode batch of --workload model")
    ap.add_argument("--model-layers", type=int, default=MODEL_CFG["layers"], help="layers of --workload model (fewer: profiler captures)")
    ap.add_argument("--decode-steps", type=int, default=64, help="offline: greedy decode steps after the prefill")
    ap.add_argument("--chunk-tokens", type=int, default=8192, help="offline: most prompt tokens per prefill forward")
    ap.add_argument("--no-kernels", action="store_true", help="model on one GPU: skip the component records")
    ap.add_argument("--no-tp32b", action="store_true", help="model on several GPUs: skip the 32B-shaped layer record")
    ap.add_argument("--cluster", type=int, default=0, help="attn: CTAs per (sequence, KV head); 0 = library default")
    ap.add_argument("--pool-pages", type=int, default=ATTN_CFG["pool_pages"], help="attn: pages in the KV pool")
    ap.add_argument("--rows", type=int, default=16384, help="rows for --workload rowops")
    ap.add_argument("--m", type=int, default=4096, help="M for --workload gemm")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        {"model": run_model, "attn": run_attn, "rowops": run_rowops, "gemm": run_gemm, "prefill": run_prefill, "offline": run_offline,
         "tp_layer": run_tp_layer, "tp_linear": run_tp_linear}[args.workload](args)


if __name__ == "__main__":
    main()
