#!/usr/bin/env python
"""Benchmark of the int8 paged decode attention (the headline workload).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one decode-attention call over a batch of 64 sequences (32 query heads, 8 KV heads,
head_dim 128, 16-token pages, contexts uniform in [512, 4096], page tables drawn from a
200k-page int8 pool with a (multiplier, shift) per token and KV head).  Inputs are synthetic
and seeded.  With N > 1 every rank holds its own pool and batch (independent sequences, no
collective on the data path: weak scaling) and the rate is the sum over ranks.

The script prints ONE JSON line:
  value      tokens/s with everything resident in HBM (CUDA-event time over the K steps, max over ranks)
  e2e        the same rate through the C ABI with the step's inputs (queries, their scales, page table,
             lengths) coming from pinned host memory and the int8 result copied back, every step; the
             KV pool is the cache itself and stays resident
  roofline   algorithmic bytes of one launch / mean kernel time, against the measured HBM copy peak
  cpu_baseline  the CPU oracle (numpy port of the reference arithmetic) timed on this host

``--impl reference`` times only the CPU oracle port on the host cores (the reference's attention is
Python/torch code that cannot travel with this repository; its arithmetic is restated in oracle/).
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

WORKLOAD = dict(batch=64, q_heads=32, kv_heads=8, head_dim=128, page=16, ctx_lo=512, ctx_hi=4096, pool_pages=200_000)
METRIC = "int8 paged decode attention throughput (decode tokens/s; HBM GB/s in roofline)"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised in
# profiles/ (None until a capture exists)
NCU_TRAFFIC_BYTES = 334636800   # dram__bytes_read + dram__bytes_write of one launch (ncu capture of this kernel)


def draw_lens(seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(WORKLOAD["ctx_lo"], WORKLOAD["ctx_hi"] + 1, WORKLOAD["batch"])


def row_order_hint(lens: np.ndarray, scheme: str) -> np.ndarray:
    """The order in which the decode kernel should take the batch rows (a permutation, int32): longest first
    ("lpt", what a scheduler that knows the lengths passes) or as given ("identity")."""
    if scheme == "identity":
        return np.arange(len(lens), dtype=np.int32)
    return np.argsort(-lens, kind="stable").astype(np.int32)


def algorithmic_bytes(lens: np.ndarray) -> int:
    """Minimum HBM traffic of one launch: K and V codes, their scales, page ids, q in, int8 out."""
    w = WORKLOAD
    per_seq = lens.astype(np.int64) * w["kv_heads"] * w["head_dim"] * 2 + lens.astype(np.int64) * w["kv_heads"] * 2 * 5 \
        + ((lens + 15) // 16).astype(np.int64) * 4
    return int(per_seq.sum() + w["batch"] * w["q_heads"] * w["head_dim"] * 2)


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ----------------------------------------------------------------------------- CPU oracle leg
def cpu_oracle_rate(seed: int, n_seq: int, repeats: int = 1):
    """Tokens/s of the numpy oracle on the first ``n_seq`` sequences of the seeded batch."""
    from oracle import attention as oattn
    w = WORKLOAD
    lens = draw_lens(seed)[:n_seq]
    rng = np.random.default_rng(seed + 1)
    n_pg = (lens + 15) // 16
    pool = oattn.PagedKV(int(n_pg.sum()), w["kv_heads"], w["head_dim"])
    pool.k_codes[:] = rng.integers(-127, 128, pool.k_codes.shape, dtype=np.int8)
    pool.v_codes[:] = rng.integers(-127, 128, pool.v_codes.shape, dtype=np.int8)
    pool.meta[:, :, 0:32] = rng.integers(2**30, 2**31, pool.meta[:, :, 0:32].shape)
    pool.meta[:, :, 32:36].view(np.int8)[:] = rng.integers(35, 39, (pool.P, pool.H, 16))
    pool.meta[:, :, 36:40].view(np.int8)[:] = rng.integers(33, 38, (pool.P, pool.H, 16))
    perm = rng.permutation(pool.P)
    tables, off = [], 0
    for n in n_pg:
        tables.append(perm[off:off + n]); off += n
    q = rng.integers(-127, 128, (n_seq, w["q_heads"], w["head_dim"]), dtype=np.int8)
    qm = rng.integers(2**30, 2**31, (n_seq, w["q_heads"])); qs = rng.integers(43, 46, (n_seq, w["q_heads"]))
    t0 = time.perf_counter()
    for _ in range(repeats):
        out = oattn.paged_attention(q, qm, qs, pool, tables, lens, [1] * n_seq)
        oattn.quant_heads_int8(out)
    dt = (time.perf_counter() - t0) / repeats
    return n_seq / dt, dt


def host_threads() -> int:
    try:
        import torch
        return int(torch.get_num_threads())
    except Exception:
        return os.cpu_count() or 1


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_seq = 16
    for _ in range(args.warmup):
        cpu_oracle_rate(0, 4)
    t0 = time.perf_counter()
    total = 0.0
    for _ in range(args.steps):
        _, dt = cpu_oracle_rate(0, n_seq)
        total += dt
    rate = n_seq * args.steps / total
    sample = f"{n_seq} of the 64 sequences per step (all 32 heads), numpy oracle port, BLAS threads for the dot products"
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "int8 paged decode attention, batch 64, 32q/8kv heads, head_dim 128, page 16, "
                               "ctx U[512,4096] (CPU sample)", **WORKLOAD},
        "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": host_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line))


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


# ----------------------------------------------------------------------------- GPU leg
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    from mini_sgl_integer_b200 import _lib
    from mini_sgl_integer_b200.attention import Int8PagedKVCache

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = WORKLOAD
    B, Hq, Hkv, D, P = w["batch"], w["q_heads"], w["kv_heads"], w["head_dim"], args.pool_pages

    # ---- seeded synthetic state and inputs (each rank its own draw)
    lens_np = draw_lens(rank)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    pool = Int8PagedKVCache(Hkv, 1, D, P, dev)
    pool.k_cache(0).copy_(torch.randint(-127, 128, pool.k_cache(0).shape, dtype=torch.int8, device=dev, generator=g))
    pool.v_cache(0).copy_(torch.randint(-127, 128, pool.v_cache(0).shape, dtype=torch.int8, device=dev, generator=g))
    meta = pool.meta(0)
    meta[:, :, 0:32] = torch.randint(2**30, 2**31, (P, Hkv, 32), dtype=torch.int64, device=dev, generator=g).to(torch.int32)
    meta[:, :, 32:36] = torch.randint(35, 39, (P, Hkv, 16), dtype=torch.int8, device=dev, generator=g).view(torch.int32)
    meta[:, :, 36:40] = torch.randint(33, 38, (P, Hkv, 16), dtype=torch.int8, device=dev, generator=g).view(torch.int32)
    rng = np.random.default_rng(2000 + rank)
    perm = rng.permutation(P)
    n_pg = (lens_np + 15) // 16
    pitch = int(((w["ctx_hi"] + 15) // 16))
    table_np = np.zeros((B, pitch), dtype=np.int32)
    off = 0
    for b in range(B):
        table_np[b, : n_pg[b]] = perm[off:off + n_pg[b]]; off += n_pg[b]
    # The inputs of a step live in ONE pinned host buffer and one device buffer (256-byte aligned fields), the results
    # likewise, so the end-to-end step is one host-to-device copy, one launch and one device-to-host copy.
    fields = [("q", rng.integers(-127, 128, (B, Hq, D), dtype=np.int8)),
              ("qm", rng.integers(2**30, 2**31, (B, Hq)).astype(np.int32)),
              ("qs", rng.integers(43, 46, (B, Hq)).astype(np.int32)),
              ("table", table_np), ("lens", lens_np.astype(np.int32)),
              # the batch rows by descending length: a scheduling hint that whoever builds the batch can give
              ("order", row_order_hint(lens_np, args.row_order))]

    def layout(items):
        offs, off = {}, 0
        for name, nbytes in items:
            offs[name] = off
            off += (nbytes + 255) // 256 * 256
        return offs, off

    in_off, in_bytes = layout([(n, a.nbytes) for n, a in fields])
    h_in = torch.empty(in_bytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(in_bytes, dtype=torch.uint8, device=dev)
    for name, a in fields:
        h_in[in_off[name]: in_off[name] + a.nbytes] = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).reshape(-1))
    d_in.copy_(h_in)

    def dview(buf, off, shape, dtype):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return buf[off: off + n].view(dtype).view(shape)

    d_q = dview(d_in, in_off["q"], (B, Hq, D), torch.int8)
    d_qm, d_qs = dview(d_in, in_off["qm"], (B, Hq), torch.int32), dview(d_in, in_off["qs"], (B, Hq), torch.int32)
    d_table = dview(d_in, in_off["table"], (B, pitch), torch.int32)
    d_lens, d_order = dview(d_in, in_off["lens"], (B,), torch.int32), dview(d_in, in_off["order"], (B,), torch.int32)
    out_off, out_bytes = layout([("codes", B * Hq * D), ("absmax", B * Hq * 4)])
    h_res = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
    d_res = torch.empty(out_bytes, dtype=torch.uint8, device=dev)
    d_out = dview(d_res, out_off["codes"], (B, Hq, D), torch.int8)
    d_absmax = dview(d_res, out_off["absmax"], (B, Hq), torch.int32)
    stream = torch.cuda.current_stream()
    sp = _lib.c_void_p(stream.cuda_stream)
    p = _lib.ptr

    ws_bytes = int(_lib.load().b200_attn_workspace_bytes(B, Hq, Hkv, w["ctx_hi"]))
    d_ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)      # caller-owned scratch of the workspace variant

    def launch():
        if args.attn_impl == "split":
            _lib.call("b200_attn_paged_ws", p(d_q), p(d_qm), p(d_qs), p(pool.k_cache(0)), p(pool.v_cache(0)), p(pool.meta(0)),
                      p(d_table), pitch, p(d_lens), None, None, None, p(d_out), p(d_absmax), B, Hq, Hkv, P, w["ctx_hi"],
                      p(d_ws), ws_bytes, sp)
        else:
            _lib.call("b200_attn_decode", p(d_q), p(d_qm), p(d_qs), p(pool.k_cache(0)), p(pool.v_cache(0)), p(pool.meta(0)),
                      p(d_table), pitch, p(d_lens), p(d_order), None, p(d_out), p(d_absmax), B, Hq, Hkv, P, w["ctx_hi"], args.cluster, sp)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    for _ in range(args.warmup):
        launch()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    t_sus = time.perf_counter()       # untimed load of the same kernel so that nvidia-smi can sample clocks
    while time.perf_counter() - t_sus < args.sustain_s:
        for _ in range(50):
            launch()
        torch.cuda.synchronize()
    barrier()
    t_wall0 = time.perf_counter()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for a, b in evs:
        a.record(stream); launch(); b.record(stream)
    e1.record(stream)
    barrier()
    t_wall1 = time.perf_counter()
    total_ms = e0.elapsed_time(e1)
    kern_ms = float(np.mean([a.elapsed_time(b) for a, b in evs]))

    # ---- end to end: host inputs -> device, launch, result -> host, every step
    def e2e_step():
        d_in.copy_(h_in, non_blocking=True)
        launch()
        h_res.copy_(d_res, non_blocking=True)
        stream.synchronize()

    for _ in range(args.warmup):
        e2e_step()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for _ in range(args.steps):
        e2e_step()
    f1.record(stream)
    barrier()
    e2e_ms = f0.elapsed_time(f1)
    clocks = sampler.stop(t_sus, time.perf_counter()) if sampler else None

    t = torch.tensor([total_ms, e2e_ms, kern_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, kern_ms = (float(x) for x in t.tolist())
    if rank == 0:
        alg = algorithmic_bytes(lens_np)
        peak, how = measured_peak()
        achieved = alg / (kern_ms * 1e-3) / 1e9
        h2d = int(in_bytes)
        d2h = int(out_bytes)
        n_cpu = 8
        cpu_rate, cpu_dt = cpu_oracle_rate(0, n_cpu)
        line = {
            "metric": METRIC, "value": world * B * args.steps / (total_ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "int8 paged decode attention, batch 64 per GPU, 32q/8kv heads, head_dim 128, page 16, "
                                   "ctx U[512,4096], 200k-page pool", **w, "sum_ctx": int(lens_np.sum()),
                       "l2": "inputs larger than L2 (about 314 MB of KV touched per launch vs 126 MB)",
                       "cluster": args.cluster, "attn_impl": args.attn_impl},
            "e2e": {"value": world * B * args.steps / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": args.steps * (5 if args.attn_impl == "split" else 1),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES, "peak_source": how, "algorithmic_bytes": alg,
                         "kernel_ms": kern_ms, "kernel": "split_scores + split_expsum + split_pv (+ init, final)" if args.attn_impl == "split" else "attn_decode_kernel<4>",
                         "workspace_bytes": ws_bytes if args.attn_impl == "split" else 0, "frac_of_8TBs": achieved / 8000.0},
            "cpu_baseline": {"value": cpu_rate, "unit": "tokens/s", "cores": host_threads(), "kind": "port",
                             "sample": f"{n_cpu} of the 64 sequences, one pass ({cpu_dt:.2f} s), numpy oracle port"},
            "clocks": clocks, "wall_s": t_wall1 - t_wall0,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()



# ----------------------------------------------------------------------------- secondary workloads
def _time_cuda(fn, steps, warmup):
    import torch
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_rowops(args) -> None:
    """Configuration 3: add+RMSNorm+quant (A) on [rows, 5120] and SiLU*up+FWHT128+quant (B) on [rows, 2*17408]."""
    import torch
    from mini_sgl_integer_b200.kernel import fixed_point as fp
    from oracle import fixed_point as ofp
    torch.cuda.set_device(0)
    T, H, I = args.rows, 5120, 17408
    g = torch.Generator(device="cuda").manual_seed(0)
    clip = lambda t: t.round().clamp(-(2**23), 2**23).to(torch.int32)
    x = clip(torch.randn(T, H, device="cuda", generator=g) * 4096.0)
    r = clip(torch.randn(T, H, device="cuda", generator=g) * 4096.0)
    w = torch.randint(2**13, 2**15 + 1, (H,), device="cuda", dtype=torch.int32, generator=g)
    gu = (torch.randn(T, 2 * I, device="cuda", generator=g) * 2.0**17).round().to(torch.int32)
    ms_a = _time_cuda(lambda: fp.fused_add_rmsnorm_quant(x, r, w), args.steps, args.warmup)
    ms_b = _time_cuda(lambda: fp.silu_mul_fwht_quant(gu, 128), args.steps, args.warmup)
    bytes_a, bytes_b = T * (13 * H + 8), T * (9 * I + 8)
    peak, how = measured_peak()
    n_cpu = 64
    t0 = time.perf_counter()
    xo, ro, wo, go = (t[:n_cpu].cpu().numpy() if t.ndim == 2 else t.cpu().numpy() for t in (x, r, w, gu))
    eo, _ = ofp.fused_add_rmsnorm_v2(ro, xo, wo); ofp.per_token_quant_from_q15(eo)
    ofp.per_token_quant_from_q15(ofp.blockwise_fwht_q15(ofp.silu_and_mul(go), 128))
    cpu_dt = time.perf_counter() - t0
    kern = {"A_add_rmsnorm_quant": {"ms": ms_a, "GBs": bytes_a / ms_a / 1e6, "frac": bytes_a / ms_a / 1e6 / peak, "bytes": bytes_a},
            "B_silu_fwht_quant": {"ms": ms_b, "GBs": bytes_b / ms_b / 1e6, "frac": bytes_b / ms_b / 1e6 / peak, "bytes": bytes_b}}
    tot = ms_a + ms_b
    print(json.dumps({
        "metric": "fused fixed-point row kernels A+B (tokens/s; HBM GB/s in roofline)", "value": T / (tot * 1e-3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": f"add+RMSNorm+quant on [{T},5120] and SiLU*up+FWHT128+quant on [{T},2*17408]",
                   "rows": T, "hidden": H, "inter": I, "l2": "inputs larger than L2"},
        "gpu_launches": 2 * args.steps, "kernels": kern,
        "roofline": {"bound": "hbm", "achieved": (bytes_a + bytes_b) / tot / 1e6, "peak": peak, "unit": "GB/s",
                     "frac": (bytes_a + bytes_b) / tot / 1e6 / peak, "traffic": None, "peak_source": how},
        "cpu_baseline": {"value": n_cpu / cpu_dt, "unit": "tokens/s", "cores": host_threads(), "kind": "port",
                         "sample": f"{n_cpu} of the {T} rows through the vectorised numpy oracle ({cpu_dt:.2f} s)"},
    }))


def run_gemm(args) -> None:
    """W8A8 GEMM micro-benchmark: the (N, K) pairs of the 8B-shaped model at the given M."""
    import torch
    from mini_sgl_integer_b200.layers import int8_gemm_q15
    torch.cuda.set_device(0)
    M = args.m
    out = {}
    for name, (N, K) in {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288)}.items():
        x8 = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
        w8 = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda")
        xm = torch.randint(2**30, 2**31 - 1, (M,), dtype=torch.int64, device="cuda").to(torch.int32)
        xs = torch.full((M,), 40, dtype=torch.int32, device="cuda")
        wm = torch.randint(2**29, 2**30, (N,), dtype=torch.int32, device="cuda")
        ms = _time_cuda(lambda: int8_gemm_q15(x8, xm, xs, w8, wm), args.steps, args.warmup)
        lib = _time_cuda(lambda: torch._int_mm(x8, w8.t()), args.steps, args.warmup) if M > 16 else float("nan")
        out[name] = {"N": N, "K": K, "ms": ms, "TOPS": 2 * M * N * K / ms / 1e9,
                     "GBs": (M * K + N * K + 4 * M * N) / ms / 1e6, "library_int_mm_TOPS": 2 * M * N * K / lib / 1e9}
    tot_ops = sum(2 * M * v["N"] * v["K"] for v in out.values())
    tot_ms = sum(v["ms"] for v in out.values())
    print(json.dumps({
        "metric": "W8A8 GEMM with fixed-point epilogue (int8 TOPS)", "value": tot_ops / tot_ms / 1e9, "unit": "TOPS",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": f"four linears of the 8B-shaped layer at M={M}", "M": M}, "gpu_launches": 4 * args.steps,
        "kernels": out,
        "roofline": {"bound": "tensor", "achieved": tot_ops / tot_ms / 1e9, "peak": 4500.0, "unit": "TOPS",
                     "frac": tot_ops / tot_ms / 1e9 / 4500.0, "traffic": None,
                     "peak_source": "nominal dense int8 (no measured int8 figure in MEASURED_PEAKS.json)"},
    }))


def run_tp_layer(args) -> None:
    """Configuration 5 proxy: ONE Qwen3-32B-shaped integer decoder layer, decode step of batch 256 with contexts
    U[1024, 8192], tensor-parallel over the launched ranks (attention by KV head, column/row-split GEMMs, two
    int32 all-reduces per layer over NCCL).  tokens/s are quoted for the 64-layer model (64 x this layer)."""
    import torch
    import torch.distributed as dist
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.distributed import DistributedCommunicator
    from mini_sgl_integer_b200.layers.decoder_layer import AttnBatch, Qwen3DecoderLayerInteger, _Linear

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    HID, HQ, HK, INTER, LAYERS, B = 5120, 64, 8, 25600, 64, args.tp_batch
    hq, hk, inter = HQ // world, HK // world, INTER // world
    g = torch.Generator(device=dev).manual_seed(7)            # same seed on every rank: replicated tensors agree
    ri8 = lambda *shape: torch.randint(-127, 128, shape, dtype=torch.int8, device=dev, generator=g)
    def lin(n, k):
        l = _Linear(ri8(n, k), weight_mul=torch.randint(2**29, 2**30, (n,), dtype=torch.int32, device=dev, generator=g),
                    weight_shift=torch.full((n,), 38, dtype=torch.int32, device=dev))
        return l
    weights = {"qkv": lin((hq + 2 * hk) * 128, HID), "o": lin(HID, hq * 128), "gate_up": lin(2 * inter, HID), "down": lin(HID, inter),
               "input_norm": torch.randint(2**13, 2**15, (HID,), dtype=torch.int32, device=dev, generator=g),
               "post_norm": torch.randint(2**13, 2**15, (HID,), dtype=torch.int32, device=dev, generator=g),
               "q_norm": torch.randint(2**11, 2**13, (128,), dtype=torch.int32, device=dev, generator=g),
               "k_norm": torch.randint(2**12, 2**14, (128,), dtype=torch.int32, device=dev, generator=g)}
    rng = np.random.default_rng(11)
    lens = rng.integers(1024, 8193, B)
    n_pg = (lens + 15) // 16
    P = int(n_pg.sum()) + 8
    pool = Int8PagedKVCache(hk, 1, 128, P, dev)
    pool.k_cache(0).copy_(ri8(*pool.k_cache(0).shape)); pool.v_cache(0).copy_(ri8(*pool.v_cache(0).shape))
    meta = pool.meta(0)
    meta[:, :, 0:32] = torch.randint(2**30, 2**31, (P, hk, 32), dtype=torch.int64, device=dev, generator=g).to(torch.int32)
    meta[:, :, 32:36] = torch.randint(35, 39, (P, hk, 16), dtype=torch.int8, device=dev, generator=g).view(torch.int32)
    meta[:, :, 36:40] = torch.randint(36, 40, (P, hk, 16), dtype=torch.int8, device=dev, generator=g).view(torch.int32)
    perm = rng.permutation(P)
    pitch = 512
    table = np.zeros((B, pitch), dtype=np.int32)
    off = 0
    for b in range(B):
        table[b, : n_pg[b]] = perm[off:off + n_pg[b]]; off += n_pg[b]
    out_loc = np.array([table[b, (lens[b] - 1) // 16] * 16 + (lens[b] - 1) % 16 for b in range(B)], dtype=np.int32)
    inv = 1.0 / (1000000.0 ** (torch.arange(0, 128, 2, dtype=torch.float) / 128))
    fr = torch.einsum("i,j -> ij", torch.arange(8192, dtype=torch.float), inv)
    cache = torch.clamp(torch.round(torch.cat((fr.cos(), fr.sin()), -1) * 32768), -32768, 32767).to(torch.int32).to(dev)
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    comm = DistributedCommunicator()
    bufs = None
    if world > 1 and args.fused_reduce:
        from mini_sgl_integer_b200.layers.tp_linear import PeerReduceBuffers
        bufs = PeerReduceBuffers(comm, B, HID, dev)
    layer = Qwen3DecoderLayerInteger(0, hq, hk, HID, inter, weights, cache, pool, comm=comm, peer_buffers=bufs)
    batch = AttnBatch(d((lens - 1).astype(np.int32)), d(out_loc), d(table), d(lens.astype(np.int32)), None, 8192,
                      d(np.argsort(-lens, kind="stable").astype(np.int32)))
    x = (torch.randn(B, HID, device=dev, generator=g) * 4096.0).round().to(torch.int32)
    res = (torch.randn(B, HID, device=dev, generator=g) * 4096.0).round().to(torch.int32)
    eager = lambda: layer.forward_q15(x, res, batch)
    for _ in range(max(args.warmup, 3)):
        eager()
    torch.cuda.synchronize()
    step = eager
    if args.graph and world == 1:
        # the layer step replayed from one CUDA graph, as the engine's decode does (single rank only: capturing
        # the NCCL collectives of a multi-rank step did not complete on this pool and stays off)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            eager()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            eager()
        step = graph.replay
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms)
    if rank == 0:
        w_bytes = ((HQ + 2 * HK) * 128 * HID + HID * HQ * 128 + 2 * INTER * HID + HID * INTER) / world
        kv_bytes = float(lens.sum()) * hk * 266
        peak, how = measured_peak()
        ach = (w_bytes + kv_bytes) / (ms * 1e-3) / 1e9
        print(json.dumps({
            "metric": "decode tok/s of a 64-layer 32B-shaped integer model, from one tensor-parallel layer step", "value": B / (LAYERS * ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "one Qwen3-32B-shaped decoder layer, decode batch %d, ctx U[1024,8192], TP=%d" % (B, world),
                       "per_gpu_tok_s": B / (LAYERS * ms * 1e-3) / world, "cuda_graph": bool(args.graph and world == 1),
                       "row_parallel_sum": "in the GEMM kernel over peer memory" if bufs is not None else "NCCL all-reduce"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                         "peak_source": how, "bytes_per_rank": w_bytes + kv_bytes},
        }))
    if world > 1:
        dist.destroy_process_group()


def run_model(args) -> None:
    """Configuration 4's model on one GPU: a full Qwen3-8B-shaped integer model (36 layers, hidden 4096, 32/8 heads,
    intermediate 12288, vocab 151936; random-init int8 weights), greedy decode of a batch of 256 sequences whose
    contexts are drawn from U[100, 2048] (the spread of prompt + generated lengths of the offline run).  One step =
    bookkeeping on the device, embedding, 36 layers, final norm, integer lm_head, arg-max, token fed back; the step
    is captured once in a CUDA graph and replayed.  KV pages hold seeded random codes instead of a real prefill."""
    import torch
    from mini_sgl_integer_b200.attention import Int8PagedKVCache
    from mini_sgl_integer_b200.models import DecodeBatch, Qwen3ForCausalLMInteger, Qwen3IntegerConfig, random_weights

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cfg = Qwen3IntegerConfig(args.model_layers, 4096, 32, 8, 12288, 151936, max_pos=4096)
    B = args.tp_batch
    rng = np.random.default_rng(21)
    lens = rng.integers(100, 2049, B)
    total_steps = args.warmup + args.steps + 4
    max_len = int(-(-(int(lens.max()) + total_steps + 1) // 16) * 16)
    n_pg = (lens + total_steps + 16) // 16
    P = int(n_pg.sum()) + 8
    w = random_weights(cfg, seed=4, device=dev, generate_on_device=True)
    pool = Int8PagedKVCache(cfg.num_kv_heads, cfg.num_layers, 128, P, dev)
    g = torch.Generator(device=dev).manual_seed(5)
    for i in range(cfg.num_layers):
        pool.k_cache(i).copy_(torch.randint(-127, 128, pool.k_cache(i).shape, dtype=torch.int8, device=dev, generator=g))
        pool.v_cache(i).copy_(torch.randint(-127, 128, pool.v_cache(i).shape, dtype=torch.int8, device=dev, generator=g))
        meta = pool.meta(i)
        meta[:, :, 0:32] = torch.randint(2**30, 2**31, (P, 8, 32), dtype=torch.int64, device=dev, generator=g).to(torch.int32)
        meta[:, :, 32:36] = torch.randint(35, 39, (P, 8, 16), dtype=torch.int8, device=dev, generator=g).view(torch.int32)
        meta[:, :, 36:40] = torch.randint(36, 40, (P, 8, 16), dtype=torch.int8, device=dev, generator=g).view(torch.int32)
    perm = rng.permutation(P)
    pitch = max_len // 16
    table = np.zeros((B, pitch), dtype=np.int32)
    off = 0
    for b in range(B):
        table[b, : n_pg[b]] = perm[off:off + n_pg[b]]; off += n_pg[b]
    state = DecodeBatch(torch.from_numpy(table).to(dev), torch.from_numpy(lens.astype(np.int32)).to(dev), max_len)
    lm = Qwen3ForCausalLMInteger(cfg, w, pool)
    h_in = torch.from_numpy(rng.integers(0, cfg.vocab, B).astype(np.int32)).pin_memory()
    h_out = torch.empty(B, dtype=torch.int32).pin_memory()
    cur = h_in.to(dev)

    def step():
        cur.copy_(lm.greedy(cur, state.advance()))

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                              # loads modules, sizes attributes (outside the capture)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(args.warmup):
        graph.replay()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    t_wall0 = time.perf_counter()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t_wall1 = time.perf_counter()
    ms = e0.elapsed_time(e1) / args.steps
    # end to end: the scheduler's view of a step - tokens in from pinned host memory, tokens out to it
    lens_after = state.seq_lens.cpu().numpy()
    t0 = time.perf_counter()
    e2e_steps = min(args.steps, 4)
    for _ in range(e2e_steps):
        cur.copy_(h_in, non_blocking=True)
        graph.replay()
        h_out.copy_(cur, non_blocking=True)
        torch.cuda.synchronize()
        h_in.copy_(h_out)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    clocks = sampler.stop(t_wall0, t_wall1)
    per_layer_w = (32 + 16) * 128 * 4096 + 4096 * 32 * 128 + 2 * 12288 * 4096 + 4096 * 12288
    w_bytes = cfg.num_layers * per_layer_w + cfg.vocab * cfg.hidden
    kv_bytes = float(lens_after.mean()) * B * 8 * 266 * cfg.num_layers
    peak, how = measured_peak()
    ach = (w_bytes + kv_bytes) / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "decode tokens/s per GPU, full integer model", "value": B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "Qwen3-8B-shaped integer model (%d layers), greedy decode, batch %d, ctx U[100,2048] (mean %.0f), page 16, CUDA graph"
                               % (cfg.num_layers, B, float(lens_after.mean())), "l2": "weights + KV per step (%.1f GB) exceed L2" % ((w_bytes + kv_bytes) / 1e9)},
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "traffic": None,
                     "peak_source": how, "weight_bytes": w_bytes, "kv_bytes": kv_bytes},
        "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
        "clocks": clocks,
    }))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cluster", type=int, default=0, help="CTAs per (sequence, KV head); 0 = library default")
    ap.add_argument("--attn-impl", default="cluster", choices=["split", "cluster"],
                    help="split = grid-wide passes over a workspace (5 launches per step); cluster = one kernel per step")
    ap.add_argument("--row-order", default="lpt", choices=["lpt", "identity"],
                    help="scheduling hint passed to the decode kernel (see row_order_hint)")
    ap.add_argument("--pool-pages", type=int, default=WORKLOAD["pool_pages"],
                    help="pages in the KV pool (smaller pools are for profiler captures only)")
    ap.add_argument("--sustain-s", type=float, default=1.0,
                    help="seconds of untimed back-to-back launches before the timed region (clock sampling)")
    ap.add_argument("--workload", default="attn", choices=["attn", "rowops", "gemm", "tp_layer", "model"],
                    help="attn = the headline decode attention (default); rowops / gemm = the other kernels of the path")
    ap.add_argument("--rows", type=int, default=16384, help="rows for --workload rowops")
    ap.add_argument("--m", type=int, default=4096, help="M for --workload gemm")
    ap.add_argument("--tp-batch", type=int, default=256, help="decode batch for --workload tp_layer / model")
    ap.add_argument("--model-layers", type=int, default=36, help="layers for --workload model")
    ap.add_argument("--fused-reduce", action="store_true",
                    help="tp_layer on several GPUs: the row-parallel GEMMs add their partial sums over NVLink peer memory themselves")
    ap.add_argument("--graph", action="store_true", help="tp_layer on one GPU: replay the layer step from a CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "rowops":
        run_rowops(args)
    elif args.workload == "gemm":
        run_gemm(args)
    elif args.workload == "tp_layer":
        run_tp_layer(args)
    elif args.workload == "model":
        run_model(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
