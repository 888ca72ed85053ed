"""Driver for tests/test_gpu_engine_reference.py, run in a fresh process: builds the UNMODIFIED reference's
``minisgl.engine.Engine`` (installed under baseline/_ref) with this package's integer model, int8 paged pool and
attention backend plugged in at three places (backend registry, model factory, pool factory), runs one prefill and a few greedy
decode steps through ``Engine.forward_batch`` and writes the token ids (and the rotary table the model built) to a file.

    python tests/engine_under_reference.py <reference site dir> <model dir> <steps> <out.npz>
"""
from __future__ import annotations

import json
import os
import sys


def main(ref_dir: str, model_dir: str, steps: int, out_path: str) -> None:
    sys.path.insert(0, ref_dir)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import numpy as np
    import torch

    import minisgl.attention as ref_attention
    import minisgl.engine.engine as ref_engine
    from minisgl.core import Batch, Req, SamplingParams
    from minisgl.distributed import DistributedInfo
    from minisgl.engine.config import EngineConfig
    from minisgl.engine.sample import BatchSamplingArgs

    import mini_sgl_integer_b200.core as b_core
    import mini_sgl_integer_b200.distributed as b_dist
    from mini_sgl_integer_b200.attention import B200Int8Backend
    from mini_sgl_integer_b200.attention.backend import token_locations
    from mini_sgl_integer_b200.kvcache import Int8PagedKVCache
    from mini_sgl_integer_b200.models.integer import Qwen3ForCausalLMInteger

    # ---- the patch: backend registration, model class, pool; and this package's copies of the two process globals
    ref_attention.SUPPORTED_ATTENTION_BACKENDS.register("b200_int8")(lambda config, kvcache: B200Int8Backend(config, kvcache))
    ref_engine.create_model = lambda model_config: Qwen3ForCausalLMInteger(model_config)
    ref_engine.create_kvcache = lambda model_config, num_pages, device, dtype: Int8PagedKVCache(
        model_config.num_kv_heads, model_config.num_layers, model_config.head_dim, num_pages, torch.int8, device)
    ref_set_ctx, ref_set_tp = ref_engine.set_global_ctx, ref_engine.set_tp_info

    def set_ctx(ctx):
        ref_set_ctx(ctx)
        b_core.set_global_ctx(ctx, replace=True)

    def set_tp(rank, size):
        ref_set_tp(rank=rank, size=size)
        b_dist.set_tp_info(rank, size)
    ref_engine.set_global_ctx, ref_engine.set_tp_info = set_ctx, set_tp

    case = json.load(open(os.path.join(model_dir, "case.json")))
    prompts, pages = case["prompts"], case["pages"]
    config = EngineConfig(model_path=model_dir, tp_info=DistributedInfo(0, 1), dtype=torch.bfloat16, max_running_req=len(prompts),
                          attention_backend="b200_int8", cuda_graph_bs=[], page_size=16, max_seq_len_override=case["max_len"],
                          num_page_override=case["num_pages"])
    # Environment shim, not part of the patch: the image's transformers (5.x) keeps the rotary base under
    # `rope_parameters`, while the reference's ModelConfig.from_hf reads `config.rope_theta` (models/config.py:144).
    # (and reports plain rotary embeddings as rope_scaling {"rope_type": "default"}, which layers/rotary.py:102-128 rejects).
    from types import SimpleNamespace
    from minisgl.utils import cached_load_hf_config
    fields = cached_load_hf_config(model_dir).to_dict()
    rope = fields.get("rope_parameters") or {}
    fields.setdefault("rope_theta", rope.get("rope_theta"))
    if (fields.get("rope_scaling") or rope).get("rope_type", "default") == "default":
        fields["rope_scaling"] = None
    config.__dict__["hf_config"] = SimpleNamespace(**fields)      # EngineConfig.hf_config is a cached property
    engine = ref_engine.Engine(config)
    assert isinstance(engine.model, Qwen3ForCausalLMInteger) and isinstance(engine.kv_cache, Int8PagedKVCache)
    assert isinstance(engine.attn_backend, B200Int8Backend)
    dev = engine.device
    # the page table holds page ids (16-token pages), one row per request
    for b, row in enumerate(pages):
        engine.page_table[b, :len(row)] = torch.tensor(row, dtype=torch.int32, device=dev)

    def run(phase, reqs, input_ids):
        batch = Batch(reqs=reqs, phase=phase)
        batch.padded_reqs = reqs
        batch.input_ids = torch.tensor(input_ids, dtype=torch.int32, device=dev)
        pos = np.concatenate([np.arange(r.cached_len, r.device_len) for r in reqs]).astype(np.int32)
        rows = np.concatenate([np.full(r.extend_len, i) for i, r in enumerate(reqs)])
        batch.positions = torch.from_numpy(pos).to(dev)
        batch.out_loc = token_locations(engine.page_table[[r.table_idx for r in reqs]], batch.positions, torch.from_numpy(rows).to(dev))
        engine.attn_backend.prepare_metadata(batch)
        out = engine.forward_batch(batch, BatchSamplingArgs(temperatures=None))
        out.copy_done_event.synchronize()
        return out.next_tokens_cpu.numpy().astype(np.int32)

    reqs = [Req(input_ids=torch.tensor(p, dtype=torch.int32), table_idx=b, cached_len=0, output_len=steps + 1, uid=b,
                sampling_params=SamplingParams(), cache_handle=None) for b, p in enumerate(prompts)]
    tokens = [run("prefill", reqs, [t for p in prompts for t in p])]
    for _ in range(steps):
        for r, t in zip(reqs, tokens[-1]):
            r.append_host(torch.tensor([int(t)], dtype=torch.int32))
        tokens.append(run("decode", reqs, tokens[-1].tolist()))
    rotary = engine.model.model.layers.op_list[0].self_attn.attn.rotary._cos_sin_cache_q15.cpu().numpy()
    from mini_sgl_integer_b200 import _lib
    np.savez(out_path, tokens=np.stack(tokens), rotary=rotary, calls=np.int64(_lib.CALLS))
    engine.shutdown()


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2], int(sys.argv[3]), sys.argv[4])
