"""The class-level boundary on CPU: state-dict loading as the reference's BaseOP does it, the layer constructors and
their shard sizes, the rotary tables (incl. the llama3 frequency re-scaling, against reference-generated rows), the
backend registry and the reference-form constructors of the backend and the KV pool."""
from __future__ import annotations

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from mini_sgl_integer_b200 import distributed as tpd


@pytest.fixture()
def tp1():
    tpd._reset_tp_info_for_tests()
    tpd.set_tp_info(0, 1)
    yield
    tpd._reset_tp_info_for_tests()


@pytest.fixture()
def tp2_rank1():
    tpd._reset_tp_info_for_tests()
    tpd.set_tp_info(1, 2)
    yield
    tpd._reset_tp_info_for_tests()


def _config(layers=1):
    from mini_sgl_integer_b200.models.config import HadamardTransformConfig, ModelConfig, RotaryConfig
    return ModelConfig(layers, 4, 2, 128, 256, 1000, 512, 1e-6, RotaryConfig(128, 128, 64, 1e6),
                       hadamard_transform=HadamardTransformConfig(True, 128, ("down_proj",)))


def test_state_dict_keys_follow_the_reference_names(tp1):
    from mini_sgl_integer_b200.models.integer import Qwen3ForCausalLMInteger
    keys = set(Qwen3ForCausalLMInteger(_config()).state_dict())
    assert keys == {
        "lm_head.weight", "model.embed_tokens.weight", "model.norm.weight", "model.layers.0.input_layernorm.weight",
        "model.layers.0.post_attention_layernorm.weight", "model.layers.0.self_attn.qkv_proj.weight",
        "model.layers.0.self_attn.o_proj.weight", "model.layers.0.self_attn.q_norm.weight",
        "model.layers.0.self_attn.k_norm.weight", "model.layers.0.mlp.gate_up_proj.weight", "model.layers.0.mlp.down_proj.weight"}


def test_load_state_dict_attaches_quant_params_and_drops_hadamard_matrices(tp1):
    from mini_sgl_integer_b200.models.utils_integer import GatedMLPInteger
    mlp = GatedMLPInteger(_config(), layer_id=0)
    sd = {"mlp.gate_up_proj.weight": torch.zeros(1024, 256, dtype=torch.int8), "mlp.gate_up_proj.weight_scale": torch.ones(1024, 1),
          "mlp.gate_up_proj.input_scale": torch.tensor([0.5]),
          "mlp.down_proj.weight": torch.zeros(256, 512, dtype=torch.int8), "mlp.down_proj.weight_scale": torch.ones(256, 1),
          "mlp.down_proj.R4_input.weight": torch.zeros(128, 128)}
    mlp.load_state_dict(sd, prefix="mlp")
    assert not sd                                                   # everything consumed, the dense Hadamard matrix dropped
    assert mlp.gate_up_proj.weight.dtype == torch.int8 and mlp.gate_up_proj.weight_scale.shape == (1024, 1)
    assert float(mlp.gate_up_proj.input_scale) == 0.5 and hasattr(mlp.down_proj, "weight_scale")
    assert mlp._apply_hadamard and mlp._hadamard_block_size == 128
    with pytest.raises(RuntimeError, match="Unexpected keys"):
        GatedMLPInteger(_config()).load_state_dict({"gate_up_proj.weight": torch.zeros(1024, 256), "down_proj.weight": torch.zeros(256, 512),
                                                    "stray.weight": torch.zeros(1)})
    with pytest.raises(ValueError, match="Shape mismatch"):
        GatedMLPInteger(_config()).load_state_dict({"gate_up_proj.weight": torch.zeros(8, 8), "down_proj.weight": torch.zeros(256, 512)})
    with pytest.raises(KeyError):
        GatedMLPInteger(_config()).load_state_dict({"gate_up_proj.weight": torch.zeros(1024, 256)})


def test_linear_shard_sizes(tp2_rank1):
    from mini_sgl_integer_b200.layers.embedding import ParallelLMHead, VocabParallelEmbedding
    from mini_sgl_integer_b200.layers.linear import LinearColParallelMerged, LinearOProj, LinearQKVMerged, LinearRowParallel
    assert LinearQKVMerged(256, 128, 4, 2, False).weight.shape == (4 * 128, 256)          # 2 q + 1 k + 1 v heads of this rank
    assert LinearColParallelMerged(256, [512, 512], False).weight.shape == (512, 256)
    assert LinearOProj(512, 256, False).weight.shape == (256, 256)
    assert LinearRowParallel(512, 256, True).bias.shape == (256,)
    emb = VocabParallelEmbedding(1001, 64)
    assert emb.weight.shape == (501, 64) and emb.vocab_range == (501, 500)
    assert ParallelLMHead(1001, 64).weight.shape == (501, 64)
    with pytest.raises(ValueError):
        LinearOProj(513, 256, False)
    with pytest.raises(TypeError, match="int8 checkpoints"):
        LinearOProj(512, 256, False).forward(torch.zeros(2, 256, dtype=torch.int32))      # float placeholder weight


def test_rotary_tables_match_the_reference(golden):
    from mini_sgl_integer_b200.layers.rotary_integer import RotaryEmbeddingInteger, get_rope_integer
    rot = RotaryEmbeddingInteger(128, 128, 4096, 1000000.0)
    np.testing.assert_array_equal(rot._cos_sin_cache_q15[golden["rope_pos"]].numpy(), golden["rope_cache_rows"])
    l3 = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 64}
    got = get_rope_integer(128, 128, 512, 500000.0, tuple(l3.items()))
    np.testing.assert_array_equal(got._cos_sin_cache_q15[[0, 1, 7, 63, 300, 511]].numpy(), golden["rope_llama3_rows"])
    l3["low_freq_factor"] = l3["high_freq_factor"] = 2.0
    got = get_rope_integer(128, 128, 512, 500000.0, tuple(l3.items()))
    np.testing.assert_array_equal(got._cos_sin_cache_q15[[1, 63, 511]].numpy(), golden["rope_llama3_step_rows"])
    assert get_rope_integer(128, 128, 512, 500000.0, tuple(l3.items())) is got            # cached per configuration
    with pytest.raises(ValueError):
        get_rope_integer(128, 128, 64, 1e4, (("rope_type", "yarn"),))
    with pytest.raises(TypeError):
        rot.forward_q15(torch.zeros(1, dtype=torch.int32), torch.zeros(1, 128), torch.zeros(1, 128, dtype=torch.int32))
    with pytest.raises(ValueError):
        rot.forward_q15(torch.zeros(1, dtype=torch.int32), torch.zeros(1, 100, dtype=torch.int32), torch.zeros(1, 128, dtype=torch.int32))


def test_backend_registry_and_reference_form_constructors(tp2_rank1):
    from mini_sgl_integer_b200 import core
    from mini_sgl_integer_b200.attention import SUPPORTED_ATTENTION_BACKENDS, B200Int8Backend, create_attention_backend
    from mini_sgl_integer_b200.kvcache import BaseKVCache, Int8PagedKVCache
    assert "b200_int8" in SUPPORTED_ATTENTION_BACKENDS.supported_names()
    with pytest.raises(KeyError):
        SUPPORTED_ATTENTION_BACKENDS["triton_int8"]
    kv = SimpleNamespace(device=torch.device("cpu"))
    be = create_attention_backend("b200_int8", SimpleNamespace(num_qo_heads=16, num_kv_heads=8, head_dim=128), kv)
    assert isinstance(be, B200Int8Backend) and be.qo_head_local == 8 and be.kv_head_local == 4 and be.requires_q_scale_fusion
    table = torch.zeros((4, 8), dtype=torch.int32)
    core.set_global_ctx(core.Context(page_size=16, page_table=table), replace=True)
    try:
        assert be.page_table is table                                # read from the global context, like the reference
    finally:
        core.set_global_ctx(None)
    assert issubclass(Int8PagedKVCache, BaseKVCache)
    with pytest.raises(TypeError, match="int8"):
        Int8PagedKVCache(8, 1, 128, 4, torch.bfloat16, "cuda")
    with pytest.raises(RuntimeError, match="GPU memory"):
        Int8PagedKVCache(8, 1, 128, 4, torch.int8, "cpu")            # reference argument order; heads split by tp info


def test_context_rules():
    from mini_sgl_integer_b200 import core
    core.set_global_ctx(None)
    with pytest.raises(RuntimeError):
        core.get_global_ctx()
    ctx = core.Context()
    core.set_global_ctx(ctx)
    with pytest.raises(RuntimeError, match="already set"):
        core.set_global_ctx(core.Context())
    batch = core.Batch(reqs=[core.Req(0, 0, 5)], phase="prefill")
    with ctx.forward_batch(batch):
        assert core.get_global_ctx().batch is batch and batch.is_prefill and batch.size == 1 and batch.reqs[0].extend_len == 5
        with pytest.raises(RuntimeError, match="Nested"):
            with ctx.forward_batch(batch):
                pass
    with pytest.raises(RuntimeError, match="No active batch"):
        ctx.batch
    core.set_global_ctx(None)
