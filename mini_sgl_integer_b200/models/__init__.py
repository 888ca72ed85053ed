from .qwen3_integer import (  # noqa: F401
    DecodeBatch, Qwen3ForCausalLMInteger, check_device_status, Qwen3IntegerConfig, Qwen3ModelInteger, argmax_int32, embedding_to_fixed,
    merge_sharded_argmax, random_weights, rope_cache_q15, shard_layer_weights,
)
