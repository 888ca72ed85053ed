from .kv_pool import Int8PagedKVCache, PAGE_SIZE  # noqa: F401
from .ops import (  # noqa: F401
    decode_attention_int8_paged, extend_attention_int8_paged, prefill_attention_int8_paged, qkv_rope_quant_store,
    quantize_per_tensor_int8_ms,
)
