from .kv_pool import Int8PagedKVCache, PAGE_SIZE  # noqa: F401
from .ops import decode_attention_int8_paged, extend_attention_int8_paged, qkv_rope_quant_store  # noqa: F401
