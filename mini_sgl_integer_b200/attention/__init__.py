from .kv_pool import Int8PagedKVCache, PAGE_SIZE  # noqa: F401
from .ops import (  # noqa: F401
    decode_attention_int8_paged, extend_attention_int8_paged, prefill_attention_int8_paged, qkv_rope_quant_store,
    quantize_per_tensor_int8_ms,
)
from .backend import B200Int8Backend, BaseAttnBackend, BaseAttnMetadata, Int8Metadata  # noqa: F401,E402


class Registry:
    """name -> factory (utils/registry.py:6-40)."""

    def __init__(self, kind: str):
        self._kind, self._items = kind, {}

    def register(self, name: str):
        if name in self._items:
            raise KeyError(f"{self._kind} '{name}' is already registered.")

        def decorator(item):
            self._items[name] = item
            return item
        return decorator

    def __getitem__(self, name: str):
        if name not in self._items:
            raise KeyError(f"Unsupported {self._kind}: {name}")
        return self._items[name]

    def supported_names(self):
        return list(self._items)


# The registry the reference selects backends from with ``--attn`` (attention/__init__.py:20-37); this package
# registers one name.  Inside the reference, the same two lines register it next to "triton_int8".
SUPPORTED_ATTENTION_BACKENDS = Registry("Attention Backend")


@SUPPORTED_ATTENTION_BACKENDS.register("b200_int8")
def create_b200_int8_backend(config, kvcache):
    return B200Int8Backend(config, kvcache)


def create_attention_backend(backend: str, config, kvcache):
    """attention/__init__.py:66-89 for the one backend of this package."""
    return SUPPORTED_ATTENTION_BACKENDS[backend](config, kvcache)
