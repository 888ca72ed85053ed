from .qwen3_integer import Qwen3DecoderLayerInteger, Qwen3ForCausalLMInteger, Qwen3ModelInteger  # noqa: F401
