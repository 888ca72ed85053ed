from .w8a8_int8 import W8A8Int8LinearMethod, int8_gemm_q15, weight_scale_to_mul_shift  # noqa: F401
