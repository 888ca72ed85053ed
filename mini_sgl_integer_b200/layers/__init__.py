from .w8a8_int8 import W8A8Int8LinearMethod, int8_gemm_q15, weight_scale_to_mul_shift  # noqa: F401
from .activation_integer import silu_and_mul_fixed, silu_and_mul_q15  # noqa: F401,E402
from .base import BaseOP, OPList, StateLessOP  # noqa: F401,E402
from .norm_integer import RMSNormFusedInteger, RMSNormInteger  # noqa: F401,E402
from .rotary_integer import RotaryEmbeddingInteger, get_rope_integer  # noqa: F401,E402
