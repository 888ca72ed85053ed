"""B200-native kernels for mini-sgl-integer's integer-only W8A8 forward path.

The sub-packages mirror the part of the ``minisgl`` Python API that sits on that
path (same names, argument meaning and error behaviour), backed by hand-written
sm_100a CUDA in ``libb200int.so``:

  kernel.fixed_point   <- minisgl.kernel.fixed_point
  layers               <- minisgl.layers.{norm_integer, activation_integer, rotary_integer,
                          quantization.w8a8_int8}
  attention            <- minisgl.attention (backend plug-in) and minisgl.kvcache (KV pool)
"""
from . import _lib  # noqa: F401

__all__ = ["kernel", "layers", "attention"]
