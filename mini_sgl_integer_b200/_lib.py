"""ctypes binding of ``libb200int.so`` (the C ABI declared in ``include/b200int.h``).

There is no fallback: if the library has not been built, or an entry point
rejects its arguments, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_void_p

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libb200int.so")

P, I, L = c_void_p, c_int, c_int64

# name -> argument types (every function returns int unless listed in _RESTYPES)
SIGNATURES: dict[str, list] = {
    "b200_version": [],
    "b200_last_error_string": [],
    "b200_get_lut": [I, P],
    "b200_to_fixed_f32": [P, P, L, P],
    "b200_to_fixed_bf16": [P, P, L, P],
    "b200_from_fixed_f32": [P, P, L, P],
    "b200_from_fixed_bf16": [P, P, L, P],
    "b200_rmsnorm_q15": [P, P, P, P, P, P, P, P, L, I, P],
    "b200_silu_mul_q15": [P, P, P, P, P, L, I, I, P],
    "b200_fwht_q15": [P, P, L, I, I, P],
    "b200_qk_rope_q15": [P, P, L, P, L, P, I, P, P, P, P, L, I, I, I, P],
    "b200_per_token_quant_q15": [P, P, P, P, L, I, P],
    "b200_absmax_to_mul_shift": [P, P, P, L, P],
    "b200_kv_store_q15": [P, L, P, L, P, P, P, P, L, I, L, P],
    "b200_kv_store_codes": [P, P, P, P, P, P, P, P, P, P, L, I, L, P],
    "b200_attn_extend": [P, P, P, P, P, P, P, L, P, P, P, P, P, P, I, I, I, L, I, I, P],
    "b200_attn_prefill": [P, P, P, P, P, P, P, L, P, P, P, P, P, P, I, I, I, I, L, I, P],
    "b200_attn_workspace_bytes": [I, I, I, I],
    "b200_attn_paged_ws": [P, P, P, P, P, P, P, L, P, P, P, P, P, P, I, I, I, L, I, P, ctypes.c_size_t, P],
    "b200_attn_paged_static": [P, P, P, P, P, P, P, L, P, P, P, P, P, P, I, I, I, L, I, P],
    "b200_embedding_bf16_q15": [P, P, P, L, I, L, L, P],
    "b200_argmax_i32": [P, L, L, L, I, P, P, P],
    "b200_decode_prepare": [P, L, P, P, P, P, I, I, P],
    "b200_static_quant_q15": [P, ctypes.c_float, P, L, P],
    "b200_qkv_prepare_q15": [P, P, L, P, L, P, L, P, I, P, P, P, P, P, P, P, P, P, L, I, I, L, I, P],
    "b200_gemm_w8a8": [P, P, P, P, P, P, P, P, L, L, L, P],
    "b200_gemm_w8a8_absmax": [P, P, P, P, P, P, P, L, L, L, P],
    "b200_gemm_w8a8_reduce_peers": [P, P, P, I, L, L, L, P],
    "b200_gemm_w8a8_absmax_ws": [P, P, P, P, P, P, P, L, L, L, P],
    "b200_gemm_w8a8_acc_ws": [P, P, P, L, L, L, P],
    "b200_gemm_gate_up_silu": [P, P, P, P, P, P, P, L, L, L, P],
    "b200_fwht_quant_q15": [P, P, P, P, L, I, I, P],
    "b200_rmsnorm_q15_pending": [P, P, P, P, P, P, P, P, P, P, P, L, I, P],
    "b200_qkv_prepare_pending": [P, P, P, P, P, P, I, P, P, P, P, P, P, P, P, P, L, I, I, L, I, P],
    "b200_gemm_status": [P, I],
    "b200_quant_given_absmax_q15": [P, P, P, L, I, P],
    "b200_requant_q15": [P, P, P, P, P, P, L, L, P],
    "b200_attn_decode": [P, P, P, P, P, P, P, L, P, P, P, P, P, I, I, I, L, I, I, P],
    "b200_quantize_per_tensor_int8_ms": [P, L, P, P, P, P],
    "b200_tp_block_bytes": [I, L],
    "b200_tp_block_clear": [P, P],
    "b200_tp_absmax_put": [P, P, L, I, I, P],
    "b200_tp_quant_wait": [P, P, L, I, I, P, P, P],
    "b200_tp_absmax_quant": [P, P, L, I, I, P, P, P],
    "b200_gemm_w8a8_tp": [P, P, P, L, L, L, P],
    "b200_tp_requant_scatter": [P, P, P, P, I, P],
    "b200_tp_collect": [P, P, I, P],
    "b200_tp_requant_direct": [P, P, P, P, P, I, P],
    "b200_tp_all_gather": [P, P, I, P, P],
    "b200_tp_owner_norm": [P, P, P, P, P, P, I, P],
    "b200_tp_collect_codes": [P, P, P, I, P],
    "b200_tp_silu_absmax_quant": [P, P, P, P, I, I, I, P],
    "b200_tp_status": [P, I],
    "b200_tp_set_timeout_us": [L],
}
_RESTYPES = {"b200_last_error_string": c_char_p, "b200_attn_workspace_bytes": ctypes.c_size_t,
             "b200_tp_block_bytes": ctypes.c_size_t}

_lib = None


class B200Error(RuntimeError):
    """An entry point of libb200int.so returned a negative status."""

    def __init__(self, name: str, code: int, message: str):
        super().__init__(f"{name} failed with status {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mini_sgl_integer_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError here = header and library disagree
            fn.argtypes = args
            fn.restype = _RESTYPES.get(name, c_int)
        _lib = lib
    return _lib


CALLS = 0      # entry-point calls made through `call` (bench.py counts the launches of a captured step with it)


def call(name: str, *args) -> None:
    global CALLS
    lib = load()
    CALLS += 1
    rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.b200_last_error_string().decode("utf-8", "replace")
        raise B200Error(name, rc, msg)


def ptr(t: torch.Tensor | None):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


def stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "this op only runs on a CUDA device (sm_100a); got a tensor on "
                f"{t.device} — there is no CPU fallback"
            )
