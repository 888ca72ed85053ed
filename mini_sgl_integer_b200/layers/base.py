"""State-dict plumbing of the layer classes: the interface of ``minisgl.layers.base`` (layers/base.py:16-160).

A ``BaseOP`` owns tensors and other ``BaseOP`` objects as plain attributes (names starting with ``_`` are private
buffers).  ``load_state_dict`` replaces every tensor attribute by the checkpoint's tensor of the same dotted name
and, as the reference does for W8A8 checkpoints (:85-106), attaches ``weight_scale`` / ``input_scale`` /
``input_zero_point`` as extra attributes of the layer that owns the weight, and drops the dense Hadamard matrices
(``R<n>_input.weight``) of compressed-tensors checkpoints: the integer path rotates with the FWHT kernels.
"""
from __future__ import annotations

import re
from typing import Dict, Generic, List, Optional, TypeVar

import torch

StateDict = Dict[str, torch.Tensor]
_QUANT_PARAMS = ("weight_scale", "input_scale", "input_zero_point")
_HADAMARD_AUX = re.compile(r"(^|\.)R\d+_input\.weight$")


def _join(prefix: str, name: str) -> str:
    return f"{prefix}.{name}" if prefix else name


class BaseOP:
    def forward(self, *args, **kwargs):
        raise NotImplementedError

    def _members(self):
        return [(n, v) for n, v in self.__dict__.items() if not n.startswith("_")]

    def state_dict(self, *, prefix: str = "", result: Optional[StateDict] = None) -> StateDict:
        result = {} if result is None else result
        for name, value in self._members():
            if isinstance(value, torch.Tensor):
                result[_join(prefix, name)] = value
            elif isinstance(value, BaseOP):
                value.state_dict(prefix=_join(prefix, name), result=result)
        return result

    def load_state_dict(self, state_dict: StateDict, *, prefix: str = "", _internal: bool = False) -> None:
        for name, value in self._members():
            if isinstance(value, torch.Tensor):
                key = _join(prefix, name)
                if key not in state_dict:
                    raise KeyError(f"missing key in state_dict: {key}")
                item = state_dict.pop(key)
                # the placeholder only fixes the shape; the checkpoint's dtype wins (int8 weights, bf16 tables, float
                # norm gains - the reference compares dtypes too, but builds its placeholders under the model's
                # default dtype, which this package does not set)
                if value.shape != item.shape:
                    raise ValueError(f"Shape mismatch for {key}: {tuple(value.shape)} vs {tuple(item.shape)}")
                setattr(self, name, item)
            elif isinstance(value, BaseOP):
                value.load_state_dict(state_dict, prefix=_join(prefix, name), _internal=True)
        dotted = prefix + "." if prefix else ""
        for key in [k for k in state_dict if not prefix or k.startswith(dotted)]:
            rel = key[len(dotted):]
            if any(rel == q or rel.endswith("." + q) for q in _QUANT_PARAMS):
                setattr(self, rel.replace(".", "_"), state_dict.pop(key))
            elif _HADAMARD_AUX.search(rel):
                state_dict.pop(key)
        if not _internal and state_dict:
            raise RuntimeError(f"Unexpected keys in state_dict: {list(state_dict.keys())}")


class StateLessOP(BaseOP):
    def load_state_dict(self, state_dict: StateDict, *, prefix: str = "", _internal: bool = False) -> None:
        if not _internal and state_dict:
            raise RuntimeError(f"Unexpected keys in state_dict: {list(state_dict.keys())}")

    def state_dict(self, *, prefix: str = "", result: Optional[StateDict] = None) -> StateDict:
        return {} if result is None else result


T = TypeVar("T", bound=BaseOP)


class OPList(BaseOP, Generic[T]):
    def __init__(self, ops: List[T]):
        self.op_list = ops

    def state_dict(self, *, prefix: str = "", result: Optional[StateDict] = None) -> StateDict:
        result = {} if result is None else result
        for i, op in enumerate(self.op_list):
            op.state_dict(prefix=_join(prefix, str(i)), result=result)
        return result

    def load_state_dict(self, state_dict: StateDict, *, prefix: str = "", _internal: bool = False) -> None:
        for i, op in enumerate(self.op_list):
            op.load_state_dict(state_dict, prefix=_join(prefix, str(i)), _internal=True)
        if not _internal and state_dict:
            raise RuntimeError(f"Unexpected keys in state_dict: {list(state_dict.keys())}")
