"""The few types of ``minisgl.core`` that the integer path reads (core.py:29-135): a request, a batch, and the
global context that carries the page table, the attention backend and the batch being run.

They exist so that the layer classes of this package run on their own (tests, the benchmark).  Inside the
reference's engine its own ``Req`` / ``Batch`` / ``Context`` objects are used instead - the classes here only read
the attributes named below, so either kind works.
"""
from __future__ import annotations

from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, List, Literal, Optional

import torch


@dataclass(eq=False)
class Req:
    """core.py:29-69, reduced to what the attention backend reads."""

    table_idx: int          # row of the request in the page table
    cached_len: int         # tokens whose K/V are already in the pool
    device_len: int         # tokens after this step's new ones

    @property
    def extend_len(self) -> int:
        return self.device_len - self.cached_len


@dataclass
class Batch:
    """core.py:72-97."""

    reqs: List[Any]
    phase: Literal["prefill", "decode"]
    input_ids: torch.Tensor = field(init=False, default=None)
    positions: torch.Tensor = field(init=False, default=None)
    out_loc: torch.Tensor = field(init=False, default=None)
    padded_reqs: List[Any] = field(init=False, default=None)
    attn_metadata: Any = field(init=False, default=None)

    def __post_init__(self) -> None:
        if self.padded_reqs is None:
            self.padded_reqs = list(self.reqs)

    @property
    def is_prefill(self) -> bool:
        return self.phase == "prefill"

    @property
    def is_decode(self) -> bool:
        return self.phase == "decode"

    @property
    def size(self) -> int:
        return len(self.reqs)

    @property
    def padded_size(self) -> int:
        return len(self.padded_reqs)


@dataclass
class Context:
    """core.py:101-122.  ``page_table``: int32 [max_requests, max_pages] of PAGE ids (16-token pages) for the
    backend of this package (the reference's table holds token locations with page size 1, core.py:103)."""

    page_size: int = 16
    page_table: Optional[torch.Tensor] = None
    attn_backend: Any = None
    _batch: Optional[Batch] = None

    @property
    def batch(self) -> Batch:
        if self._batch is None:
            raise RuntimeError("No active batch in context")
        return self._batch

    @contextmanager
    def forward_batch(self, batch: Batch):
        if self._batch is not None:
            raise RuntimeError("Nested forward_batch is not allowed")
        try:
            self._batch = batch
            yield
        finally:
            self._batch = None


_GLOBAL_CTX: Optional[Context] = None


def set_global_ctx(ctx: Optional[Context], *, replace: bool = False) -> None:
    """core.py:128-131 (may be set once; ``replace`` is for tests)."""
    global _GLOBAL_CTX
    if _GLOBAL_CTX is not None and ctx is not None and not replace:
        raise RuntimeError("Global context is already set")
    _GLOBAL_CTX = ctx


def get_global_ctx() -> Context:
    if _GLOBAL_CTX is None:
        raise RuntimeError("Global context is not set")
    return _GLOBAL_CTX
