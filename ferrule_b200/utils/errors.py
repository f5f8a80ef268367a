"""Cross-layer error type and the GGUF quantisation-type table.

`FerruleError` carries a kind, a context chain (outermost first) and, for failures that happened
while several things had to be undone, the list of clean-up failures and of per-item failures of a
batch.  Counterpart of crates/ferrule-common/src/lib.rs:32-140 (Error) and :143-227 (QuantType).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, List, Optional


class ErrorKind(Enum):
    INVALID_ARGUMENT = "invalid_argument"
    NOT_FOUND = "not_found"
    UNSUPPORTED = "unsupported"
    RESOURCE_EXHAUSTED = "resource_exhausted"
    IO = "io"
    DEVICE = "device"
    PROTOCOL = "protocol"
    CANCELLED = "cancelled"
    INTERNAL = "internal"


class FerruleError(Exception):
    def __init__(self, kind: ErrorKind, message: str, *, retryable: bool = False,
                 cleanup: Optional[List[BaseException]] = None, batch: Optional[Dict[str, BaseException]] = None):
        super().__init__(message)
        self.kind, self.message, self.retryable = kind, message, retryable
        self.contexts: List[str] = []
        self.cleanup_failures: List[BaseException] = list(cleanup or [])
        self.batch_failures: Dict[str, BaseException] = dict(batch or {})

    def context(self, what: str) -> "FerruleError":
        self.contexts.insert(0, what)
        return self

    def __str__(self) -> str:
        chain = ": ".join(self.contexts + [self.message])
        extra = ""
        if self.cleanup_failures:
            extra += f" (+{len(self.cleanup_failures)} clean-up failure(s))"
        if self.batch_failures:
            extra += f" (+{len(self.batch_failures)} failed item(s))"
        return f"[{self.kind.value}] {chain}{extra}"


@dataclass(frozen=True)
class QuantType:
    name: str
    ggml_id: int
    block_elems: int
    block_bytes: int

    def bytes_for(self, elems: int) -> int:
        return (elems + self.block_elems - 1) // self.block_elems * self.block_bytes


QUANT_TYPES: Dict[int, QuantType] = {q.ggml_id: q for q in [
    QuantType("F32", 0, 1, 4), QuantType("F16", 1, 1, 2), QuantType("Q4_0", 2, 32, 18), QuantType("Q4_1", 3, 32, 20),
    QuantType("Q5_0", 6, 32, 22), QuantType("Q5_1", 7, 32, 24), QuantType("Q8_0", 8, 32, 34),
    QuantType("Q8_1", 9, 32, 36), QuantType("Q2_K", 10, 256, 84), QuantType("Q3_K", 11, 256, 110),
    QuantType("Q4_K", 12, 256, 144), QuantType("Q5_K", 13, 256, 176), QuantType("Q6_K", 14, 256, 210),
    QuantType("Q8_K", 15, 256, 292), QuantType("BF16", 30, 1, 2),
]}


def quant_type(ggml_id: int) -> QuantType:
    q = QUANT_TYPES.get(ggml_id)
    if q is None:
        raise FerruleError(ErrorKind.UNSUPPORTED, f"unknown GGML type id {ggml_id}")
    return q
