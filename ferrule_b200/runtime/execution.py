"""Execution ABI between the runtime and a model runner: one packed, ragged batch.

A batch is a flat list of token rows plus one record per sequence describing which rows
belong to it, how much context is already in the KV pool, and which pages it may touch.
`ExecutionBatch.validate` enforces the contract before anything reaches a device, and
`ExecutionOutput.validate` checks what comes back (strictly increasing rows, top-k sorted
logit-descending / token-ascending, finite values).

Counterpart of crates/ferrule-common/src/execution.rs:182-200 (batch), :300-501 (validator),
:678-692 (capabilities), :756-821 (output validator), :972-1060 (KV schema types).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, List, Optional, Sequence, Tuple


class ExecutionError(ValueError):
    pass


class Phase(Enum):
    PREFILL = "prefill"
    DECODE = "decode"


class Intent(Enum):
    COMMITTED = "committed"                       # rows become part of the sequence
    PROVISIONAL_VERIFICATION = "provisional"      # speculative rows, kept only up to the accepted prefix


class LogitsKind(Enum):
    NONE = 0
    TOPK = 1
    FULL = 2


@dataclass(frozen=True)
class LogitsRequest:
    kind: LogitsKind = LogitsKind.NONE
    k: int = 0

    @staticmethod
    def none() -> "LogitsRequest":
        return LogitsRequest(LogitsKind.NONE, 0)

    @staticmethod
    def topk(k: int) -> "LogitsRequest":
        return LogitsRequest(LogitsKind.TOPK, k)

    @staticmethod
    def full() -> "LogitsRequest":
        return LogitsRequest(LogitsKind.FULL, 0)


@dataclass(frozen=True)
class KvPlaneDescriptor:
    name: str
    elements_per_token: int
    layer_count: int


@dataclass(frozen=True)
class KvLayoutSchema:
    """Which planes a token occupies in the pool, and the paging geometry."""
    planes: Tuple[KvPlaneDescriptor, ...]
    page_size: int
    max_sequence_len: int

    def pages_for_tokens(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    def bytes_per_page(self, element_bytes: int = 2) -> int:
        return sum(p.elements_per_token * p.layer_count for p in self.planes) * self.page_size * element_bytes


@dataclass(frozen=True)
class KvCowReplacement:
    logical_page: int      # index of the page inside the sequence
    source: int            # physical page holding the shared rows
    replacement: int       # private physical page that receives the copy


@dataclass
class SequenceSlice:
    state_slot: int
    phase: Phase
    query_start: int       # first row of this sequence in the batch
    query_len: int
    context_len: int       # tokens already committed in the KV pool before this batch
    sequence_len: int      # context_len + query_len
    block_start: int       # range into ExecutionBatch.block_ids
    block_len: int
    cow: Tuple[KvCowReplacement, ...] = ()


@dataclass
class ExecutionBatch:
    token_ids: List[int]
    positions: List[int]
    write_slots: List[int]             # pool row per token (page * page_size + offset)
    logits: List[LogitsRequest]
    sequences: List[SequenceSlice]
    block_ids: List[int]
    intent: Intent = Intent.COMMITTED
    page_size: int = 16

    @property
    def rows(self) -> int:
        return len(self.token_ids)

    def validate(self, caps: Optional["ExecutionCapabilities"] = None) -> None:
        n = self.rows
        if n == 0:
            raise ExecutionError("empty batch")
        if not (len(self.positions) == len(self.write_slots) == len(self.logits) == n):
            raise ExecutionError("row arrays have different lengths")
        if not self.sequences:
            raise ExecutionError("no sequences")
        cursor = 0
        seen_slots = set()
        for i, s in enumerate(self.sequences):
            if s.query_start != cursor:
                raise ExecutionError(f"sequence {i}: query span not contiguous (starts {s.query_start}, expected {cursor})")
            if s.query_len <= 0:
                raise ExecutionError(f"sequence {i}: empty query span")
            if s.state_slot in seen_slots:
                raise ExecutionError(f"sequence {i}: duplicate state slot {s.state_slot}")
            seen_slots.add(s.state_slot)
            if s.sequence_len != s.context_len + s.query_len:
                raise ExecutionError(f"sequence {i}: sequence_len != context_len + query_len")
            if s.context_len < 0:
                raise ExecutionError(f"sequence {i}: negative context")
            if s.phase == Phase.DECODE and s.query_len != 1 and self.intent == Intent.COMMITTED:
                raise ExecutionError(f"sequence {i}: decode phase must carry exactly one row")
            if self.intent == Intent.PROVISIONAL_VERIFICATION and s.phase != Phase.PREFILL:
                raise ExecutionError(f"sequence {i}: provisional verification rows use the prefill phase")
            if s.block_start < 0 or s.block_start + s.block_len > len(self.block_ids):
                raise ExecutionError(f"sequence {i}: block table range out of bounds")
            need = (s.sequence_len + self.page_size - 1) // self.page_size
            if s.block_len < need:
                raise ExecutionError(f"sequence {i}: {s.block_len} pages cannot hold {s.sequence_len} tokens")
            blocks = self.block_ids[s.block_start:s.block_start + s.block_len]
            for j in range(s.query_len):
                r = s.query_start + j
                pos = s.context_len + j
                if self.positions[r] != pos:
                    raise ExecutionError(f"sequence {i}: position discontinuity at row {r}")
                expect = blocks[pos // self.page_size] * self.page_size + pos % self.page_size
                if self.write_slots[r] != expect:
                    raise ExecutionError(f"sequence {i}: write slot of row {r} does not match its page binding")
            cursor += s.query_len
        if cursor != n:
            raise ExecutionError("rows not covered by sequences")
        if len(set(self.write_slots)) != n:
            raise ExecutionError("duplicate KV write slot")
        for r, tok in enumerate(self.token_ids):
            if tok < 0:
                raise ExecutionError(f"row {r}: negative token id")
        for r, lr in enumerate(self.logits):
            if lr.kind == LogitsKind.TOPK and lr.k <= 0:
                raise ExecutionError(f"row {r}: top-k request with k <= 0")
        if caps is not None:
            caps.check(self)

    def logit_rows(self) -> List[int]:
        return [r for r, lr in enumerate(self.logits) if lr.kind != LogitsKind.NONE]


class KvBindingMode(Enum):
    PAGED = "paged"
    CONTIGUOUS = "contiguous"


class LogitsRowPolicy(Enum):
    PER_ROW = "per_row"
    LAST_ROW_ONLY = "last_row_only"


@dataclass(frozen=True)
class ExecutionCapabilities:
    """What a runner accepts; the runtime lowers batches inside these bounds."""
    kv_binding: KvBindingMode = KvBindingMode.PAGED
    max_batch_rows: int = 4096
    max_sequences: int = 256
    max_decode_rows_per_sequence: int = 1
    max_topk: int = 40
    logits_rows: LogitsRowPolicy = LogitsRowPolicy.PER_ROW
    supports_provisional: bool = True
    supports_full_logits: bool = False

    def check(self, b: ExecutionBatch) -> None:
        if b.rows > self.max_batch_rows:
            raise ExecutionError(f"batch has {b.rows} rows, runner accepts {self.max_batch_rows}")
        if len(b.sequences) > self.max_sequences:
            raise ExecutionError("too many sequences for the runner")
        if b.intent == Intent.PROVISIONAL_VERIFICATION and not self.supports_provisional:
            raise ExecutionError("runner does not support provisional verification")
        for r, lr in enumerate(b.logits):
            if lr.kind == LogitsKind.TOPK and lr.k > self.max_topk:
                raise ExecutionError(f"row {r}: top-{lr.k} exceeds the runner limit {self.max_topk}")
            if lr.kind == LogitsKind.FULL and not self.supports_full_logits:
                raise ExecutionError(f"row {r}: full logits not supported")
        if self.logits_rows == LogitsRowPolicy.LAST_ROW_ONLY:
            for s in b.sequences:
                for j in range(s.query_len - 1):
                    if b.logits[s.query_start + j].kind != LogitsKind.NONE:
                        raise ExecutionError("runner only produces logits for the last row of a sequence")


@dataclass
class RowOutput:
    input_row: int
    token_ids: List[int]               # top-k ids (k >= 1), best first
    logits: List[float]
    full_logits: Optional[Sequence[float]] = None

    @property
    def top1(self) -> Optional[int]:
        return self.token_ids[0] if self.token_ids else None


@dataclass
class ExecutionOutput:
    rows: List[RowOutput] = field(default_factory=list)

    def validate(self, batch: ExecutionBatch) -> None:
        want = batch.logit_rows()
        got = [r.input_row for r in self.rows]
        if got != sorted(got) or len(set(got)) != len(got):
            raise ExecutionError("output rows are not strictly increasing")
        if got != want:
            raise ExecutionError(f"output rows {got} do not match requested rows {want}")
        for ro in self.rows:
            req = batch.logits[ro.input_row]
            if len(ro.token_ids) != len(ro.logits):
                raise ExecutionError(f"row {ro.input_row}: ids and logits differ in length")
            if req.kind == LogitsKind.TOPK and len(ro.token_ids) > req.k:
                raise ExecutionError(f"row {ro.input_row}: more candidates than requested")
            for a in range(len(ro.logits)):
                if not math.isfinite(ro.logits[a]):
                    raise ExecutionError(f"row {ro.input_row}: non-finite logit")
                if a:
                    if ro.logits[a] > ro.logits[a - 1]:
                        raise ExecutionError(f"row {ro.input_row}: candidates not sorted by logit")
                    if ro.logits[a] == ro.logits[a - 1] and ro.token_ids[a] <= ro.token_ids[a - 1]:
                        raise ExecutionError(f"row {ro.input_row}: tied candidates not in token order")
            if ro.full_logits is not None and any(not math.isfinite(v) for v in ro.full_logits):
                raise ExecutionError(f"row {ro.input_row}: non-finite full logits")

    def by_row(self) -> Dict[int, RowOutput]:
        return {r.input_row: r for r in self.rows}
