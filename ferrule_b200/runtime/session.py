"""Requests, per-sequence state and finish reasons.

Counterpart of crates/ferrule-runtime/src/scheduling/session.rs:27-112 and the fixed
slot pool of scheduling/slot_pool.rs:13-62.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import List, Optional


class FinishReason(Enum):
    MAX_TOKENS = "max_tokens"
    EOS = "eos"
    STOP_STRING = "stop_string"
    CONTEXT = "context"
    NO_CANDIDATE = "no_candidate"
    CANCELLED = "cancelled"
    ERROR = "error"

    def openai(self) -> str:
        """OpenAI `finish_reason` string."""
        if self in (FinishReason.MAX_TOKENS, FinishReason.CONTEXT):
            return "length"
        if self == FinishReason.CANCELLED:
            return "cancelled"
        if self == FinishReason.ERROR:
            return "error"
        return "stop"


@dataclass
class GenerateRequest:
    request_id: str
    prompt_tokens: List[int]
    max_new_tokens: int = 16
    stop: List[str] = field(default_factory=list)
    ignore_eos: bool = False
    session_id: Optional[str] = None       # continue / retain a named session across requests
    retain_session: bool = False


class SeqStatus(Enum):
    WAITING = "waiting"
    PREFILL = "prefill"
    DECODE = "decode"
    RUNNING = "running"          # claimed by an in-flight transaction
    SUSPENDED = "suspended"      # preempted to host
    FINISHED = "finished"


@dataclass
class SequenceState:
    request: GenerateRequest
    slot: int = -1                         # logical state slot
    held_slot: int = -1                    # slot a retained session keeps between requests (slot-bound runner state)
    kv_seq: int = -1                       # KvPageManager sequence id
    status: SeqStatus = SeqStatus.WAITING
    tokens: List[int] = field(default_factory=list)   # prompt + committed generated tokens
    prompt_len: int = 0
    position: int = 0                      # tokens whose KV is committed
    generated: int = 0
    staged_token: Optional[int] = None     # greedy token chosen for the next decode row
    text: str = ""
    decoder: object = None                 # utils.tokenizer.IncrementalDecodeState of the generated tokens
    finish: Optional[FinishReason] = None
    arrival_ns: int = 0
    first_token_ns: int = 0
    last_token_ns: int = 0
    deferrals: int = 0
    hidden_tap: object = None              # model-owned handle for the MTP head (opaque)

    @property
    def request_id(self) -> str:
        return self.request.request_id

    @property
    def prefill_remaining(self) -> int:
        return max(self.prompt_len - self.position, 0)


class SlotPool:
    """Fixed pool of logical sequence slots."""

    def __init__(self, n: int):
        self._free = list(range(n - 1, -1, -1))
        self.capacity = n

    def acquire(self) -> Optional[int]:
        return self._free.pop() if self._free else None

    def release(self, slot: int) -> None:
        if slot in self._free or not 0 <= slot < self.capacity:
            raise ValueError(f"slot {slot} released twice or out of range")
        self._free.append(slot)

    @property
    def available(self) -> int:
        return len(self._free)
