"""Resident scheduler: admission, chunked prefill, decode cohorts, mixed batches.

Every decision first admits waiting requests (FIFO, while a sequence slot is free and
`active < max_active_sequences`), then - unless the decode cohort is being deferred - takes
up to `max_decode_batch` ready decode rows under `max_batch_tokens`, then fills what is left
of the token budget with prefill chunks (`min(prefill_chunk_size, remaining)`, round-robin).
Mixed mode returns one `Execute` action; otherwise a `DecodeBatch` or a single
`PrefillChunk`.  Decode may be deferred at most `decode_cohort_max_deferrals` times while the
cohort is below target and prefill work exists.

Counterpart of crates/ferrule-runtime/src/scheduling/resident.rs:44-78 (config), :513-550
(admission), :588-681 (batch policy), :827-960 (commit/finish/suspend), and
scheduling/actions.rs:25-60.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, Dict, List, Optional, Tuple, Union

from .session import FinishReason, SeqStatus, SequenceState, SlotPool


@dataclass
class SchedulerConfig:
    max_active_sequences: int = 64
    max_decode_batch: int = 64
    max_batch_tokens: int = 4096
    prefill_chunk_size: int = 256
    mixed_batches: bool = True
    decode_cohort_target: int = 1
    decode_cohort_max_deferrals: int = 0
    ctx_size: int = 4096


@dataclass
class Execute:
    prefills: List[Tuple[SequenceState, int]]      # (sequence, tokens in this chunk)
    decodes: List[SequenceState]


@dataclass
class PrefillChunk:
    seq: SequenceState
    tokens: int


@dataclass
class DecodeBatch:
    seqs: List[SequenceState]


@dataclass
class Finish:
    seq: SequenceState
    reason: FinishReason


@dataclass
class Cancel:
    seq: SequenceState


SchedulerAction = Union[Execute, PrefillChunk, DecodeBatch, Finish, Cancel]


@dataclass
class SchedulerStats:
    admitted: int = 0
    finished: int = 0
    cancelled: int = 0
    deferrals: int = 0
    prefill_chunks: int = 0
    prefill_tokens: int = 0
    decode_rows: int = 0
    queue_depth_high_water: int = 0


class ResidentScheduler:
    def __init__(self, cfg: SchedulerConfig):
        self.cfg = cfg
        self.slots = SlotPool(cfg.max_active_sequences)
        self.waiting: Deque[SequenceState] = deque()
        self.prefill: Deque[SequenceState] = deque()
        self.decode_ready: Deque[SequenceState] = deque()
        self.active: Dict[str, SequenceState] = {}
        self.pending_cancel: Deque[SequenceState] = deque()
        self.suspended: Dict[str, SequenceState] = {}
        self._deferrals = 0
        self.stats = SchedulerStats()

    # ------------------------------------------------------------------ intake
    def submit(self, seq: SequenceState) -> None:
        if seq.request_id in self.active or any(s.request_id == seq.request_id for s in self.waiting):
            raise ValueError(f"duplicate request id {seq.request_id}")
        seq.status = SeqStatus.WAITING
        self.waiting.append(seq)
        self.stats.queue_depth_high_water = max(self.stats.queue_depth_high_water, len(self.waiting))

    def _admit(self) -> None:
        while self.waiting and len(self.active) < self.cfg.max_active_sequences:
            held = self.waiting[0].held_slot
            slot = held if held >= 0 else self.slots.acquire()     # a continued session comes back to its own slot
            if slot is None:
                return
            seq = self.waiting.popleft()
            seq.slot, seq.held_slot = slot, -1
            self.active[seq.request_id] = seq
            self.stats.admitted += 1
            if seq.prefill_remaining > 0:
                seq.status = SeqStatus.PREFILL
                self.prefill.append(seq)
            else:                               # continued session whose prompt is already cached
                seq.status = SeqStatus.DECODE
                self.decode_ready.append(seq)

    # ------------------------------------------------------------------ policy
    def has_work(self) -> bool:
        return bool(self.waiting or self.prefill or self.decode_ready or self.pending_cancel)

    def next_action(self) -> Optional[SchedulerAction]:
        if self.pending_cancel:
            return Cancel(self.pending_cancel.popleft())
        self._admit()
        cfg = self.cfg
        budget = cfg.max_batch_tokens
        ready = [s for s in self.decode_ready if s.staged_token is not None]
        defer = (bool(self.prefill) and 0 < len(ready) < cfg.decode_cohort_target
                 and self._deferrals < cfg.decode_cohort_max_deferrals)
        decodes: List[SequenceState] = []
        if defer:
            self._deferrals += 1
            self.stats.deferrals += 1
        else:
            while ready and len(decodes) < cfg.max_decode_batch and budget > 0:
                s = ready.pop(0)
                decodes.append(s)
                budget -= 1
            if decodes:
                self._deferrals = 0
        if not cfg.mixed_batches:
            if decodes:
                return self._claim_decodes(decodes)
            if self.prefill:
                s = self.prefill.popleft()
                n = min(cfg.prefill_chunk_size, s.prefill_remaining, cfg.max_batch_tokens)
                s.status = SeqStatus.RUNNING
                self._count_prefill(n)
                return PrefillChunk(s, n)
            return None
        prefills: List[Tuple[SequenceState, int]] = []
        seen = 0
        n_pref = len(self.prefill)
        while self.prefill and budget > 0 and seen < n_pref:
            s = self.prefill.popleft()
            seen += 1
            n = min(cfg.prefill_chunk_size, s.prefill_remaining, budget)
            if n <= 0:
                self.prefill.append(s)
                continue
            prefills.append((s, n))
            budget -= n
        if not prefills and not decodes:
            return None
        for s in decodes:
            self.decode_ready.remove(s)
            s.status = SeqStatus.RUNNING
        for s, n in prefills:
            s.status = SeqStatus.RUNNING
            self._count_prefill(n)
        self.stats.decode_rows += len(decodes)
        if prefills:
            return Execute(prefills, decodes)
        return DecodeBatch(decodes)

    def _claim_decodes(self, decodes: List[SequenceState]) -> DecodeBatch:
        for s in decodes:
            self.decode_ready.remove(s)
            s.status = SeqStatus.RUNNING
        self.stats.decode_rows += len(decodes)
        return DecodeBatch(decodes)

    def _count_prefill(self, n: int) -> None:
        self.stats.prefill_chunks += 1
        self.stats.prefill_tokens += n

    # ------------------------------------------------------------------ results
    def commit_prefill(self, seq: SequenceState, tokens: int) -> None:
        """`tokens` prompt tokens are now cached.  Requeue for more prefill or move to decode."""
        seq.position += tokens
        if seq.prefill_remaining > 0:
            seq.status = SeqStatus.PREFILL
            self.prefill.append(seq)               # round-robin: back of the queue
        else:
            seq.status = SeqStatus.DECODE
            self.decode_ready.append(seq)

    def commit_decode(self, seq: SequenceState, token: int) -> None:
        """The staged token's KV is committed and the token is part of the sequence."""
        seq.tokens.append(token)
        seq.position += 1
        seq.generated += 1
        seq.staged_token = None
        seq.status = SeqStatus.DECODE
        self.decode_ready.append(seq)

    def commit_speculative(self, seq: SequenceState, tokens: List[int]) -> None:
        """Several tokens accepted at once (their KV rows are committed)."""
        seq.tokens.extend(tokens)
        seq.position += len(tokens)
        seq.generated += len(tokens)
        seq.staged_token = None
        seq.status = SeqStatus.DECODE
        self.decode_ready.append(seq)

    def requeue_unchanged(self, seq: SequenceState) -> None:
        """A transaction aborted without effect: put the sequence back where it was."""
        if seq.prefill_remaining > 0:
            seq.status = SeqStatus.PREFILL
            self.prefill.appendleft(seq)
        else:
            seq.status = SeqStatus.DECODE
            self.decode_ready.appendleft(seq)

    def release_held(self, seq: SequenceState) -> int:
        """Return a retained session's slot to the pool -> the slot (or -1)."""
        slot, seq.held_slot = seq.held_slot, -1
        if slot >= 0:
            self.slots.release(slot)
        return slot

    def stage(self, seq: SequenceState, token: int) -> None:
        seq.staged_token = token

    def finish(self, seq: SequenceState, reason: FinishReason, keep_slot: bool = False) -> None:
        """`keep_slot`: the sequence becomes a retained session of a runner whose state lives in the slot - the
        slot stays out of the pool (`held_slot`) until the session continues or is dropped (`release_held`)."""
        seq.finish = reason
        seq.status = SeqStatus.FINISHED
        for q in (self.prefill, self.decode_ready, self.waiting):
            if seq in q:
                q.remove(seq)
        if self.active.pop(seq.request_id, None) is not None and seq.slot >= 0:
            if keep_slot:
                seq.held_slot = seq.slot
            else:
                self.slots.release(seq.slot)
            seq.slot = -1
        elif seq.held_slot >= 0 and not keep_slot:
            self.release_held(seq)                 # ended while still waiting for admission
        if reason == FinishReason.CANCELLED:
            self.stats.cancelled += 1
        else:
            self.stats.finished += 1

    def cancel(self, request_id: str) -> Optional[SequenceState]:
        """Cooperative: a running sequence is cancelled when its transaction ends."""
        for s in list(self.waiting):
            if s.request_id == request_id:
                self.waiting.remove(s)
                s.finish, s.status = FinishReason.CANCELLED, SeqStatus.FINISHED
                self.stats.cancelled += 1
                return s
        s = self.active.get(request_id)
        if s is None:
            return None
        if s.status == SeqStatus.RUNNING:
            s.finish = FinishReason.CANCELLED        # honoured at transaction end
            return s
        for q in (self.prefill, self.decode_ready):
            if s in q:
                q.remove(s)
        self.pending_cancel.append(s)
        return s

    # ------------------------------------------------------------------ suspend / restore
    def suspend(self, seq: SequenceState) -> None:
        for q in (self.prefill, self.decode_ready):
            if seq in q:
                q.remove(seq)
        seq.status = SeqStatus.SUSPENDED
        self.suspended[seq.request_id] = seq

    def resume(self, seq: SequenceState) -> None:
        self.suspended.pop(seq.request_id, None)
        self.requeue_unchanged(seq)
