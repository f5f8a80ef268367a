"""The resident engine: owner of requests, scheduling, execution transactions and KV custody.

`step()` runs one owner-loop turn: drive transaction endings -> retire pages -> flush the
committed-token outbox -> progress materializations -> resume ready transactions -> ask the
scheduler for an action -> execute it as an ordinary or speculative transaction.

An ordinary transaction: lower the action to an `ExecutionBatch` -> claim the sessions ->
reserve KV pages (one hard credit per physical page) -> bind write slots -> runner
`prepare_batch` -> `execute` -> on `Complete`: prepare the logical commit ->
`end_transaction(PUBLISH)` until `COMPLETE` -> publish KV -> commit the scheduler state ->
move tokens to the outbox -> stage the next greedy token.  On `Waiting` the transaction parks
as a continuation until its dependencies are published.  An abort keeps every page, slot and
credit until the backend answers `COMPLETE`.

Tokens become visible outside only from the outbox, i.e. after their KV rows and the
scheduler state are committed.

Counterpart of crates/ferrule-runtime/src/engine/driver.rs (step :4192-4284, ordinary
transaction :3049-3204/:3282-3444, abort :3667-3775, finish rules :3858-4026, fork/preempt/
restore :1679-1795/:2310-2440, shutdown :4034-4190).
"""
from __future__ import annotations

import time
from collections import OrderedDict, deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

from .execution import (ExecutionBatch, ExecutionOutput, Intent, LogitsRequest, Phase, SequenceSlice)
from .kv_pages import KvPageManager, KvRetirement, OutOfPages
from .resources import Grant, PhysicalResourceBroker, ResourceKind
from .runner import Complete, EndIntent, EndStatus, ModelRunner, Waiting
from .scheduler import Cancel, DecodeBatch, Finish, PrefillChunk, ResidentScheduler, SchedulerConfig
from .session import FinishReason, GenerateRequest, SeqStatus, SequenceState


class MaterializationFailed(RuntimeError):
    """A payload a parked transaction needed could not be loaded.  `retryable`: the destination had no free frame
    (other parked transactions hold them) - the transaction is rolled back, gives its own frames up and its
    sequences run again; any other reason (read / upload / install error, provider lost) ends the requests."""

    def __init__(self, reason=None):
        from .io_protocol import FailureReason
        self.reason = reason
        self.retryable = reason == FailureReason.RESOURCE_EXHAUSTED
        super().__init__(f"a required materialization failed ({getattr(reason, 'value', reason)})")


@dataclass
class EngineConfig:
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    kv_pages: int = 256
    page_size: int = 16
    # a transaction that parks on missing payloads may name up to this many further payloads it expects to need
    # (the runner's `prefetch_candidates`): they are requested without a waiter, load behind the required ones and
    # stay owned by the transaction until it ends.  0 = off
    transaction_prefetch: int = 0
    # a transaction parked longer than this on its materializations is rolled back and its requests end with an
    # error (a completion the provider never delivers would otherwise hold them for ever).  0 = wait without limit
    materialization_timeout_s: float = 0.0
    speculative: bool = False
    max_draft: int = 1
    confidence_threshold: float = 0.2
    auto_preempt: bool = False          # preempt the youngest decode sequence when pages run out
    # prompt-prefix cache: finished requests leave the KV pages of their prompt (cut to whole `prefix_block`s)
    # behind, up to this many tokens in total; a later prompt that starts with the same tokens forks those pages
    # instead of recomputing them.  0 = off.  Entries go oldest-first when over budget or when pages run out.
    prefix_cache_tokens: int = 0
    prefix_block: int = 512             # granularity of a reusable prefix (a multiple of the page size)


@dataclass
class TokenEvent:
    request_id: str
    token: int
    text: str
    index: int                          # 0-based index among generated tokens


@dataclass
class FinishEvent:
    request_id: str
    reason: FinishReason
    prompt_tokens: int
    generated_tokens: int
    text: str
    ttft_s: float = 0.0
    tpot_s: float = 0.0
    tail: str = ""              # text the detokeniser still held when the stream ended (already part of `text`)


class TxnState(Enum):
    EXECUTING = "executing"
    WAITING = "waiting"
    PUBLISHING = "publishing"
    ABORTING = "aborting"
    DONE = "done"


@dataclass
class TxnSeq:
    seq: SequenceState
    res_id: int
    rows: int
    is_prefill: bool
    query_start: int = 0


@dataclass
class Transaction:
    txn_id: int
    members: List[TxnSeq]
    batch: Optional[ExecutionBatch] = None
    grant: Optional[Grant] = None
    state: TxnState = TxnState.EXECUTING
    output: Optional[ExecutionOutput] = None
    commit_id: Optional[int] = None
    speculative: object = None          # speculation.SpecCohort for verification transactions
    error: Optional[BaseException] = None
    t_start_ns: int = 0
    prefetch_ops: List[int] = field(default_factory=list)      # registry operations requested as this transaction's prefetch
    t_parked_ns: int = 0                # when it last began to wait for materializations


@dataclass
class EngineStats:
    steps: int = 0
    actions: int = 0
    transactions: int = 0
    aborted_transactions: int = 0
    prefill_chunks: int = 0
    prefill_tokens: int = 0
    decode_steps: int = 0
    decode_rows: int = 0
    emitted_tokens: int = 0
    staged_tokens: int = 0
    finished: int = 0
    kv_stalls: int = 0
    page_deadlocks: int = 0             # requests ended because no page would ever come back for them
    prefix_hits: int = 0
    prefix_tokens_reused: int = 0
    prefix_entries: int = 0
    prefix_evictions: int = 0
    auto_preemptions: int = 0
    waits: int = 0
    resumes: int = 0
    prefetch_requests: int = 0
    materialization_timeouts: int = 0   # parked transactions rolled back after `materialization_timeout_s`
    frame_deadlocks: int = 0            # parked transactions rolled back because the loads they waited for had no frame
    session_evictions: int = 0          # idle retained sessions dropped so that a request could get their slot or pages
    host_ns: int = 0
    runner_ns: int = 0
    ttft_sum_s: float = 0.0
    tpot_sum_s: float = 0.0
    e2e_sum_s: float = 0.0


EmitFn = Callable[[object], None]


class Engine:
    def __init__(self, runner: ModelRunner, cfg: Optional[EngineConfig] = None,
                 detokenize: Optional[Callable[[List[int]], str]] = None,
                 registry=None, broker: Optional[PhysicalResourceBroker] = None):
        self.runner = runner
        self.last_error: Optional[BaseException] = None
        self.cfg = cfg or EngineConfig()
        # limits the runner can never serve are refused here, before any request is taken: a full prompt chunk or a
        # full decode cohort must fit one batch of the runner
        caps, sc = runner.capabilities(), self.cfg.scheduler
        if min(sc.prefill_chunk_size, sc.max_batch_tokens) > caps.max_batch_rows or sc.max_decode_batch > caps.max_batch_rows:
            raise ValueError(f"scheduler limits (prompt chunk {sc.prefill_chunk_size}, batch tokens {sc.max_batch_tokens}, "
                             f"decode batch {sc.max_decode_batch}) exceed the runner's {caps.max_batch_rows} rows per batch")
        if sc.max_decode_batch > caps.max_sequences:
            raise ValueError(f"decode batch of {sc.max_decode_batch} sequences exceeds the runner's {caps.max_sequences}")
        self.scheduler = ResidentScheduler(self.cfg.scheduler)
        self.kv = KvPageManager(self.cfg.kv_pages, self.cfg.page_size, self.cfg.scheduler.ctx_size + 8)
        self.broker = broker or PhysicalResourceBroker()
        self.broker.set_limit(ResourceKind.KV_PAGES, self.cfg.kv_pages)
        self.registry = registry
        self.detokenize = detokenize
        self.stats = EngineStats()
        self._next_txn = 0
        self._ending: Deque[Transaction] = deque()
        self._waiting: Dict[int, Transaction] = {}
        self._outbox: Deque[object] = deque()
        self._retired: KvRetirement = KvRetirement()
        self._sessions: Dict[str, SequenceState] = {}
        self._session_busy: set = set()                  # session ids with a request in flight
        self._frame_backoff = False                      # set by a frame deadlock, cleared when nothing is parked
        self._snapshots: Dict[str, Tuple[object, list]] = {}
        self._shutdown = False
        # prefix cache: chained block hash -> (kv sequence, tokens); entries in insertion / last-use order
        self._prefix_index: Dict[bytes, Tuple[int, int]] = {}
        self._prefix_lru: "OrderedDict[int, Tuple[List[int], List[bytes]]]" = OrderedDict()
        self._prefix_tokens = 0
        self._prefix_hot: set = set()       # entries that have been forked at least once: they outlive the others
        if self.cfg.prefix_cache_tokens and self.cfg.prefix_block % self.cfg.page_size:
            raise ValueError("prefix_block must be a multiple of the page size")
        self.spec = None
        if self.cfg.speculative:
            from .speculation import SpeculativeDecoder
            self.spec = SpeculativeDecoder(self)
        self._executing: Optional[Transaction] = None
        hook = getattr(self.runner, "set_decode_predictor", None)
        if hook is not None:
            hook(self._predict_next_decode)

    # ------------------------------------------------------------------ public API
    def submit(self, req: GenerateRequest) -> SequenceState:
        if self._shutdown:
            raise RuntimeError("engine is shut down")
        if req.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be >= 0")
        if req.session_id and req.session_id in self._session_busy:
            # a second request would start from nothing and overwrite the first one's retained state when it ends
            raise ValueError(f"session {req.session_id!r} has a request in flight")
        prev = self._sessions.get(req.session_id) if req.session_id else None
        now = time.perf_counter_ns()
        # validate before anything is taken: a rejected continuation leaves its retained session intact
        total = (len(prev.tokens) if prev is not None else 0) + len(req.prompt_tokens)
        if prev is None and not req.prompt_tokens:
            raise ValueError("empty prompt")
        if total + 1 > self.cfg.scheduler.ctx_size:
            raise ValueError("prompt does not fit the context window")
        if prev is not None:
            committed = self.kv.sequence(prev.kv_seq).committed_tokens
            if committed != prev.position:
                raise RuntimeError(f"retained session {req.session_id!r}: KV holds {committed} tokens, "
                                   f"sequence position is {prev.position}")
            del self._sessions[req.session_id]
            seq = SequenceState(req, kv_seq=prev.kv_seq, tokens=prev.tokens + list(req.prompt_tokens),
                                position=prev.position, arrival_ns=now, held_slot=prev.held_slot)
            prev.held_slot = -1
        else:
            hit = (self._prefix_lookup(req.prompt_tokens)
                   if (self.cfg.prefix_cache_tokens and not req.session_id
                       and getattr(self.runner, "supports_prefix_sharing", True)) else None)
            if hit is not None:
                donor, n = hit
                seq = SequenceState(req, kv_seq=self.kv.publish_fork_sequence_prefix(donor, n),
                                    tokens=list(req.prompt_tokens), position=n, arrival_ns=now)
                self.stats.prefix_hits += 1
                self.stats.prefix_tokens_reused += n
            else:
                seq = SequenceState(req, kv_seq=self.kv.alloc_sequence(), tokens=list(req.prompt_tokens),
                                    arrival_ns=now)
        seq.prompt_len = len(seq.tokens)
        try:
            self.scheduler.submit(seq)
        except Exception:
            if prev is not None:
                prev.held_slot, seq.held_slot = seq.held_slot, -1
                self._sessions[req.session_id] = prev
            else:
                self._retire(self.kv.free_sequence_pages(seq.kv_seq))
            raise
        if req.session_id:
            self._session_busy.add(req.session_id)
        return seq

    # ------------------------------------------------------------------ prompt-prefix cache
    def _prefix_keys(self, tokens: Sequence[int], blocks: int) -> List[bytes]:
        """Chained digests of the first `blocks` prefix blocks: key k covers tokens[: (k + 1) * prefix_block]."""
        import hashlib
        from array import array
        B = self.cfg.prefix_block
        keys, prev = [], b""
        for k in range(blocks):
            prev = hashlib.blake2b(prev + array("q", tokens[k * B:(k + 1) * B]).tobytes(), digest_size=16).digest()
            keys.append(prev)
        return keys

    def _prefix_lookup(self, prompt: Sequence[int]) -> Optional[Tuple[int, int]]:
        """-> (kv sequence to fork, tokens to share) for the longest cached prefix that leaves the request at
        least one prompt token of its own to run."""
        B = self.cfg.prefix_block
        blocks = (len(prompt) - 1) // B
        if blocks <= 0 or not self._prefix_index:
            return None
        keys = self._prefix_keys(prompt, blocks)
        for k in range(blocks - 1, -1, -1):
            ent = self._prefix_index.get(keys[k])
            if ent is None:
                continue
            donor, n = ent
            cached = self._prefix_lru.get(donor)
            if cached is None or cached[0][:n] != list(prompt[:n]):
                continue                                    # digest collision: not the same tokens
            self._prefix_lru.move_to_end(donor)
            self._prefix_hot.add(donor)
            return donor, n
        return None

    def _prefix_offer(self, seq: SequenceState) -> bool:
        """A finishing sequence leaves its prompt's whole prefix blocks to the cache (True: the cache now owns
        the KV sequence) unless every one of them is cached already."""
        B = self.cfg.prefix_block
        have = self.kv.sequence(seq.kv_seq).committed_tokens
        n = min(seq.prompt_len, have, self.cfg.prefix_cache_tokens) // B * B
        if n < B:
            return False
        keys = self._prefix_keys(seq.tokens, n // B)
        new = [k for k in keys if k not in self._prefix_index]
        if not new:
            donor = self._prefix_index[keys[-1]][0]
            if donor in self._prefix_lru:
                self._prefix_lru.move_to_end(donor)
            return False
        self._retire(self.kv.truncate_sequence(seq.kv_seq, n))
        for i, k in enumerate(keys):
            if k not in self._prefix_index:
                self._prefix_index[k] = (seq.kv_seq, (i + 1) * B)
        self._prefix_lru[seq.kv_seq] = (list(seq.tokens[:n]), new)
        self._prefix_tokens += n
        self.stats.prefix_entries += 1
        while self._prefix_tokens > self.cfg.prefix_cache_tokens and len(self._prefix_lru) > 1:
            self._prefix_evict()
        return True

    def _prefix_evict(self) -> bool:
        """Drop a cache entry - the oldest that no request ever reused, else the least recently used; its pages go
        back once no fork shares them."""
        if not self._prefix_lru:
            return False
        victim = next((k for k in self._prefix_lru if k not in self._prefix_hot), None)
        if victim is None:
            victim = next(iter(self._prefix_lru))
        kv_seq, (tokens, keys) = victim, self._prefix_lru.pop(victim)
        self._prefix_hot.discard(kv_seq)
        for k in keys:
            if self._prefix_index.get(k, (None, 0))[0] == kv_seq:
                del self._prefix_index[k]
        self._prefix_tokens -= len(tokens)
        self._retire(self.kv.free_sequence_pages(kv_seq))
        self.stats.prefix_evictions += 1
        return True

    def cancel_request(self, request_id: str) -> bool:
        seq = self.scheduler.cancel(request_id)
        if seq is None:
            return False
        if seq.status == SeqStatus.FINISHED:       # was still waiting: nothing else to release
            self._release_sequence(seq, FinishReason.CANCELLED)
        return True

    def has_work(self) -> bool:
        return bool(self.scheduler.has_work() or self._ending or self._waiting or self._outbox
                    or self._retired or (self.cfg.auto_preempt and self.scheduler.suspended))

    def fork_session_exact(self, request_id: str, new_req: GenerateRequest) -> SequenceState:
        """New request that continues from an exact copy of a live sequence's committed state.
        Pages are shared by refcount; the partially filled tail page is copied on first write."""
        if not getattr(self.runner, "supports_prefix_sharing", True):
            raise ValueError("this runner binds sequence state to a slot: a sequence cannot be forked by sharing pages")
        src = self.scheduler.active.get(request_id) or self._sessions.get(request_id)
        if src is None:
            raise KeyError(request_id)
        if src.status == SeqStatus.RUNNING:
            raise RuntimeError("cannot fork a sequence inside a transaction")
        child_kv = self.kv.publish_fork_sequence_exact(src.kv_seq)
        committed = src.tokens[:src.position]
        seq = SequenceState(new_req, kv_seq=child_kv, tokens=committed + list(new_req.prompt_tokens),
                            position=src.position, arrival_ns=time.perf_counter_ns())
        seq.prompt_len = len(seq.tokens)
        if seq.prefill_remaining == 0:
            # nothing new to run: re-run the last committed token to obtain logits
            raise ValueError("a fork needs at least one new prompt token")
        self.scheduler.submit(seq)
        return seq

    def reset_session(self, session_id: str) -> bool:
        """Drop a retained session: its pages go back, the next request under this id starts from nothing.
        False when no session of that name is retained (a session inside a request is not retained yet)."""
        seq = self._sessions.pop(session_id, None)
        if seq is None:
            return False
        self._drop_session(seq)
        self._drive_retirements()
        return True

    def _evict_idle_session_for_slot(self) -> bool:
        """Every slot is taken and a new request waits for one: retained sessions of slot-bound runners hold slots
        while idle - the one retained longest gives its slot (and its cached state) up.  A waiting continuation of
        a session keeps its own slot and is not what this is about."""
        if self.scheduler.waiting[0].held_slot >= 0:
            return False
        for sid, seq in self._sessions.items():            # insertion order: oldest retained first
            if seq.held_slot >= 0:
                del self._sessions[sid]
                self._drop_session(seq)
                self.stats.session_evictions += 1
                return True
        return False

    def _evict_idle_session_for_pages(self) -> bool:
        """Nothing of this action could reserve its pages: idle retained sessions are caches of their conversations
        and come before any running request - the one retained longest that still holds pages is dropped."""
        for sid, seq in self._sessions.items():
            if seq.kv_seq >= 0 and self.kv.sequence(seq.kv_seq).pages:
                del self._sessions[sid]
                self._drop_session(seq)
                self.stats.session_evictions += 1
                return True
        return False

    def _drop_session(self, seq: SequenceState) -> None:
        if seq.kv_seq >= 0:
            self._retire(self.kv.free_sequence_pages(seq.kv_seq))
            seq.kv_seq = -1
        slot = self.scheduler.release_held(seq)
        if slot >= 0:
            self.runner.release_slot(slot)

    def preempt_session(self, request_id: str) -> None:
        seq = self.scheduler.active.get(request_id)
        if seq is None or seq.status == SeqStatus.RUNNING:
            raise RuntimeError("sequence not preemptible now")
        rec = self.kv.preempt_sequence(seq.kv_seq)
        pages = [p for _, p in rec.exclusive]
        snap = self.runner.snapshot_pages(pages) if pages else None
        self._snapshots[request_id] = (snap, pages)
        self._retire(self.kv.release_preempted_pages(seq.kv_seq))
        self.scheduler.suspend(seq)

    def restore_session(self, request_id: str) -> None:
        seq = self.scheduler.suspended.get(request_id)
        if seq is None:
            raise KeyError(request_id)
        self._drive_retirements()
        mapping = self.kv.restore_sequence(seq.kv_seq)          # may raise OutOfPages
        snap, old_pages = self._snapshots.pop(request_id)
        if mapping:
            self.runner.restore_pages([p for _, p in mapping], snap)
        self.scheduler.resume(seq)

    def shutdown(self) -> bool:
        """Non-blocking: returns True once nothing is in flight and all custody is returned."""
        self._shutdown = True
        for s in list(self.scheduler.waiting) + list(self.scheduler.active.values()):
            self.cancel_request(s.request_id)
        self.step(lambda ev: None)
        idle = not (self._ending or self._waiting)
        if idle:
            for s in list(self._sessions.values()):
                self._drop_session(s)
            self._sessions.clear()
            while self._prefix_evict():
                pass
            self._drive_retirements()
            self.runner.shutdown()
        return idle

    # ------------------------------------------------------------------ owner loop
    def step(self, emit: EmitFn) -> bool:
        t0 = time.perf_counter_ns()
        self.stats.steps += 1
        progressed = self._drive_endings()
        progressed |= self._drive_retirements()
        if self.scheduler.suspended and self.cfg.auto_preempt:
            progressed |= self.maybe_restore_suspended() > 0        # swapped-out sequences return when pages allow
        progressed |= self._flush_outbox(emit)
        if self.registry is not None:
            progressed |= bool(self.registry.drive())
            progressed |= self._resume_ready()
            if self._waiting:
                progressed |= self._break_frame_deadlock()
            if self._waiting and self.cfg.materialization_timeout_s > 0:
                progressed |= self._expire_parked()
        if self.scheduler.waiting and self.scheduler.slots.available == 0:
            progressed |= self._evict_idle_session_for_slot()
        if self._frame_backoff and not self._waiting:
            self._frame_backoff = False
        # after a frame deadlock nothing new starts while a transaction is parked: what was rolled back would lease
        # the same frames again and meet the survivor in the same place
        action = None if self._frame_backoff else self.scheduler.next_action()
        if action is not None:
            self.stats.actions += 1
            self._execute_action(action)
            progressed = True
        progressed |= self._flush_outbox(emit)
        self.stats.host_ns += time.perf_counter_ns() - t0
        return progressed

    def run_until_idle(self, emit: EmitFn, max_steps: int = 1_000_000) -> int:
        n = 0
        while self.has_work() and n < max_steps:
            if not self.step(emit) and not self.has_work():
                break
            n += 1
        return n

    # ------------------------------------------------------------------ actions
    def _execute_action(self, action) -> None:
        if isinstance(action, Cancel):
            self._finish(action.seq, FinishReason.CANCELLED)
            return
        if isinstance(action, Finish):
            self._finish(action.seq, action.reason)
            return
        if isinstance(action, PrefillChunk):
            prefills, decodes = [(action.seq, action.tokens)], []
        elif isinstance(action, DecodeBatch):
            prefills, decodes = [], action.seqs
        else:
            prefills, decodes = action.prefills, action.decodes
        if not prefills and self.spec is not None and self.runner.proposals_enabled():
            if self.spec.try_execute(decodes):
                return
        self._execute_ordinary(prefills, decodes)

    def _reserve(self, seq: SequenceState, n: int, members: List[TxnSeq], is_prefill: bool,
                 claimed: Dict[ResourceKind, int]) -> bool:
        budget = self._page_budget - claimed[ResourceKind.KV_PAGES]
        r, need = self.kv.try_reserve(seq.kv_seq, n, budget)
        if r is None:
            return False
        claimed[ResourceKind.KV_PAGES] += need
        members.append(TxnSeq(seq, r.res_id, n, is_prefill))
        return True

    def _execute_ordinary(self, prefills, decodes) -> None:
        self._drive_retirements()
        members: List[TxnSeq] = []
        claimed = {ResourceKind.KV_PAGES: 0}
        stalled: List[SequenceState] = []
        self._page_budget = self.broker.available(ResourceKind.KV_PAGES)     # constant while this batch is assembled
        for seq in decodes:
            if not self._reserve(seq, 1, members, False, claimed):
                stalled.append(seq)
        for seq, n in prefills:
            if not self._reserve(seq, n, members, True, claimed):
                stalled.append(seq)
        for seq in stalled:
            self.stats.kv_stalls += 1
            self.scheduler.requeue_unchanged(seq)
        if stalled and self._prefix_lru:
            self._prefix_evict()            # cached prefixes give way to running sequences, oldest first
        if not members:
            if stalled:
                self._break_page_deadlock(stalled)
            return
        grant = self.broker.try_claim(claimed, required=True)
        txn = Transaction(self._next_txn, members, grant=grant, t_start_ns=time.perf_counter_ns())
        self._next_txn += 1
        self.stats.transactions += 1
        try:
            txn.batch = self._lower(txn)
            self.runner.prepare_batch(txn.txn_id, txn.batch)
            if grant is not None:
                self.broker.mark_submitted(grant)
            t0 = time.perf_counter_ns()
            self._executing = txn
            progress = self.runner.execute(txn.txn_id)
            self.stats.runner_ns += time.perf_counter_ns() - t0
        except Exception as exc:  # noqa: BLE001 - every backend failure aborts the transaction
            self._executing = None
            self._abort(txn, exc)
            return
        self._executing = None
        self._on_progress(txn, progress)

    def _predict_next_decode(self, tokens_by_slot: Dict[int, int]) -> Optional[List[int]]:
        """Called by the runner from inside `execute` of a pure-decode transaction, with the token every
        sequence just produced: the state slots of the next decode batch in order, if the next action is
        certain to be a pure decode batch of exactly the sequences that continue.  Mirrors the commit and
        finish rules of `_publish` / `_post_commit_finish` / `_apply_output` without changing anything."""
        txn = self._executing
        sch = self.scheduler
        if (txn is None or self.spec is not None or self.registry is not None or self._shutdown
                or self._ending or self._waiting or sch.waiting or sch.prefill or sch.pending_cancel
                or sch.decode_ready or sch.suspended):
            return None
        ctx = self.cfg.scheduler.ctx_size
        eos = self.runner.eos_token_id
        out: List[int] = []
        for m in txn.members:
            seq = m.seq
            req = seq.request
            if m.is_prefill or seq.finish is not None or req.stop:
                return None
            tok = tokens_by_slot.get(seq.slot)
            if tok is None or tok < 0:
                return None
            if seq.generated + 1 >= req.max_new_tokens or seq.position + 1 >= ctx:
                continue
            if tok == eos and not req.ignore_eos:
                continue
            out.append(seq.slot)
        return out or None

    def _lower(self, txn: Transaction) -> ExecutionBatch:
        ps = self.cfg.page_size
        token_ids: List[int] = []
        positions: List[int] = []
        write_slots: List[int] = []
        logits: List[LogitsRequest] = []
        seqs: List[SequenceSlice] = []
        block_ids: List[int] = []
        none, top1 = LogitsRequest.none(), LogitsRequest.topk(1)
        skip_unread = bool(getattr(self.runner, "skip_unread_logits", False))
        for m in txn.members:
            seq = m.seq
            r, blocks, slots = self.kv.bind_and_bindings(m.res_id, txn.txn_id)
            m.query_start = len(token_ids)
            start = seq.position
            if m.is_prefill:
                toks = seq.tokens[start:start + m.rows]
                last_chunk = start + m.rows >= seq.prompt_len
                token_ids.extend(toks)
                logits.extend([none] * (m.rows - 1))
                logits.append(top1 if last_chunk else none)
            else:
                token_ids.append(seq.staged_token)
                # committing this token ends the request by its length: the logits after it would be discarded.
                # Runners that replay a captured step compute every row anyway and keep the uniform request.
                last = skip_unread and seq.generated + 1 >= seq.request.max_new_tokens
                logits.append(none if last else top1)
            positions.extend(range(start, start + m.rows))
            write_slots.extend(slots)
            seqs.append(SequenceSlice(seq.slot, Phase.PREFILL if m.is_prefill else Phase.DECODE, m.query_start,
                                      m.rows, start, start + m.rows, len(block_ids), len(blocks),
                                      (r.cow,) if r.cow is not None else ()))
            block_ids.extend(blocks)
        return ExecutionBatch(token_ids, positions, write_slots, logits, seqs, block_ids, Intent.COMMITTED, ps)

    # ------------------------------------------------------------------ progress / endings
    def _on_progress(self, txn: Transaction, progress) -> None:
        if isinstance(progress, Waiting):
            self.stats.waits += 1
            txn.state = TxnState.WAITING
            txn.t_parked_ns = time.perf_counter_ns()
            self._waiting[txn.txn_id] = txn
            if self.registry is None:
                self._abort(txn, RuntimeError("runner is waiting on materializations but no registry is attached"))
                self._waiting.pop(txn.txn_id, None)
                return
            try:
                self.registry.register_continuation(txn.txn_id, progress.dependencies)
            except Exception as exc:  # noqa: BLE001 - a dependency list the registry refuses fails the transaction
                self._waiting.pop(txn.txn_id, None)
                self._abort(txn, exc)
                return
            self._transaction_prefetch(txn, progress)
            return
        assert isinstance(progress, Complete)
        try:
            progress.output.validate(txn.batch)
        except Exception as exc:  # noqa: BLE001
            self._abort(txn, exc)
            return
        txn.output = progress.output
        if txn.speculative is not None:
            self.spec.on_verified(txn)
            return
        txn.commit_id = self.kv.prepare_commit([(m.res_id, m.rows) for m in txn.members])
        txn.state = TxnState.PUBLISHING
        self._end(txn)

    def _expire_parked(self) -> bool:
        from .io_protocol import FailureReason
        limit = time.perf_counter_ns() - int(self.cfg.materialization_timeout_s * 1e9)
        late = [t for t, txn in self._waiting.items() if txn.t_parked_ns < limit]
        for txn_id in late:
            self.stats.materialization_timeouts += 1
            self._abort(self._waiting.pop(txn_id), MaterializationFailed(FailureReason.PROVIDER_LOST))
        return bool(late)

    def _break_frame_deadlock(self) -> bool:
        """Parked transactions keep the payloads they already hold leased while they wait for more.  When the
        destination has no free frame left, the loads they wait for starve - and nobody will give a frame up by
        itself.  The oldest transaction waiting for a starving load keeps what it holds; every other one is rolled
        back (retryable: its sequences run again later), which returns their frames.  One transaction alone never
        needs more frames than exist (it takes its experts in waves), so the oldest then gets through."""
        starving = getattr(self.registry.provider, "starving", None)
        ops = starving(2) if starving is not None else []
        if not ops:
            return False
        waiters = sorted({t for op in ops for t in getattr(self.registry.ops.get(op), "waiters", ()) if t in self._waiting})
        parked = sorted(self._waiting)
        if not waiters or len(parked) < 2:
            return False
        from .io_protocol import FailureReason
        keep = waiters[0]
        for txn_id in parked:
            if txn_id != keep:
                txn = self._waiting.pop(txn_id)
                self.stats.frame_deadlocks += 1
                self._abort(txn, MaterializationFailed(FailureReason.RESOURCE_EXHAUSTED))
        # the starving load takes a freed frame now; the rolled-back sequences wait until the survivor is through
        self.registry.drive()
        self._frame_backoff = True
        return True

    def _transaction_prefetch(self, txn: Transaction, progress) -> None:
        """While the transaction waits for what it must have, ask for what it will probably want next: no waiter,
        no lease, prefetch band (behind every required load).  The requests belong to the transaction and are
        detached when it ends, whatever became of them."""
        n = self.cfg.transaction_prefetch
        want = getattr(self.runner, "prefetch_candidates", None)
        if n <= 0 or want is None:
            return
        from .registry import OwnerKind
        have = set(progress.dependencies.keys if hasattr(progress.dependencies, "keys") else progress.dependencies)
        keys = [k for k in want(getattr(progress, "layer", 0), n) if k not in have][:n]
        owner = (OwnerKind.TRANSACTION_PREFETCH, txn.txn_id)
        for k in keys:
            op = self.registry.request(k, owner)
            if op not in txn.prefetch_ops:
                txn.prefetch_ops.append(op)
                self.stats.prefetch_requests += 1

    def _release_registry(self, txn: Transaction) -> None:
        """The transaction reached its end: its custody and its prefetch ownership go back to the registry."""
        if self.registry is None:
            return
        self.registry.release_transaction(txn.txn_id)
        if txn.prefetch_ops:
            from .registry import OwnerKind
            owner = (OwnerKind.TRANSACTION_PREFETCH, txn.txn_id)
            for op in txn.prefetch_ops:
                o = self.registry.ops.get(op)
                if o is not None and owner in o.owners:
                    self.registry.detach(op, owner)
            txn.prefetch_ops.clear()

    def _resume_ready(self) -> bool:
        did = False
        for txn_id in self.registry.pop_failed():
            txn = self._waiting.pop(txn_id, None)
            if txn is not None:
                did = True
                self._abort(txn, MaterializationFailed(self.registry.failure_of(txn_id)))
        for txn_id in self.registry.pop_ready():
            txn = self._waiting.pop(txn_id, None)
            if txn is None:
                continue
            self.stats.resumes += 1
            did = True
            try:
                t0 = time.perf_counter_ns()
                progress = self.runner.resume(txn_id)
                self.stats.runner_ns += time.perf_counter_ns() - t0
            except Exception as exc:  # noqa: BLE001
                self._abort(txn, exc)
                continue
            txn.state = TxnState.EXECUTING
            self._on_progress(txn, progress)
        return did

    def _end(self, txn: Transaction) -> None:
        """Ask the backend to end the transaction; publish or roll back once it is COMPLETE."""
        if txn.state == TxnState.DONE:
            if txn in self._ending:
                self._ending.remove(txn)
            return
        intent = EndIntent.PUBLISH if txn.state == TxnState.PUBLISHING else EndIntent.ABORT
        try:
            status = self.runner.end_transaction(txn.txn_id, intent)
        except Exception as exc:  # noqa: BLE001
            if intent == EndIntent.PUBLISH:
                txn.error = exc
                self.last_error = exc
                self.stats.aborted_transactions += 1
                if txn.commit_id is not None:
                    self.kv.abort_prepared_commit(txn.commit_id)
                    txn.commit_id = None
                txn.state = TxnState.ABORTING
                if txn not in self._ending:      # it may be here already (an ending that was pending before)
                    self._ending.append(txn)
                return
            status = EndStatus.COMPLETE       # an abort that fails has nothing more to undo
        if status == EndStatus.PENDING:
            if txn not in self._ending:
                self._ending.append(txn)
            return
        if txn in self._ending:
            self._ending.remove(txn)
        if txn.state == TxnState.PUBLISHING:
            self._publish(txn)
        else:
            self._rollback(txn)

    def _drive_endings(self) -> bool:
        if not self._ending:
            return False
        for txn in list(self._ending):
            self._end(txn)
        return True

    def _abort(self, txn: Transaction, exc: BaseException) -> None:
        self.stats.aborted_transactions += 1
        txn.error = exc
        self.last_error = exc            # for callers that want to report why requests ended in ERROR
        if txn.commit_id is not None:
            self.kv.abort_prepared_commit(txn.commit_id)
            txn.commit_id = None
        txn.state = TxnState.ABORTING
        self._end(txn)

    def _rollback(self, txn: Transaction) -> None:
        """Backend is done with the aborted transaction: now ownership may be returned."""
        self._retire(self.kv.abort_reservations([m.res_id for m in txn.members]))
        if txn.grant is not None:
            self.broker.complete(txn.grant)
        self._release_registry(txn)
        txn.state = TxnState.DONE
        for m in txn.members:
            seq = m.seq
            if seq.finish == FinishReason.CANCELLED:
                self._finish(seq, FinishReason.CANCELLED)
            elif txn.error is not None and not getattr(txn.error, "retryable", False):
                self._finish(seq, FinishReason.ERROR)
            else:
                self.scheduler.requeue_unchanged(seq)

    # ------------------------------------------------------------------ publish
    def _publish(self, txn: Transaction) -> None:
        """Backend confirmed the publish: commit KV, scheduler, tokens; stage the next greedy tokens."""
        self._release_registry(txn)
        if txn.speculative is not None:
            self.spec.publish(txn)
            return
        ret = self.kv.publish_commit(txn.commit_id)
        txn.commit_id = None
        self._retire(ret)
        if txn.grant is not None:
            self.broker.complete(txn.grant)      # pages are now accounted by the page manager itself
        txn.state = TxnState.DONE
        out = txn.output.by_row()
        now = time.perf_counter_ns()
        n_prefill = n_decode = 0
        for m in txn.members:
            seq = m.seq
            if m.is_prefill:
                n_prefill += m.rows
                self.scheduler.commit_prefill(seq, m.rows)
                last_row = m.query_start + m.rows - 1
            else:
                n_decode += 1
                tok = seq.staged_token
                self.scheduler.commit_decode(seq, tok)
                self._emit_token(seq, tok, now)
                last_row = m.query_start
            if seq.finish == FinishReason.CANCELLED:
                self._finish(seq, FinishReason.CANCELLED)
                continue
            if not m.is_prefill and self._post_commit_finish(seq):
                continue                             # its fresh logits are discarded
            ro = out.get(last_row)
            if ro is not None:
                self._apply_output(seq, ro.top1)
        if n_prefill:
            self.stats.prefill_chunks += sum(1 for m in txn.members if m.is_prefill)
            self.stats.prefill_tokens += n_prefill
        if n_decode:
            self.stats.decode_steps += 1
            self.stats.decode_rows += n_decode

    def _post_commit_finish(self, seq: SequenceState) -> bool:
        req = seq.request
        if seq.generated >= req.max_new_tokens:
            self._finish(seq, FinishReason.MAX_TOKENS)
            return True
        if req.stop and seq.text:
            for s in req.stop:
                if s and seq.text.endswith(s):
                    self._finish(seq, FinishReason.STOP_STRING)
                    return True
        return False

    def _apply_output(self, seq: SequenceState, top1: Optional[int]) -> None:
        """Post-forward finish rules, in order, else stage the greedy token."""
        req = seq.request
        if seq.generated >= req.max_new_tokens:
            self._finish(seq, FinishReason.MAX_TOKENS)
        elif seq.position >= self.cfg.scheduler.ctx_size:
            self._finish(seq, FinishReason.CONTEXT)
        elif top1 is None or top1 < 0:
            self._finish(seq, FinishReason.NO_CANDIDATE)
        elif top1 == self.runner.eos_token_id and not req.ignore_eos:
            self._finish(seq, FinishReason.EOS)
        else:
            self.scheduler.stage(seq, top1)
            self.stats.staged_tokens += 1

    def _emit_token(self, seq: SequenceState, tok: int, now_ns: int) -> None:
        delta = ""
        if self.detokenize is not None:
            # incremental: a few token decodes per token however long the output is (an incomplete UTF-8 tail is
            # held back until it completes)
            dec = seq.decoder
            if dec is None:
                from ..utils.tokenizer import IncrementalDecodeState
                dec = seq.decoder = IncrementalDecodeState(decode=self.detokenize)
            delta = dec.push(tok)
            seq.text = seq.text + delta
        if seq.first_token_ns == 0:
            seq.first_token_ns = now_ns
        seq.last_token_ns = now_ns
        self._outbox.append(TokenEvent(seq.request_id, tok, delta, seq.generated - 1))
        self.stats.emitted_tokens += 1

    def _finish(self, seq: SequenceState, reason: FinishReason) -> None:
        if seq.status == SeqStatus.FINISHED and seq.slot < 0 and seq.kv_seq < 0:
            return
        # a suspended (preempted) sequence that ends never comes back: drop its host snapshot
        self.scheduler.suspended.pop(seq.request_id, None)
        self._snapshots.pop(seq.request_id, None)
        slot = seq.slot                                   # the scheduler returns the slot to its pool and clears it
        # a runner whose sequence state lives in the slot (no page sharing): a retained session keeps its slot
        keep_slot = (self._keeps_session(seq, reason) and slot >= 0
                     and not getattr(self.runner, "supports_prefix_sharing", True))
        self.scheduler.finish(seq, reason, keep_slot=keep_slot)
        self._release_sequence(seq, reason, -1 if keep_slot else slot)

    @staticmethod
    def _keeps_session(seq: SequenceState, reason: FinishReason) -> bool:
        return bool(seq.request.retain_session and reason not in (FinishReason.CANCELLED, FinishReason.ERROR))

    def _release_sequence(self, seq: SequenceState, reason: FinishReason, slot: int = -1) -> None:
        seq.staged_token = None
        slot = seq.slot if seq.slot >= 0 else slot
        ttft = (seq.first_token_ns - seq.arrival_ns) / 1e9 if seq.first_token_ns else 0.0
        tpot = ((seq.last_token_ns - seq.first_token_ns) / 1e9 / (seq.generated - 1)) if seq.generated > 1 else 0.0
        keep = self._keeps_session(seq, reason)
        if seq.request.session_id:
            self._session_busy.discard(seq.request.session_id)
        if keep:
            # the session keeps its committed KV; uncommitted staged state is dropped
            seq.tokens = seq.tokens[:seq.position]
            self._sessions[seq.request.session_id or seq.request_id] = seq
        elif seq.kv_seq >= 0:
            cache = (self.cfg.prefix_cache_tokens and not self._shutdown
                     and getattr(self.runner, "supports_prefix_sharing", True)
                     and reason not in (FinishReason.CANCELLED, FinishReason.ERROR))
            if not (cache and self._prefix_offer(seq)):
                self._retire(self.kv.free_sequence_pages(seq.kv_seq))
            seq.kv_seq = -1
        if slot >= 0:
            self.runner.release_slot(slot)                # slot-bound runner state (if any) is dropped with it
        self.stats.finished += 1
        self.stats.ttft_sum_s += ttft
        self.stats.tpot_sum_s += tpot
        self.stats.e2e_sum_s += (time.perf_counter_ns() - seq.arrival_ns) / 1e9
        tail = ""
        if seq.decoder is not None:
            tail = seq.decoder.finish()
            seq.text = seq.text + tail
        self._outbox.append(FinishEvent(seq.request_id, reason, seq.prompt_len, seq.generated, seq.text, ttft, tpot,
                                        tail))

    def _flush_outbox(self, emit: EmitFn) -> bool:
        if not self._outbox:
            return False
        while self._outbox:
            # the event leaves the outbox only after the consumer took it: a consumer that raises gets the same
            # committed event again on the next step, and nothing of the engine's own state depends on delivery
            emit(self._outbox[0])
            self._outbox.popleft()
        return True

    # ------------------------------------------------------------------ page retirement
    def _retire(self, ret: KvRetirement) -> None:
        if ret:
            self._retired.extend(ret)

    def _drive_retirements(self) -> bool:
        """Hand retired pages to the backend; once it returns they are reusable."""
        if not self._retired:
            return False
        pages = self._retired.pages
        self._retired = KvRetirement()
        self.runner.release_pages(pages)
        self.kv.confirm_page_retirement(pages)
        return True

    def _break_page_deadlock(self, stalled: List[SequenceState]) -> None:
        """No sequence of this action could reserve its pages.  Pages may still be on their way back (endings,
        parked transactions, retirements, cached prefixes): then the next step tries again.  Idle retained
        sessions are dropped next, oldest first (they are caches of their conversations).  Otherwise nobody
        will ever free a page by itself: with `auto_preempt` the youngest sequence is swapped out (an idle one if
        there is one, else one of the stalled ones - the others then fit); without it, or when a single sequence
        cannot fit the pool on its own, the youngest stalled request ends with an error instead of spinning."""
        if self._ending or self._waiting or self._retired:
            return
        if self._prefix_lru:
            self._prefix_evict()            # cached prefixes go first (the speculative path stalls through here too)
            return
        if self._evict_idle_session_for_pages():
            return                          # an idle retained session gave its pages up: the next step tries again
        if self.cfg.auto_preempt:
            idle = [s for s in self.scheduler.decode_ready if s not in stalled]
            holders = [s for s in idle if self.kv.sequence(s.kv_seq).pages]
            cands = holders or ([s for s in stalled if self.kv.sequence(s.kv_seq).pages]
                                if len(self.scheduler.active) > 1 else [])
            if cands:
                victim = max(cands, key=lambda s: s.arrival_ns)
                self.preempt_session(victim.request_id)
                self.stats.auto_preemptions += 1
                return
        if self.kv.stats().quarantined_pages:
            return
        victim = max(stalled, key=lambda s: s.arrival_ns)
        self.last_error = OutOfPages(f"request {victim.request_id}: the KV pool cannot hold its next tokens")
        self.stats.page_deadlocks += 1
        self._finish(victim, FinishReason.ERROR)

    def maybe_restore_suspended(self) -> int:
        """Bring suspended sequences back while pages allow (oldest first).  A sequence returns only if, after its
        own pages, one page of headroom per running sequence remains: restoring into a pool that the running
        sequences are about to outgrow would only get it swapped out again."""
        n = 0
        self._drive_retirements()
        for rid, seq in sorted(self.scheduler.suspended.items(), key=lambda kv: kv[1].arrival_ns):
            need = sum(1 for p in self.kv.sequence(seq.kv_seq).pages if p < 0) + 1
            if self.kv.free_pages < need + len(self.scheduler.active):
                break
            try:
                self.restore_session(rid)
                n += 1
            except OutOfPages:
                break
        return n

    def snapshot_stats(self) -> Dict[str, object]:
        st = dict(vars(self.stats))
        st["kv"] = dict(vars(self.kv.stats()))
        st["scheduler"] = dict(vars(self.scheduler.stats))
        st["resources"] = self.broker.snapshot()
        if self.spec is not None:
            st["speculative"] = self.spec.metrics.to_dict()
        return st
