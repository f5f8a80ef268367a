"""Runner contract between the engine and a model backend, plus a deterministic mock.

A transaction is: `prepare_batch` (physical page work: zeroing, copy-on-write copies) ->
`execute` -> zero or more `resume` calls while it reports `Waiting` on materializations ->
`end_transaction(PUBLISH | ABORT)` repeated until it returns `COMPLETE`.  The engine keeps
every page, slot and credit of the transaction until that `COMPLETE`.

Counterpart of crates/ferrule-model/src/runner.rs:72-96 (ModelRunner), :221-236 (terminal
protocol), :249-468 (MultiSessionRunner), :556-592 (ResidentModelRunner).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from .execution import (ExecutionBatch, ExecutionCapabilities, ExecutionOutput, Intent, KvLayoutSchema,
                        KvPlaneDescriptor, RowOutput, SequenceSlice)


class EndIntent(Enum):
    PUBLISH = "publish"
    ABORT = "abort"


class EndStatus(Enum):
    PENDING = "pending"
    COMPLETE = "complete"


@dataclass
class Complete:
    output: ExecutionOutput


@dataclass
class Waiting:
    """The batch stopped at a layer that needs resources which are not resident yet."""
    dependencies: List[object]          # MaterializationKey list
    layer: int = -1


Progress = object  # Complete | Waiting


@dataclass
class Proposal:
    """Draft tokens for one sequence with the head's confidence logit per draft."""
    tokens: List[int]
    confidence: List[float]


class ModelRunner:
    """Interface; concrete runners override everything below."""

    # True: the engine asks for no logits on a decode row whose token ends its request by length (nobody would
    # read them).  Runners whose decode step is a captured graph compute every row in any case and leave it False,
    # so that every decode batch keeps the one shape their graph and their look-ahead were built for.
    skip_unread_logits = False

    vocab_size: int = 0
    eos_token_id: int = -1

    def capabilities(self) -> ExecutionCapabilities:
        return ExecutionCapabilities()

    def kv_schema(self) -> KvLayoutSchema:
        raise NotImplementedError

    def prepare_batch(self, txn_id: int, batch: ExecutionBatch) -> None:
        raise NotImplementedError

    def execute(self, txn_id: int) -> Progress:
        raise NotImplementedError

    def resume(self, txn_id: int) -> Progress:
        raise NotImplementedError

    def end_transaction(self, txn_id: int, intent: EndIntent) -> EndStatus:
        raise NotImplementedError

    def retain_provisional_prefixes(self, txn_id: int, rows_by_slot: Dict[int, int]) -> None:
        """Speculative verification: keep only the first `rows` provisional rows of each sequence."""

    def release_pages(self, pages: Sequence[int]) -> None:
        """The runtime retired these physical pages; return once the backend cannot touch them."""

    def snapshot_pages(self, pages: Sequence[int]):
        raise NotImplementedError

    def restore_pages(self, pages: Sequence[int], snapshot) -> None:
        raise NotImplementedError

    def release_slot(self, state_slot: int) -> None:
        """Drop per-sequence backend state (hidden taps etc.)."""

    # speculation
    def proposals_enabled(self) -> bool:
        return False

    def propose(self, slots: Sequence[int], anchors: Sequence[int], positions: Sequence[int],
                views: Sequence[object], max_draft: int) -> List[Proposal]:
        return [Proposal([], []) for _ in slots]

    def observability(self) -> Dict[str, object]:
        return {}

    def shutdown(self) -> None:
        pass

    # decode look-ahead
    def set_decode_predictor(self, fn: Optional[Callable[[Dict[int, int]], Optional[List[int]]]]) -> None:
        """The engine's answer to "which sequences decode next?": `fn({state slot: token just produced})`
        returns the state slots of the next pure-decode batch in order, or None when the next action is
        not (known to be) a pure decode batch.  A runner may use it to launch the next step on the device,
        fed by the tokens still on the device, before the host has published the current one."""
        self._predict_next_decode = fn


def predict_next_decode_batch(b: ExecutionBatch, tokens: Sequence[int], next_slots: Sequence[int]
                              ) -> Optional[ExecutionBatch]:
    """The batch the engine will lower for the step after pure-decode batch `b`, given the tokens `b`
    produced (row order) - or None when it cannot be told from `b` alone: a sequence ends, the order
    changes, or a sequence's next position has no page yet (the engine must reserve one first)."""
    seqs = b.sequences
    if len(next_slots) != len(seqs) or any(s.state_slot != ns for s, ns in zip(seqs, next_slots)):
        return None
    ps = b.page_size
    positions, slots, new_seqs = [], [], []
    for s in seqs:
        if s.query_len != 1:
            return None
        pos = b.positions[s.query_start] + 1
        blk = pos // ps
        if blk >= s.block_len:
            return None
        positions.append(pos)
        slots.append(b.block_ids[s.block_start + blk] * ps + pos % ps)
        new_seqs.append(SequenceSlice(s.state_slot, s.phase, s.query_start, 1, s.context_len + 1,
                                      s.sequence_len + 1, s.block_start, s.block_len, ()))
    return ExecutionBatch(list(tokens), positions, slots, list(b.logits), new_seqs, b.block_ids, b.intent, ps)


def same_decode_batch(a: ExecutionBatch, b: ExecutionBatch) -> bool:
    """True when two pure-decode batches make the device do exactly the same work."""
    return (a.token_ids == b.token_ids and a.positions == b.positions and a.write_slots == b.write_slots
            and a.block_ids == b.block_ids and a.intent == b.intent and len(a.sequences) == len(b.sequences)
            and all(x.state_slot == y.state_slot and x.block_start == y.block_start and x.block_len == y.block_len
                    and not x.cow and not y.cow for x, y in zip(a.sequences, b.sequences))
            and all(x.kind == y.kind and x.k == y.k for x, y in zip(a.logits, b.logits)))


class MockRunner(ModelRunner):
    """Deterministic CPU runner for state-machine tests.

    next token = (7 * token + 3 * position + 1) % vocab unless `next_token_fn` is given.
    Scripts: `fail_next_execute`, `fail_next_end` (end_transaction raises), `wait_next` (returns Waiting once),
    `pending_ends` (number of PENDING answers before an end completes), `no_candidate_rows`.
    """

    def __init__(self, vocab: int = 1000, eos: int = -1, page_size: int = 16,
                 next_token_fn: Optional[Callable[[int, int], int]] = None, draft_len: int = 0,
                 draft_accuracy: Optional[Callable[[int, int, int], int]] = None, skip_unread_logits: bool = False):
        self.vocab_size, self.eos_token_id, self.page_size = vocab, eos, page_size
        self.skip_unread_logits = skip_unread_logits
        self.next_token_fn = next_token_fn or (lambda tok, pos: (7 * tok + 3 * pos + 1) % vocab)
        self.txns: Dict[int, ExecutionBatch] = {}
        self.kv: Dict[int, Tuple[int, int]] = {}           # pool row -> (token, position)
        self.provisional: Dict[int, List[int]] = {}        # txn -> rows written provisionally
        self.fail_next_execute = 0
        self.fail_next_end = 0
        self.wait_next: List[List[object]] = []
        self.pending_ends = 0
        self.no_candidate_rows: set = set()
        self.calls: List[Tuple[str, int]] = []
        self.released_pages: List[int] = []
        self.draft_len = draft_len
        self.draft_fn = draft_accuracy
        self._pending_left: Dict[int, int] = {}
        self.copied_pages: List[Tuple[int, int]] = []
        # decode look-ahead bookkeeping: what the engine's predictor promised against what it then lowered
        self._predict_next_decode = None
        self.predicted: Optional[ExecutionBatch] = None
        self.prediction_hits = 0
        self.prediction_misses = 0

    def kv_schema(self) -> KvLayoutSchema:
        return KvLayoutSchema((KvPlaneDescriptor("latent_kv", 8, 1),), self.page_size, 1 << 20)

    def prepare_batch(self, txn_id: int, batch: ExecutionBatch) -> None:
        batch.validate(self.capabilities())
        self.calls.append(("prepare", txn_id))
        ps = batch.page_size
        for s in batch.sequences:
            for c in s.cow:
                self.copied_pages.append((c.source, c.replacement))
                for off in range(ps):
                    src = c.source * ps + off
                    if src in self.kv:
                        self.kv[c.replacement * ps + off] = self.kv[src]
        self.txns[txn_id] = batch

    def _run(self, txn_id: int) -> Progress:
        b = self.txns[txn_id]
        rows = []
        written = []
        for r in range(b.rows):
            self.kv[b.write_slots[r]] = (b.token_ids[r], b.positions[r])
            written.append(b.write_slots[r])
        if b.intent == Intent.PROVISIONAL_VERIFICATION:
            self.provisional[txn_id] = written
        for s in b.sequences:
            blocks = b.block_ids[s.block_start:s.block_start + s.block_len]
            # context check: every earlier position must be present in the bound pages
            for pos in range(s.context_len):
                slot = blocks[pos // b.page_size] * b.page_size + pos % b.page_size
                if slot not in self.kv or self.kv[slot][1] != pos:
                    raise RuntimeError(f"mock runner: context row {pos} of slot {s.state_slot} missing")
        for r in b.logit_rows():
            if r in self.no_candidate_rows:
                rows.append(RowOutput(r, [], []))
                continue
            k = max(b.logits[r].k, 1)
            t = self.next_token_fn(b.token_ids[r], b.positions[r])
            ids = [(t + j) % self.vocab_size for j in range(k)]
            rows.append(RowOutput(r, ids, [10.0 - j for j in range(k)]))
        return Complete(ExecutionOutput(rows))

    def execute(self, txn_id: int) -> Progress:
        self.calls.append(("execute", txn_id))
        b = self.txns.get(txn_id)
        if self.predicted is not None and b is not None:
            if same_decode_batch(self.predicted, b):
                self.prediction_hits += 1
            else:
                self.prediction_misses += 1
            self.predicted = None
        if self.fail_next_execute > 0:
            self.fail_next_execute -= 1
            raise RuntimeError("mock runner: scripted execute failure")
        if self.wait_next:
            return Waiting(self.wait_next.pop(0), layer=0)
        out = self._run(txn_id)
        if (self._predict_next_decode is not None and b.intent == Intent.COMMITTED and len(b.sequences) == b.rows
                and all(r.token_ids for r in out.output.rows) and len(out.output.rows) == b.rows):
            toks = [r.token_ids[0] for r in out.output.rows]
            nxt = self._predict_next_decode({s.state_slot: toks[i] for i, s in enumerate(b.sequences)})
            if nxt:
                self.predicted = predict_next_decode_batch(b, toks, nxt)
        return out

    def resume(self, txn_id: int) -> Progress:
        self.calls.append(("resume", txn_id))
        if self.wait_next:
            return Waiting(self.wait_next.pop(0), layer=0)
        return self._run(txn_id)

    def end_transaction(self, txn_id: int, intent: EndIntent) -> EndStatus:
        self.calls.append((f"end_{intent.value}", txn_id))
        if self.fail_next_end > 0:
            self.fail_next_end -= 1
            raise RuntimeError("mock runner: scripted end failure")
        left = self._pending_left.setdefault(txn_id, self.pending_ends)
        if left > 0:
            self._pending_left[txn_id] = left - 1
            return EndStatus.PENDING
        self._pending_left.pop(txn_id, None)
        b = self.txns.pop(txn_id, None)
        if intent == EndIntent.ABORT and b is not None:
            for slot in b.write_slots:
                self.kv.pop(slot, None)
        self.provisional.pop(txn_id, None)
        return EndStatus.COMPLETE

    def retain_provisional_prefixes(self, txn_id: int, rows_by_slot: Dict[int, int]) -> None:
        b = self.txns[txn_id]
        for s in b.sequences:
            keep = rows_by_slot.get(s.state_slot, 0)
            for j in range(keep, s.query_len):
                self.kv.pop(b.write_slots[s.query_start + j], None)

    def release_pages(self, pages: Sequence[int]) -> None:
        self.released_pages.extend(pages)
        for p in pages:
            for off in range(self.page_size):
                self.kv.pop(p * self.page_size + off, None)

    def snapshot_pages(self, pages: Sequence[int]):
        return {p: {off: self.kv.get(p * self.page_size + off) for off in range(self.page_size)} for p in pages}

    def restore_pages(self, pages: Sequence[int], snapshot) -> None:
        for new, (old, rows) in zip(pages, snapshot.items()):
            for off, v in rows.items():
                if v is not None:
                    self.kv[new * self.page_size + off] = v

    def proposals_enabled(self) -> bool:
        return self.draft_len > 0

    def propose(self, slots, anchors, positions, views, max_draft):
        out = []
        for slot, tok, pos in zip(slots, anchors, positions):
            toks, conf = [], []
            cur, p = tok, pos
            for j in range(min(self.draft_len, max_draft)):
                nxt = self.next_token_fn(cur, p)
                if self.draft_fn is not None:
                    nxt = self.draft_fn(slot, j, nxt)
                toks.append(nxt)
                conf.append(5.0)
                cur, p = nxt, p + 1
            out.append(Proposal(toks, conf))
        return out
