"""Logical paged-KV manager: page ownership, reservations, copy-on-write, prefix commit,
rollback, exact fork, preemption and quarantined retirement.

The manager never touches device memory.  It hands out *reservations* (new pages and, when
a shared tail page would be written, a private replacement page plus the copy the backend
must perform), turns the accepted prefix of a reservation into committed sequence state in
two phases (prepare -> publish, or abort), and returns every page that stops being
referenced as a `KvRetirement`.  Retired pages stay quarantined until the backend confirms
it no longer reads or writes them; only then do they return to the free list.

Counterpart of crates/ferrule-runtime/src/cache/page_manager.rs:280-1330 (API list in the
reference: alloc_sequence :517, reserve :609, reservation_bindings :1274, prepare_commit :705,
publish_commit :874, abort_* :904-918, fork :977-1045, preempt/restore :1098-1159,
confirm_page_retirement :431, stats :477).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from enum import Enum
from typing import Deque, Dict, Iterable, List, Optional, Sequence, Tuple

from .execution import KvCowReplacement


class KvError(RuntimeError):
    pass


class OutOfPages(KvError):
    pass


class ReservationState(Enum):
    RESERVED = "reserved"
    BOUND = "bound"
    PREPARED = "prepared"
    PUBLISHED = "published"
    ABORTED = "aborted"


@dataclass
class KvSequence:
    seq_id: int
    pages: List[int] = field(default_factory=list)
    committed_tokens: int = 0
    open_reservation: Optional[int] = None
    preempted: bool = False
    generation: int = 0


@dataclass
class KvReservation:
    res_id: int
    seq_id: int
    start: int                     # first token position covered
    tokens: int                    # tokens reserved
    new_pages: List[int]
    cow: Optional[KvCowReplacement]
    state: ReservationState = ReservationState.RESERVED
    execution_id: Optional[int] = None
    committed_rows: int = 0


@dataclass
class KvReservationView:
    """What an execution may touch: the page list as it will look while the batch runs."""
    res_id: int
    seq_id: int
    block_ids: List[int]
    context_len: int
    tokens: int
    cow: Optional[KvCowReplacement]


@dataclass
class KvRetirement:
    """Pages that left all page tables; quarantined until `confirm_page_retirement`."""
    pages: List[int] = field(default_factory=list)

    def extend(self, other: "KvRetirement") -> None:
        self.pages.extend(other.pages)

    def __bool__(self) -> bool:
        return bool(self.pages)


@dataclass
class KvStats:
    total_pages: int = 0
    free_pages: int = 0
    used_pages: int = 0
    quarantined_pages: int = 0
    shared_pages: int = 0
    sequences: int = 0
    open_reservations: int = 0
    cow_copies: int = 0
    forks: int = 0
    preemptions: int = 0
    high_water_used: int = 0
    reserve_failures: int = 0


@dataclass
class PreemptedSequence:
    seq_id: int
    committed_tokens: int
    exclusive: List[Tuple[int, int]]     # (logical index, physical page) owned only by this sequence
    shared: List[Tuple[int, int]]        # (logical index, physical page) still referenced elsewhere


class KvPageManager:
    def __init__(self, n_pages: int, page_size: int, max_sequence_len: int = 1 << 20):
        if n_pages <= 0 or page_size <= 0:
            raise KvError("page pool must be non-empty")
        self.n_pages, self.page_size, self.max_sequence_len = n_pages, page_size, max_sequence_len
        self._free: Deque[int] = deque(range(n_pages))
        self._ref = [0] * n_pages
        self._quarantine: set = set()
        self._seqs: Dict[int, KvSequence] = {}
        self._res: Dict[int, KvReservation] = {}
        self._next_seq = 0
        self._next_res = 0
        self._prepared: Dict[int, List[int]] = {}     # commit id -> reservation ids
        self._next_commit = 0
        self._preempted: Dict[int, PreemptedSequence] = {}
        self._stats = KvStats(total_pages=n_pages)

    # ------------------------------------------------------------------ helpers
    def _take(self, n: int) -> List[int]:
        if n == 0:                  # the common decode step: the tail page has room
            return []
        if n > len(self._free):
            self._stats.reserve_failures += 1
            raise OutOfPages(f"need {n} pages, {len(self._free)} free")
        out = [self._free.popleft() for _ in range(n)]
        for p in out:
            self._ref[p] = 1
        used = self.n_pages - len(self._free) - len(self._quarantine)
        self._stats.high_water_used = max(self._stats.high_water_used, used)
        return out

    def _decref(self, page: int, ret: KvRetirement) -> None:
        if not 0 <= page < self.n_pages:
            raise KvError(f"page id {page} outside the pool")
        if self._ref[page] <= 0:
            raise KvError(f"page {page} released twice")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._quarantine.add(page)
            ret.pages.append(page)

    def _seq(self, seq_id: int) -> KvSequence:
        s = self._seqs.get(seq_id)
        if s is None:
            raise KvError(f"unknown sequence {seq_id}")
        return s

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def free_page_ids(self) -> List[int]:
        """The pages on the free list, in allocation order (nothing is taken)."""
        return list(self._free)

    # ------------------------------------------------------------------ sequences
    def alloc_sequence(self) -> int:
        sid = self._next_seq
        self._next_seq += 1
        self._seqs[sid] = KvSequence(sid)
        return sid

    def sequence(self, seq_id: int) -> KvSequence:
        return self._seq(seq_id)

    def required_physical_pages(self, seq_id: int, new_tokens: int) -> int:
        """Pages a reservation of `new_tokens` would take from the free list (growth + COW)."""
        s = self._seq(seq_id)
        end = s.committed_tokens + new_tokens
        grow = max(self.pages_for(end) - len(s.pages), 0)
        return grow + (1 if self._needs_cow(s, new_tokens) else 0)

    def _needs_cow(self, s: KvSequence, new_tokens: int) -> bool:
        if new_tokens <= 0 or not s.pages:
            return False
        tail_fill = s.committed_tokens % self.page_size
        if tail_fill == 0:
            return False
        tail = s.pages[s.committed_tokens // self.page_size]
        return self._ref[tail] > 1

    # ------------------------------------------------------------------ reservations
    def reserve(self, seq_id: int, new_tokens: int) -> KvReservation:
        s = self._seq(seq_id)
        if s.preempted:
            raise KvError(f"sequence {seq_id} is preempted")
        if s.open_reservation is not None:
            raise KvError(f"sequence {seq_id} already has an open reservation")
        if new_tokens <= 0:
            raise KvError("reservation must cover at least one token")
        end = s.committed_tokens + new_tokens
        if end > self.max_sequence_len:
            raise KvError(f"sequence {seq_id} would exceed max_sequence_len")
        grow = max(self.pages_for(end) - len(s.pages), 0)
        need_cow = self._needs_cow(s, new_tokens)
        pages = self._take(grow + (1 if need_cow else 0))     # atomic: raises before any change
        cow = None
        if need_cow:
            li = s.committed_tokens // self.page_size
            cow = KvCowReplacement(li, s.pages[li], pages.pop())
            self._stats.cow_copies += 1
        r = KvReservation(self._next_res, seq_id, s.committed_tokens, new_tokens, pages, cow)
        self._next_res += 1
        self._res[r.res_id] = r
        s.open_reservation = r.res_id
        return r

    def try_reserve(self, seq_id: int, new_tokens: int, page_budget: int) -> Tuple[Optional[KvReservation], int]:
        """`reserve` if the pages it needs (growth + COW) fit both the free list and `page_budget`; otherwise
        (None, need).  One pass over the sequence instead of `required_physical_pages` followed by `reserve`."""
        s = self._seqs.get(seq_id)
        if s is None:
            raise KvError(f"unknown sequence {seq_id}")
        ps = self.page_size
        end = s.committed_tokens + new_tokens
        grow = (end + ps - 1) // ps - len(s.pages)
        if grow < 0:
            grow = 0
        need = grow + (1 if self._needs_cow(s, new_tokens) else 0)
        if need > len(self._free) or need > page_budget:
            return None, need
        return self.reserve(seq_id, new_tokens), need

    def bind_and_bindings(self, res_id: int, execution_id: int):
        """`bind_reservation_execution` + `reservation_bindings` in one lookup -> (reservation, blocks, slots)."""
        r = self._res.get(res_id)
        if r is None:
            raise KvError(f"unknown reservation {res_id}")
        if r.state != ReservationState.RESERVED:
            raise KvError(f"reservation {res_id} is {r.state.value}, cannot bind")
        r.state, r.execution_id = ReservationState.BOUND, execution_id
        s = self._seqs[r.seq_id]
        if r.cow is None and not r.new_pages:
            blocks = s.pages                      # read-only view: nothing changes while the reservation is open
        else:
            blocks = self._blocks_during(r)
        ps = self.page_size
        if r.tokens == 1:
            slots = [blocks[r.start // ps] * ps + r.start % ps]
        else:
            slots = [blocks[(r.start + j) // ps] * ps + (r.start + j) % ps for j in range(r.tokens)]
        return r, blocks, slots

    def reservation(self, res_id: int) -> KvReservation:
        r = self._res.get(res_id)
        if r is None:
            raise KvError(f"unknown reservation {res_id}")
        return r

    def bind_reservation_execution(self, res_id: int, execution_id: int) -> None:
        r = self.reservation(res_id)
        if r.state != ReservationState.RESERVED:
            raise KvError(f"reservation {res_id} is {r.state.value}, cannot bind")
        r.state, r.execution_id = ReservationState.BOUND, execution_id

    def _blocks_during(self, r: KvReservation) -> List[int]:
        s = self._seq(r.seq_id)
        blocks = list(s.pages)
        if r.cow is not None:
            blocks[r.cow.logical_page] = r.cow.replacement
        return blocks + r.new_pages

    def reservation_view(self, res_id: int) -> KvReservationView:
        r = self.reservation(res_id)
        return KvReservationView(r.res_id, r.seq_id, self._blocks_during(r), r.start, r.tokens, r.cow)

    def reservation_views(self, res_ids: Iterable[int]) -> List[KvReservationView]:
        return [self.reservation_view(i) for i in res_ids]

    def reservation_prefix_view(self, res_id: int, rows: int) -> KvReservationView:
        """The view restricted to the first `rows` reserved tokens (speculative prefix)."""
        r = self.reservation(res_id)
        if not 0 <= rows <= r.tokens:
            raise KvError("prefix longer than the reservation")
        blocks = self._blocks_during(r)[: self.pages_for(r.start + rows)]
        return KvReservationView(r.res_id, r.seq_id, blocks, r.start, rows, r.cow)

    def reservation_bindings(self, res_id: int) -> Tuple[List[int], List[int]]:
        """-> (block ids, write slot per reserved token) with slot = page * page_size + offset."""
        r = self.reservation(res_id)
        blocks = self._blocks_during(r)
        ps = self.page_size
        slots = [blocks[(r.start + j) // ps] * ps + (r.start + j) % ps for j in range(r.tokens)]
        return blocks, slots

    # ------------------------------------------------------------------ commit (two phase)
    def prepare_commit(self, commits: Sequence[Tuple[int, int]]) -> int:
        """commits = [(res_id, committed_rows)].  Validates everything first; on failure nothing
        changes and every reservation keeps all its tokens."""
        seen = set()
        for res_id, rows in commits:
            r = self.reservation(res_id)
            if res_id in seen:
                raise KvError(f"reservation {res_id} listed twice")
            seen.add(res_id)
            if r.state not in (ReservationState.RESERVED, ReservationState.BOUND):
                raise KvError(f"reservation {res_id} is {r.state.value}, cannot commit")
            if not 0 <= rows <= r.tokens:
                raise KvError(f"reservation {res_id}: committed_rows {rows} outside 0..{r.tokens}")
        for res_id, rows in commits:
            r = self._res[res_id]
            r.state, r.committed_rows = ReservationState.PREPARED, rows
        cid = self._next_commit
        self._next_commit += 1
        self._prepared[cid] = [c[0] for c in commits]
        return cid

    def publish_commit(self, commit_id: int) -> KvRetirement:
        ids = self._prepared.pop(commit_id, None)
        if ids is None:
            raise KvError(f"unknown prepared commit {commit_id}")
        ret = KvRetirement()
        for res_id in ids:
            r = self._res.pop(res_id)
            s = self._seq(r.seq_id)
            new_len = r.start + r.committed_rows
            if r.cow is not None:
                if r.committed_rows > 0:
                    s.pages[r.cow.logical_page] = r.cow.replacement
                    self._decref(r.cow.source, ret)
                else:
                    self._decref(r.cow.replacement, ret)
            keep = max(self.pages_for(new_len) - len(s.pages), 0)
            s.pages.extend(r.new_pages[:keep])
            for p in r.new_pages[keep:]:
                self._decref(p, ret)          # rejected suffix
            s.committed_tokens = new_len
            s.open_reservation = None
            r.state = ReservationState.PUBLISHED
        return ret

    def abort_prepared_commit(self, commit_id: int) -> None:
        """Back to reserved/bound: the reservations keep every page."""
        ids = self._prepared.pop(commit_id, None)
        if ids is None:
            raise KvError(f"unknown prepared commit {commit_id}")
        for res_id in ids:
            r = self._res[res_id]
            r.state = ReservationState.BOUND if r.execution_id is not None else ReservationState.RESERVED
            r.committed_rows = 0

    def abort_reservations(self, res_ids: Iterable[int]) -> KvRetirement:
        ret = KvRetirement()
        res_ids = list(res_ids)
        for res_id in res_ids:                  # checked before anything changes: a refused abort aborts nothing
            r = self._res.get(res_id)
            if r is not None and r.state == ReservationState.PREPARED:
                raise KvError(f"reservation {res_id} is part of a prepared commit; abort that first")
        for res_id in res_ids:
            r = self._res.pop(res_id, None)
            if r is None:
                continue
            for p in r.new_pages:
                self._decref(p, ret)
            if r.cow is not None:
                self._decref(r.cow.replacement, ret)
            s = self._seqs.get(r.seq_id)
            if s is not None and s.open_reservation == res_id:
                s.open_reservation = None
            r.state = ReservationState.ABORTED
        return ret

    # ------------------------------------------------------------------ release / retirement
    def free_sequence_pages(self, seq_id: int) -> KvRetirement:
        s = self._seq(seq_id)
        ret = KvRetirement()
        if s.open_reservation is not None:
            ret.extend(self.abort_reservations([s.open_reservation]))
        for p in s.pages:
            if p >= 0:              # a preempted sequence's released pages are marked -1
                self._decref(p, ret)
        del self._seqs[seq_id]
        self._preempted.pop(seq_id, None)
        return ret

    def truncate_sequence(self, seq_id: int, tokens: int) -> KvRetirement:
        """Roll a sequence back to `tokens` committed tokens (session reset / speculative undo)."""
        s = self._seq(seq_id)
        if s.open_reservation is not None:
            raise KvError("cannot truncate under an open reservation")
        if not 0 <= tokens <= s.committed_tokens:
            raise KvError("truncate target outside the committed range")
        ret = KvRetirement()
        keep = self.pages_for(tokens)
        for p in s.pages[keep:]:
            if p >= 0:
                self._decref(p, ret)
        del s.pages[keep:]
        s.committed_tokens = tokens
        s.generation += 1
        return ret

    def confirm_page_retirement(self, pages: Iterable[int]) -> int:
        """The backend no longer touches these pages: they become allocatable again."""
        n = 0
        for p in pages:
            if p not in self._quarantine:
                raise KvError(f"page {p} is not awaiting retirement")
            self._quarantine.discard(p)
            self._free.append(p)
            n += 1
        return n

    # ------------------------------------------------------------------ fork
    def prepare_fork_sequence_exact(self, src_id: int) -> Tuple[int, List[int]]:
        """-> (tokens, pages) that a child would share; nothing changes yet."""
        s = self._seq(src_id)
        if s.open_reservation is not None:
            raise KvError("cannot fork a sequence with an open reservation")
        if s.preempted:
            raise KvError("cannot fork a preempted sequence")
        return s.committed_tokens, list(s.pages)

    def publish_fork_sequence_exact(self, src_id: int) -> int:
        tokens, pages = self.prepare_fork_sequence_exact(src_id)
        cid = self.alloc_sequence()
        c = self._seqs[cid]
        c.pages, c.committed_tokens = pages, tokens
        for p in pages:
            self._ref[p] += 1
        self._stats.forks += 1
        return cid

    def publish_fork_sequence_prefix(self, src_id: int, tokens: int) -> int:
        """New sequence that shares the pages of the first `tokens` committed tokens of `src_id` (a whole number
        of pages: nothing is copied and the child's first write lands in a page of its own)."""
        s = self._seq(src_id)
        if s.open_reservation is not None:
            raise KvError("cannot fork a sequence with an open reservation")
        if s.preempted:
            raise KvError("cannot fork a preempted sequence")
        if tokens <= 0 or tokens > s.committed_tokens or tokens % self.page_size != 0:
            raise KvError("a prefix fork takes a positive whole number of committed pages")
        pages = list(s.pages[:tokens // self.page_size])
        cid = self.alloc_sequence()
        c = self._seqs[cid]
        c.pages, c.committed_tokens = pages, tokens
        for p in pages:
            self._ref[p] += 1
        self._stats.forks += 1
        return cid

    # ------------------------------------------------------------------ preempt / restore
    def preempt_sequence(self, seq_id: int) -> PreemptedSequence:
        """Mark preempted and say which pages must be snapshotted (exclusively owned)."""
        s = self._seq(seq_id)
        if s.open_reservation is not None:
            raise KvError("cannot preempt a sequence with an open reservation")
        if s.preempted:
            raise KvError("sequence already preempted")
        excl = [(i, p) for i, p in enumerate(s.pages) if self._ref[p] == 1]
        shared = [(i, p) for i, p in enumerate(s.pages) if self._ref[p] > 1]
        rec = PreemptedSequence(seq_id, s.committed_tokens, excl, shared)
        s.preempted = True
        self._preempted[seq_id] = rec
        self._stats.preemptions += 1
        return rec

    def release_preempted_pages(self, seq_id: int) -> KvRetirement:
        """After the snapshot is safe on the host: give the exclusive pages back."""
        rec = self._preempted.get(seq_id)
        if rec is None:
            raise KvError(f"sequence {seq_id} is not preempted")
        s = self._seq(seq_id)
        ret = KvRetirement()
        for i, p in rec.exclusive:
            if s.pages[i] == p:
                self._decref(p, ret)
                s.pages[i] = -1
        return ret

    def restore_sequence(self, seq_id: int) -> List[Tuple[int, int]]:
        """Allocate fresh pages for the snapshotted ones -> [(logical index, new physical page)]."""
        rec = self._preempted.get(seq_id)
        if rec is None:
            raise KvError(f"sequence {seq_id} is not preempted")
        s = self._seq(seq_id)
        missing = [i for i, p in enumerate(s.pages) if p < 0]
        pages = self._take(len(missing))
        out = []
        for i, p in zip(missing, pages):
            s.pages[i] = p
            out.append((i, p))
        s.preempted = False
        s.generation += 1
        del self._preempted[seq_id]
        return out

    # ------------------------------------------------------------------ stats / invariants
    def stats(self) -> KvStats:
        st = self._stats
        st.free_pages = len(self._free)
        st.quarantined_pages = len(self._quarantine)
        st.used_pages = self.n_pages - st.free_pages - st.quarantined_pages
        st.shared_pages = sum(1 for r in self._ref if r > 1)
        st.sequences = len(self._seqs)
        st.open_reservations = len(self._res)
        return st

    def check_invariants(self) -> None:
        """Every page is exactly one of: free, quarantined, referenced (refcount = number of holders)."""
        holders = [0] * self.n_pages
        for s in self._seqs.values():
            for p in s.pages:
                if p >= 0:
                    holders[p] += 1
        for r in self._res.values():
            for p in r.new_pages:
                holders[p] += 1
            if r.cow is not None:
                holders[r.cow.replacement] += 1
        free = set(self._free)
        if len(free) != len(self._free):
            raise KvError("free list holds a page twice")
        for p in range(self.n_pages):
            states = (p in free) + (p in self._quarantine) + (holders[p] > 0)
            if states != 1:
                raise KvError(f"page {p}: free={p in free} quarantined={p in self._quarantine} holders={holders[p]}")
            if holders[p] != self._ref[p] and holders[p] > 0:
                raise KvError(f"page {p}: refcount {self._ref[p]} but {holders[p]} holders")
