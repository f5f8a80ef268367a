"""Shape-keyed reuse of execution arenas and the committed-sequence lifecycle core.

`PersistentArenaPool` keeps idle arenas (workspace buffers, staging areas, captured graphs ...) in
exact-key buckets: an acquisition reuses an idle arena of exactly that key or builds one; a failed
build publishes nothing; a lease returns its arena to the same bucket when it ends, an owned
checkout must be checked in explicitly (exactly once).  Hit / miss / install counters are
cumulative and survive `clear()`.

`SequenceStateCore` is the family-neutral cursor of one sequence's committed state: generation,
committed position, poison flag.  A step binds to (generation, position) when it begins; it can
only be committed while both still match, so a stale or replayed step is refused; a step that
cannot be rolled back poisons the state until `reset` / `restore_from`.

Counterpart of crates/ferrule-model/src/execution/arena.rs:9-190 and
crates/ferrule-model/src/execution/sequence.rs:5-140.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Generic, Hashable, List, TypeVar

K = TypeVar("K", bound=Hashable)
A = TypeVar("A")


class ExecutionStateError(RuntimeError):
    pass


@dataclass
class ArenaPoolStats:
    hits: int = 0        # acquisitions that reused an idle arena of the exact key
    misses: int = 0      # acquisitions whose bucket had no idle arena (failed builds included)
    installs: int = 0    # arenas built successfully


class OwnedArenaCheckout(Generic[K, A]):
    """An arena taken out of the pool; give it back with `PersistentArenaPool.checkin` (once)."""

    def __init__(self, key: K, arena: A, reused: bool):
        self.key, self.arena, self.reused = key, arena, reused
        self._returned = False


class ArenaLease(Generic[K, A]):
    """Context manager form: the arena goes back to its bucket when the block ends."""

    def __init__(self, pool: "PersistentArenaPool[K, A]", checkout: OwnedArenaCheckout):
        self._pool, self._co = pool, checkout

    @property
    def arena(self) -> A:
        return self._co.arena

    @property
    def reused(self) -> bool:
        return self._co.reused

    def __enter__(self) -> A:
        return self._co.arena

    def __exit__(self, *exc) -> None:
        self._pool.checkin(self._co)


class PersistentArenaPool(Generic[K, A]):
    def __init__(self) -> None:
        self._available: Dict[K, List[A]] = {}
        self._leased = False
        self.stats = ArenaPoolStats()

    def __len__(self) -> int:
        """Buckets that hold at least one idle arena."""
        return len(self._available)

    def __contains__(self, key: K) -> bool:
        return key in self._available

    def idle(self, key: K) -> int:
        return len(self._available.get(key, ()))

    def clear(self) -> None:
        self._available.clear()

    def _take_or_build(self, key: K, build: Callable[[], A]) -> OwnedArenaCheckout:
        bucket = self._available.get(key)
        if bucket:
            arena = bucket.pop()
            if not bucket:
                del self._available[key]
            self.stats.hits += 1
            return OwnedArenaCheckout(key, arena, True)
        self.stats.misses += 1
        arena = build()                      # a failing build propagates; nothing is published
        self.stats.installs += 1
        return OwnedArenaCheckout(key, arena, False)

    def checkout(self, key: K, build: Callable[[], A]) -> OwnedArenaCheckout:
        return self._take_or_build(key, build)

    def checkin(self, checkout: OwnedArenaCheckout) -> None:
        if checkout._returned:
            raise ExecutionStateError("arena checked in twice")
        checkout._returned = True
        self._available.setdefault(checkout.key, []).append(checkout.arena)
        if self._leased and getattr(checkout, "_lease", False):
            self._leased = False

    def acquire(self, key: K, build: Callable[[], A]) -> ArenaLease:
        """One lease at a time (the reference expresses this by borrowing the pool mutably)."""
        if self._leased:
            raise ExecutionStateError("the pool already has an active lease")
        co = self._take_or_build(key, build)
        co._lease = True
        self._leased = True
        return ArenaLease(self, co)

    try_lease = acquire


@dataclass(frozen=True)
class SequenceStepBinding:
    generation: int
    committed_position: int


class SequenceStateCore:
    def __init__(self, position: int = 0):
        self.generation, self.position, self.poisoned = 0, position, False

    def begin_step(self) -> SequenceStepBinding:
        if self.poisoned:
            raise ExecutionStateError("sequence state is poisoned; reset or release it before reuse")
        return SequenceStepBinding(self.generation, self.position)

    def commit_step(self, binding: SequenceStepBinding, rows: int) -> None:
        if self.poisoned:
            raise ExecutionStateError("cannot commit a poisoned sequence state")
        if binding.generation != self.generation or binding.committed_position != self.position:
            raise ExecutionStateError(
                f"stale sequence binding: generation/position {binding.generation}/{binding.committed_position} "
                f"no longer matches {self.generation}/{self.position}")
        self.position += rows

    def poison_step(self, binding: SequenceStepBinding) -> None:
        if binding.generation == self.generation:
            self.poisoned = True

    def poison(self) -> None:
        self.poisoned = True

    def reset(self) -> None:
        self.position, self.poisoned = 0, False
        self.generation += 1

    def rewind(self, position: int) -> None:
        """Roll the committed cursor back (an aborted or rejected suffix) under a new generation."""
        if not 0 <= position <= self.position:
            raise ExecutionStateError("rewind target outside the committed range")
        self.position, self.poisoned = position, False
        self.generation += 1

    def forked(self) -> "SequenceStateCore":
        self.begin_step()
        c = SequenceStateCore(self.position)
        c.generation = self.generation + 1
        return c

    def restore_from(self, snapshot: "SequenceStateCore") -> None:
        self.position, self.poisoned = snapshot.position, False
        self.generation = max(self.generation, snapshot.generation) + 1
