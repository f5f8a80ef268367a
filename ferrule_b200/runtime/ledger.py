"""Critical-path ledger: where did the time of each output token go?

Operations record timestamped spans per phase (READ, UPLOAD, PUBLISH, WAIT, RESUME, COMMIT).
A transaction that waits on several operations is charged the *union* of their spans, and a
wait is "covered" while other runnable work was executing on the device.  `snapshot_for_token`
returns, per emitted token, total / covered / uncovered wait, which is the evidence required to
claim that I/O is hidden behind compute.

Counterpart of crates/ferrule-runtime/src/io/ledger.rs:39-47 (phases), :99-115 (snapshots),
:127-200 (interval union and cover).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, Iterable, List, Tuple


class LedgerPhase(Enum):
    READ = "read"
    UPLOAD = "upload"
    PUBLISH = "publish"
    WAIT = "wait"
    RESUME = "resume"
    COMMIT = "commit"


Span = Tuple[int, int]


def union_length(spans: Iterable[Span]) -> int:
    total, cur_s, cur_e = 0, None, None
    for s, e in sorted(spans):
        if e <= s:
            continue
        if cur_e is None or s > cur_e:
            if cur_e is not None:
                total += cur_e - cur_s
            cur_s, cur_e = s, e
        else:
            cur_e = max(cur_e, e)
    if cur_e is not None:
        total += cur_e - cur_s
    return total


def intersect(a: Iterable[Span], b: Iterable[Span]) -> List[Span]:
    out = []
    for s1, e1 in a:
        for s2, e2 in b:
            s, e = max(s1, s2), min(e1, e2)
            if e > s:
                out.append((s, e))
    return out


@dataclass
class TokenSnapshot:
    token_index: int
    wait_ns: int
    covered_ns: int

    @property
    def uncovered_ns(self) -> int:
        return self.wait_ns - self.covered_ns


class CriticalPathLedger:
    def __init__(self, keep: int = 4096):
        self.keep = keep
        self._op: Dict[int, Dict[LedgerPhase, List[Span]]] = {}
        self._wait: Dict[int, List[Span]] = {}          # transaction -> wait spans
        self._work: List[Span] = []                      # device busy with other runnable work
        self.snapshots: List[TokenSnapshot] = []

    def record_operation(self, op: int, phase: LedgerPhase, start_ns: int, end_ns: int) -> None:
        self._op.setdefault(op, {}).setdefault(phase, []).append((start_ns, end_ns))

    def record_wait(self, txn: int, start_ns: int, end_ns: int) -> None:
        self._wait.setdefault(txn, []).append((start_ns, end_ns))

    def record_runnable_work(self, start_ns: int, end_ns: int) -> None:
        self._work.append((start_ns, end_ns))
        if len(self._work) > self.keep:
            del self._work[: len(self._work) - self.keep]

    def operation_time(self, op: int, phase: LedgerPhase) -> int:
        return union_length(self._op.get(op, {}).get(phase, []))

    def shared_wait(self, ops: Iterable[int], phases=(LedgerPhase.READ, LedgerPhase.UPLOAD, LedgerPhase.PUBLISH)) -> int:
        """Wall time during which at least one of `ops` was in one of `phases` (shared waits unioned)."""
        spans: List[Span] = []
        for op in ops:
            for ph in phases:
                spans.extend(self._op.get(op, {}).get(ph, []))
        return union_length(spans)

    def snapshot_for_token(self, txn: int, token_index: int) -> TokenSnapshot:
        waits = self._wait.pop(txn, [])
        snap = TokenSnapshot(token_index, union_length(waits), union_length(intersect(waits, self._work)))
        self.snapshots.append(snap)
        if len(self.snapshots) > self.keep:
            del self.snapshots[: len(self.snapshots) - self.keep]
        return snap

    def summary(self) -> Dict[str, float]:
        n = len(self.snapshots)
        w = sum(s.wait_ns for s in self.snapshots)
        c = sum(s.covered_ns for s in self.snapshots)
        return {"tokens": n, "wait_ns": w, "covered_ns": c, "uncovered_ns": w - c,
                "covered_fraction": (c / w) if w else 1.0}
