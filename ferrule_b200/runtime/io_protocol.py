"""Typed vocabulary of the materialization layer: identities, lifecycle, completions, leases.

A *materialization* is one physical act of bringing a resource (a routed expert's weights, a
weight shard) from storage to a stable device slot.  Its identity is the full
`MaterializationKey`; any field that differs means two different operations that must never be
coalesced.  Its lifecycle is the ten-state `LoadStage` machine with an explicit table of legal
transitions.  Everything that comes back from a provider is a `CompletionEvent`, checked against
the `CompletionExpectation` the owner recorded when it submitted the work.

Counterpart of crates/ferrule-common/src/io_protocol.rs (keys :430-540, dependencies :543-655,
LoadStage :659-735, completions :744-1000, retirement :1027-1080, slab leases :1094-1410,
residency bindings :1419-1650, ModelProgress :1654-1675) and materialization_io.rs:27-191.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from enum import Enum
from typing import Dict, FrozenSet, Generic, Iterable, List, Optional, Tuple, TypeVar


class IoProtocolError(RuntimeError):
    pass


class ResourceKind(Enum):
    ROUTED_EXPERT = "routed_expert"
    SHARED_EXPERT = "shared_expert"
    DENSE_WEIGHT = "dense_weight"
    EMBEDDING = "embedding"
    OUTPUT_HEAD = "output_head"


@dataclass(frozen=True, order=True)
class ResourceId:
    kind: ResourceKind
    group: int          # e.g. layer
    item: int           # e.g. expert index

    def __str__(self) -> str:
        return f"{self.kind.value}[{self.group}:{self.item}]"


def content_hash(*parts: bytes) -> bytes:
    h = hashlib.sha256()
    for p in parts:
        h.update(len(p).to_bytes(8, "little"))
        h.update(p)
    return h.digest()


@dataclass(frozen=True)
class MaterializationKey:
    model: str
    source_identity: bytes          # hash of (path, size, mtime...) of the backing files
    content: bytes                  # hash of the tensor slices that make up the payload
    resource: ResourceId
    payload_encoding: int           # how the bytes are laid out for the device (format id)
    backend: str                    # e.g. "cuda-sm100a"
    device: int
    source_generation: int          # bumps when the checkpoint on disk is replaced
    destination_generation: int     # bumps when the destination slot set is rebuilt

    def same_payload(self, other: "MaterializationKey") -> bool:
        return self == other        # every field participates: no partial matches


class LoadStage(Enum):
    RESERVED = "reserved"
    READ_SUBMITTED = "read_submitted"
    HOST_READY = "host_ready"
    UPLOAD_SUBMITTED = "upload_submitted"
    INSTALLING = "installing"
    RESIDENT = "resident"
    FAILED = "failed"
    STALE = "stale"
    DRAINING = "draining"
    RETIRED = "retired"


_S = LoadStage
_LEGAL: Dict[LoadStage, FrozenSet[LoadStage]] = {
    _S.RESERVED: frozenset({_S.READ_SUBMITTED, _S.RETIRED}),
    _S.READ_SUBMITTED: frozenset({_S.HOST_READY, _S.FAILED, _S.STALE, _S.DRAINING}),
    _S.HOST_READY: frozenset({_S.UPLOAD_SUBMITTED, _S.FAILED, _S.STALE}),
    _S.UPLOAD_SUBMITTED: frozenset({_S.INSTALLING, _S.FAILED, _S.STALE, _S.DRAINING}),
    _S.INSTALLING: frozenset({_S.RESIDENT, _S.FAILED, _S.STALE, _S.DRAINING}),
    _S.RESIDENT: frozenset({_S.RETIRED}),
    _S.FAILED: frozenset({_S.DRAINING, _S.RETIRED}),
    _S.STALE: frozenset({_S.DRAINING, _S.RETIRED}),
    _S.DRAINING: frozenset({_S.RETIRED}),
    _S.RETIRED: frozenset(),
}


def can_transition(a: LoadStage, b: LoadStage) -> bool:
    return b in _LEGAL[a]


def validate_transition(a: LoadStage, b: LoadStage) -> None:
    if not can_transition(a, b):
        raise IoProtocolError(f"illegal load transition {a.value} -> {b.value}")


def is_submitted_stage(s: LoadStage) -> bool:
    """Stages in which a physical operation is in flight and a completion is owed."""
    return s in (_S.READ_SUBMITTED, _S.UPLOAD_SUBMITTED, _S.INSTALLING)


class Purpose(Enum):
    EXECUTION = "execution"
    PREFETCH = "prefetch"


class FailureReason(Enum):
    READ_ERROR = "read_error"
    SHORT_READ = "short_read"
    UPLOAD_ERROR = "upload_error"
    INSTALL_ERROR = "install_error"
    CANCELLED = "cancelled"
    PROVIDER_LOST = "provider_lost"
    RESOURCE_EXHAUSTED = "resource_exhausted"


class CompletionOutcome(Enum):
    OK = "ok"
    FAILED = "failed"
    CANCELLED = "cancelled"


@dataclass(frozen=True)
class CompletionEvent:
    operation: int                  # registry operation id
    key: MaterializationKey
    stage: LoadStage                # the submitted stage this completion answers
    generation: int                 # submission generation (a retry bumps it)
    outcome: CompletionOutcome
    bytes_done: int = 0
    failure: Optional[FailureReason] = None
    timestamp_ns: int = 0


@dataclass(frozen=True)
class CompletionExpectation:
    operation: int
    key: MaterializationKey
    stage: LoadStage
    generation: int
    bytes_expected: int

    def check(self, ev: CompletionEvent) -> Optional[str]:
        """None if the event answers exactly this expectation, else why not."""
        if ev.operation != self.operation:
            return "wrong operation"
        if ev.key != self.key:
            return "wrong key"
        if ev.stage != self.stage:
            return f"wrong stage ({ev.stage.value}, expected {self.stage.value})"
        if ev.generation != self.generation:
            return "stale generation"
        if ev.outcome == CompletionOutcome.OK and ev.bytes_done != self.bytes_expected:
            return f"byte count {ev.bytes_done} != {self.bytes_expected}"
        return None


class RetirementReason(Enum):
    EVICTED = "evicted"
    FAILED = "failed"
    STALE = "stale"
    SHUTDOWN = "shutdown"
    CANCELLED = "cancelled"


class RetirementToken:
    """Proof that an operation's resources may be released; consumable exactly once."""

    def __init__(self, operation: int, reason: RetirementReason):
        self.operation, self.reason = operation, reason
        self._used = False

    def consume(self) -> None:
        if self._used:
            raise IoProtocolError(f"retirement token of operation {self.operation} used twice")
        self._used = True

    @property
    def consumed(self) -> bool:
        return self._used


class SlabLeaseState(Enum):
    FREE = "free"
    LEASED = "leased"               # handed to a read
    FILLED = "filled"               # host bytes valid
    UPLOADING = "uploading"         # an async copy reads from it
    RELEASED = "released"


_SLAB_NEXT = {
    SlabLeaseState.FREE: {SlabLeaseState.LEASED},
    SlabLeaseState.LEASED: {SlabLeaseState.FILLED, SlabLeaseState.RELEASED},
    SlabLeaseState.FILLED: {SlabLeaseState.UPLOADING, SlabLeaseState.RELEASED},
    SlabLeaseState.UPLOADING: {SlabLeaseState.RELEASED},
    SlabLeaseState.RELEASED: {SlabLeaseState.FREE},
}


@dataclass
class PinnedSlabLease:
    """A registered, aligned slice of pinned host memory on loan to one operation."""
    slab: int
    offset: int
    nbytes: int
    alignment: int = 4096
    state: SlabLeaseState = SlabLeaseState.FREE
    operation: Optional[int] = None
    base_address: int = 0           # address of the slab buffer; offset is relative to it

    def advance(self, nxt: SlabLeaseState) -> None:
        if nxt not in _SLAB_NEXT[self.state]:
            raise IoProtocolError(f"slab lease {self.state.value} -> {nxt.value} is not allowed")
        self.state = nxt

    def validate(self) -> None:
        if (self.base_address + self.offset) % self.alignment or self.nbytes % self.alignment:
            raise IoProtocolError("slab lease is not aligned for direct I/O")


@dataclass(frozen=True)
class ResidencyBinding:
    """Claim that `resource` is resident in `slot` at `generation` (as seen by the model side)."""
    resource: ResourceId
    slot: int
    generation: int


@dataclass(frozen=True)
class ValidatedResidencyBinding:
    binding: ResidencyBinding
    lease: int                      # residency lease id held for the dispatch


@dataclass
class ResidencyLeaseSet:
    """All leases one dispatch holds; released together when the consumer fence has passed."""
    bindings: List[ValidatedResidencyBinding] = field(default_factory=list)
    released: bool = False

    def release(self) -> List[int]:
        if self.released:
            raise IoProtocolError("lease set released twice")
        self.released = True
        return [b.lease for b in self.bindings]


@dataclass(frozen=True)
class DependencySet:
    """Exact keys a suspended transaction needs before it can resume."""
    keys: Tuple[MaterializationKey, ...]

    @staticmethod
    def of(keys: Iterable[MaterializationKey]) -> "DependencySet":
        seen, out = set(), []
        for k in keys:
            if k not in seen:
                seen.add(k)
                out.append(k)
        return DependencySet(tuple(out))

    def __len__(self) -> int:
        return len(self.keys)


@dataclass(frozen=True)
class WaiterId:
    transaction: int
    request_generation: int
    dependency_epoch: int
    continuation: int


@dataclass
class MaterializationResourcePlan:
    """Hard resources one operation needs at each phase (fed to the resource broker)."""
    read_slots: int = 1
    storage_bytes: int = 0
    pinned_bytes: int = 0
    upload_slots: int = 1
    h2d_bytes: int = 0
    install_slots: int = 1
    device_install_bytes: int = 0
    resident_bytes: int = 0

    @staticmethod
    def for_payload(nbytes: int, alignment: int = 4096) -> "MaterializationResourcePlan":
        aligned = (nbytes + alignment - 1) // alignment * alignment
        return MaterializationResourcePlan(storage_bytes=aligned, pinned_bytes=aligned, h2d_bytes=nbytes,
                                           device_install_bytes=nbytes, resident_bytes=nbytes)


T = TypeVar("T")


@dataclass
class ModelProgress(Generic[T]):
    """Either a finished value or the exact dependencies that must be materialized first."""
    value: Optional[T] = None
    pending: Optional[DependencySet] = None

    @property
    def complete(self) -> bool:
        return self.pending is None
