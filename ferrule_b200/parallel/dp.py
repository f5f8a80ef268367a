"""Data parallelism: independent engine replicas (one per GPU or GPU group) behind one front end.

Every replica is a complete `ModelWorker` (its own engine thread, KV pool and CUDA graphs); requests are
placed on the replica with the fewest live requests, and a request with a `session_id` always returns to the
replica that holds its retained session.  Replicas share nothing, so throughput scales with their number as
long as the front end keeps them fed; a replica whose engine latched a fatal error is skipped.

The reference's `ParallelismPlan` carries `data_parallel: 1` and nothing else
(crates/ferrule-model/src/support/policies.rs:56-77); this is the data-parallel row of the parallelism inventory.
"""
from __future__ import annotations

import threading
from typing import Dict, List, Optional

from ..server.worker import ModelWorker, RequestStream, WorkerError


class DataParallelWorker:
    """Duck-types the part of `ModelWorker` the HTTP layer uses (submit / cancel / tokenize / stats / healthy)."""

    def __init__(self, replicas: List[ModelWorker], model_name: Optional[str] = None):
        if not replicas:
            raise ValueError("at least one replica is needed")
        self.replicas = replicas
        self.model_name = model_name or replicas[0].model_name
        self.tokenizer = replicas[0].tokenizer
        self._sessions: Dict[str, int] = {}
        self._owner: Dict[str, int] = {}
        self._lock = threading.Lock()
        self.placed = [0] * len(replicas)

    # the HTTP layer reads `worker.engine.cfg.scheduler.ctx_size` for /tokenize
    @property
    def engine(self):
        return self.replicas[0].engine

    def start(self, timeout: float = 600.0) -> "DataParallelWorker":
        for r in self.replicas:
            r.start(timeout)
        return self

    def stop(self, timeout: float = 30.0) -> None:
        for r in self.replicas:
            r.stop(timeout)

    @property
    def healthy(self) -> bool:
        return any(r.healthy for r in self.replicas)

    def _pick(self, session_id: Optional[str]) -> int:
        with self._lock:
            if session_id is not None and session_id in self._sessions and self.replicas[self._sessions[session_id]].healthy:
                return self._sessions[session_id]
            # fewest live requests first; ties go to the replica that has been given the least work so far
            live = [(len(r._live), self.placed[i], i) for i, r in enumerate(self.replicas) if r.healthy]
            if not live:
                raise WorkerError("no healthy replica", 503, "worker_failed")
            i = min(live)[2]
            if session_id is not None:
                self._sessions[session_id] = i
            return i

    async def submit(self, *, request_id: Optional[str] = None, session_id: Optional[str] = None, **kw) -> RequestStream:
        i = self._pick(session_id)
        stream = await self.replicas[i].submit(request_id=request_id, session_id=session_id, **kw)
        with self._lock:
            self._owner[stream.request_id] = i
            self.placed[i] += 1
            if len(self._owner) > 65536:           # finished requests are forgotten lazily
                for k in list(self._owner)[:32768]:
                    del self._owner[k]
        return stream

    def cancel(self, request_id: str) -> None:
        i = self._owner.get(request_id)
        if i is not None:
            self.replicas[i].cancel(request_id)

    def tokenize(self, text: str) -> List[int]:
        return self.tokenizer.encode(text)

    def stats(self) -> Dict[str, object]:
        return {"healthy": self.healthy, "replicas": [r.stats() for r in self.replicas], "placed": list(self.placed)}
