"""Per-layer, per-stage timing tables of a forward pass and debug taps of its intermediate tensors.

`StageProfiler` is driven by marks: `mark(layer, "attn.core")` ends the stage that was open and opens the named
one, `mark(layer, None)` ends without opening.  On a GPU a mark is one CUDA event recorded on the current stream
(durations are read back later, when the events have completed - nothing synchronises unless `sync` is set, which
waits at every mark so that host-side gaps show up inside the stage that caused them); on the CPU a mark reads
the clock.  The table has one row per (layer, stage): calls, total and mean microseconds, share of the total.

Both are configured from the environment once, when a runner is built (later changes do not reach a running
model):
    FERRULE_PROFILE=1            collect the stage table (the runner then steps eagerly: no CUDA graph, no
                                 look-ahead; a captured graph cannot hold per-stage host callbacks)
    FERRULE_PROFILE_SYNC=1       synchronise at every mark
    FERRULE_PREFILL_PROGRESS=1   log one line per prompt chunk (target `ferrule_prefill`)
    FERRULE_DEBUG_STAGE_DUMP_DIR=<dir> [FERRULE_DEBUG_LAYER=<i>] [FERRULE_DEBUG_STAGE=<name>]
                                 write tapped tensors (`<dir>/step<NNNNN>_layer<i>_<stage>.pt`)

Counterpart of the reference's frozen profiling switches and stage tables
(crates/ferrule-model/src/models/deepseek_v4/prepared.rs:195-247, operators.rs:38-130, :346-475) and of its debug
taps (crates/ferrule-model/src/models/deepseek_v4/layer.rs:42-92, attention.rs:38-117).
"""
from __future__ import annotations

import os
import time
from pathlib import Path
from typing import Dict, List, Optional, Tuple

import torch


def _flag(name: str) -> bool:
    return os.environ.get(name, "").strip().lower() in ("1", "true", "yes", "on")


class StageProfiler:
    MAX_PENDING = 8192

    def __init__(self, device, sync: bool = False):
        self.cuda = torch.device(device).type == "cuda"
        self.sync = sync
        self.rows: Dict[Tuple[int, str], List[float]] = {}       # (layer, stage) -> [total us, calls]
        self._open: Optional[Tuple[int, str, object]] = None     # (layer, stage, start event | start ns)
        self._pending: List[Tuple[Tuple[int, str], object, object]] = []
        self.marks = 0

    @staticmethod
    def from_env(device) -> Optional["StageProfiler"]:
        return StageProfiler(device, sync=_flag("FERRULE_PROFILE_SYNC")) if _flag("FERRULE_PROFILE") else None

    # ------------------------------------------------------------------ marks
    def _now(self):
        if not self.cuda:
            return time.perf_counter_ns()
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        if self.sync:
            ev.synchronize()
        return ev

    def mark(self, layer: int, stage: Optional[str]) -> None:
        """End the open stage here and (with a name) open `stage` of `layer`."""
        if self.cuda and torch.cuda.is_current_stream_capturing():
            return                                   # a graph capture cannot carry timing events: not measured
        now = self._now()
        self.marks += 1
        if self._open is not None:
            l0, s0, start = self._open
            if self.cuda:
                self._pending.append(((l0, s0), start, now))
                if len(self._pending) >= self.MAX_PENDING:
                    self.flush()
            else:
                self._add((l0, s0), (now - start) / 1e3)
        self._open = (layer, stage, now) if stage is not None else None

    def _add(self, key: Tuple[int, str], us: float) -> None:
        row = self.rows.setdefault(key, [0.0, 0])
        row[0] += us
        row[1] += 1

    def flush(self, wait: bool = False) -> None:
        """Fold finished event pairs into the table (`wait`: synchronise with the newest one first)."""
        if not self._pending:
            return
        if wait:
            self._pending[-1][2].synchronize()
        keep = []
        for key, e0, e1 in self._pending:
            if e1.query():
                self._add(key, e0.elapsed_time(e1) * 1e3)
            else:
                keep.append((key, e0, e1))
        self._pending = keep

    # ------------------------------------------------------------------ report
    def table(self) -> List[dict]:
        self.flush(wait=True)
        total = sum(r[0] for r in self.rows.values()) or 1.0
        out = []
        for (layer, stage), (us, calls) in sorted(self.rows.items()):
            out.append({"layer": layer, "stage": stage, "calls": int(calls), "total_us": round(us, 1),
                        "mean_us": round(us / max(calls, 1), 2), "share": round(us / total, 4)})
        return out

    def by_stage(self) -> List[dict]:
        """The table summed over layers, largest first."""
        acc: Dict[str, List[float]] = {}
        for row in self.table():
            a = acc.setdefault(row["stage"], [0.0, 0])
            a[0] += row["total_us"]
            a[1] += row["calls"]
        total = sum(a[0] for a in acc.values()) or 1.0
        return [{"stage": s, "calls": int(c), "total_us": round(us, 1), "mean_us": round(us / max(c, 1), 2),
                 "share": round(us / total, 4)} for s, (us, c) in sorted(acc.items(), key=lambda kv: -kv[1][0])]

    def reset(self) -> None:
        self.rows.clear()
        self._pending.clear()
        self._open = None


class DebugTap:
    """Writes tapped tensors to a directory; `wants(layer, stage)` is cheap, so call sites test it first."""

    def __init__(self, directory, layer: Optional[int] = None, stage: Optional[str] = None):
        self.dir = Path(directory)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.layer, self.stage = layer, stage
        self.step = 0
        self.written: List[str] = []

    @staticmethod
    def from_env() -> Optional["DebugTap"]:
        d = os.environ.get("FERRULE_DEBUG_STAGE_DUMP_DIR")
        if not d:
            return None
        layer = os.environ.get("FERRULE_DEBUG_LAYER")
        return DebugTap(d, int(layer) if layer not in (None, "") else None, os.environ.get("FERRULE_DEBUG_STAGE") or None)

    def wants(self, layer: int, stage: str) -> bool:
        return (self.layer is None or self.layer == layer) and (self.stage is None or self.stage == stage)

    def next_step(self) -> None:
        self.step += 1

    def write(self, layer: int, stage: str, tensor: torch.Tensor) -> None:
        if not self.wants(layer, stage):
            return
        path = self.dir / f"step{self.step:05d}_layer{layer}_{stage}.pt"
        torch.save(tensor.detach().float().cpu(), path)
        self.written.append(str(path))


def prefill_progress_enabled() -> bool:
    return _flag("FERRULE_PREFILL_PROGRESS")
