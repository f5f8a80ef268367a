"""Logging, global metrics and periodic metric dumps.

`init_tracing()` configures the `ferrule` loggers from the environment (`FERRULE_LOG` = level or
`target=level,...` list, `FERRULE_LOG_FORMAT=json` for one JSON object per line).  `METRICS` is the
process-wide counter set (prompt / generated tokens, request counts, TTFT / TPOT / end-to-end /
queue-time sums, prefix-cache hits, queue depth, preemptions, GPU memory);
`start_periodic_dump()` logs a snapshot every `FERRULE_METRICS_INTERVAL` seconds on the
`ferrule_metrics` target.

Counterpart of crates/ferrule-common/src/observability.rs:19-48 (tracing), :54-95 (metrics),
:204-226 (periodic dump).
"""
from __future__ import annotations

import json
import logging
import os
import threading
from dataclasses import dataclass, field
from typing import Dict, Optional

REQUEST_LOG = logging.getLogger("ferrule_request")
SPEC_LOG = logging.getLogger("ferrule_speculative_cycle")
METRICS_LOG = logging.getLogger("ferrule_metrics")


class _JsonFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        d = {"ts": round(record.created, 6), "level": record.levelname, "target": record.name,
             "message": record.getMessage()}
        extra = getattr(record, "fields", None)
        if isinstance(extra, dict):
            d.update(extra)
        return json.dumps(d, separators=(",", ":"))


def init_tracing(spec: Optional[str] = None, fmt: Optional[str] = None) -> None:
    spec = spec if spec is not None else os.environ.get("FERRULE_LOG", "warning")
    fmt = fmt if fmt is not None else os.environ.get("FERRULE_LOG_FORMAT", "text")
    handler = logging.StreamHandler()
    handler.setFormatter(_JsonFormatter() if fmt == "json" else logging.Formatter(
        "%(asctime)s %(levelname)s %(name)s: %(message)s"))
    root = logging.getLogger("ferrule")
    for h in list(root.handlers):
        root.removeHandler(h)
    default = "WARNING"
    for part in [p for p in spec.split(",") if p]:
        if "=" in part:
            target, lvl = part.split("=", 1)
            lg = logging.getLogger(target)
            lg.setLevel(lvl.upper())
            if not lg.handlers:
                lg.addHandler(handler)
            lg.propagate = False
        else:
            default = part.upper()
    root.addHandler(handler)
    root.setLevel(default)
    for lg in (REQUEST_LOG, SPEC_LOG, METRICS_LOG):
        if not lg.handlers:
            lg.addHandler(handler)
            lg.setLevel(default)
            lg.propagate = False


def log_event(logger: logging.Logger, message: str, **fields) -> None:
    logger.info(message, extra={"fields": fields})


@dataclass
class Metrics:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    requests_started: int = 0
    requests_finished: int = 0
    requests_failed: int = 0
    requests_cancelled: int = 0
    ttft_sum_s: float = 0.0
    tpot_sum_s: float = 0.0
    e2e_sum_s: float = 0.0
    queue_sum_s: float = 0.0
    cache_hits: int = 0
    cache_misses: int = 0
    prefix_hit_tokens: int = 0
    queue_depth: int = 0
    preemptions: int = 0
    gpu_mem_bytes: int = 0
    _lock: threading.Lock = field(default_factory=threading.Lock, repr=False, compare=False)

    def add(self, **kw) -> None:
        with self._lock:
            for k, v in kw.items():
                setattr(self, k, getattr(self, k) + v)

    def set(self, **kw) -> None:
        with self._lock:
            for k, v in kw.items():
                setattr(self, k, v)

    def snapshot(self) -> Dict[str, float]:
        with self._lock:
            d = {k: v for k, v in vars(self).items() if not k.startswith("_")}
        n = max(d["requests_finished"], 1)
        d["ttft_mean_s"] = d["ttft_sum_s"] / n
        d["tpot_mean_s"] = d["tpot_sum_s"] / n
        return d

    def reset(self) -> None:
        with self._lock:
            for k, v in vars(self).items():
                if not k.startswith("_"):
                    setattr(self, k, type(v)())


METRICS = Metrics()
_dump_thread: Optional[threading.Thread] = None
_dump_stop = threading.Event()


def start_periodic_dump(interval_s: Optional[float] = None) -> bool:
    global _dump_thread
    if interval_s is None:
        env = os.environ.get("FERRULE_METRICS_INTERVAL")
        interval_s = float(env) if env else 0.0
    if interval_s <= 0 or _dump_thread is not None:
        return False
    _dump_stop.clear()

    def loop():
        while not _dump_stop.wait(interval_s):
            log_event(METRICS_LOG, "metrics", **METRICS.snapshot())

    _dump_thread = threading.Thread(target=loop, name="ferrule-metrics", daemon=True)
    _dump_thread.start()
    return True


def stop_periodic_dump() -> None:
    global _dump_thread
    _dump_stop.set()
    if _dump_thread is not None:
        _dump_thread.join(timeout=2)
        _dump_thread = None
