"""Model worker: one OS thread owns the engine; HTTP tasks talk to it through bounded queues.

* command queue (default 256 entries): submit / cancel / stats / shutdown; `submit` waits at most
  `admission_timeout_s` for a free entry;
* at most `commands_per_tick` commands are taken between two engine steps;
* every request has a bounded event queue (default 32); if the consumer falls that far behind or
  goes away, the request is cancelled cooperatively;
* a fatal engine error latches: every live request fails and new work is refused.

Counterpart of crates/ferrule-server/src/worker.rs:290-520 (spawn, loop), :524-760 (commands, terminal
drain, fatal latch) and config.rs:28-47.
"""
from __future__ import annotations

import asyncio
import logging
import queue
import threading
import time
import uuid
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

from ..runtime.engine import Engine, FinishEvent, TokenEvent
from ..runtime.session import FinishReason, GenerateRequest
from ..utils.async_wake import CompletionHub
from ..utils.observability import METRICS, REQUEST_LOG, log_event
from ..utils.tokenizer import IncrementalDecodeState

log = logging.getLogger("ferrule.worker")


@dataclass
class WorkerConfig:
    command_queue: int = 256
    event_queue: int = 32
    commands_per_tick: int = 64
    admission_timeout_s: float = 30.0
    idle_wait_s: float = 0.05


class WorkerError(RuntimeError):
    def __init__(self, message: str, status: int = 500, code: str = "internal_error"):
        super().__init__(message)
        self.status, self.code = status, code


@dataclass
class StreamEvent:
    kind: str                    # "token" | "finish" | "error"
    text: str = ""
    token: int = -1
    reason: Optional[FinishReason] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
    message: str = ""


class RequestStream:
    """Consumer side of one request's event queue (bound to the consumer's asyncio loop)."""

    def __init__(self, request_id: str, loop: asyncio.AbstractEventLoop, capacity: int, worker: "ModelWorker"):
        self.request_id, self.loop, self.capacity, self.worker = request_id, loop, capacity, worker
        self.q: asyncio.Queue = asyncio.Queue()
        self._pending = 0
        self._lock = threading.Lock()
        self.closed = False
        self.prompt_tokens = 0

    # worker thread
    def offer(self, ev: StreamEvent) -> bool:
        with self._lock:
            if self.closed:
                return False
            if self._pending >= self.capacity and ev.kind == "token":
                return False                      # consumer too slow: caller cancels the request
            self._pending += 1
        try:
            self.loop.call_soon_threadsafe(self.q.put_nowait, ev)
        except RuntimeError:
            return False                          # loop is gone
        return True

    # consumer task
    async def next(self) -> StreamEvent:
        ev = await self.q.get()
        with self._lock:
            self._pending -= 1
        return ev

    def close(self) -> None:
        """Consumer went away (disconnect): the worker cancels the request."""
        with self._lock:
            if self.closed:
                return
            self.closed = True
        self.worker.cancel(self.request_id)


@dataclass
class _Live:
    stream: RequestStream
    decoder: IncrementalDecodeState
    t_submit: float
    tokens: int = 0
    done: bool = False


class ModelWorker:
    def __init__(self, engine_factory: Callable[[], Engine], tokenizer, cfg: Optional[WorkerConfig] = None,
                 model_name: str = "ferrule", mirror=None):
        """`mirror` (parallel.mirror.CommandMirror, leader side): this worker's engine is one rank of a replica
        spread over several ranks; every command it applies and every step it takes is published to the others,
        and nothing changes the engine outside that stream (a slow consumer's cancel is queued, not applied)."""
        self.cfg = cfg or WorkerConfig()
        self.mirror = mirror
        self._tick_log: List[tuple] = []
        self._deferred_cancels: List[str] = []
        self.tokenizer, self.model_name = tokenizer, model_name
        self._factory = engine_factory
        self.engine: Optional[Engine] = None
        self.hub = CompletionHub()
        self._cmds: "queue.Queue" = queue.Queue(maxsize=self.cfg.command_queue)
        self._live: Dict[str, _Live] = {}
        self._fatal: Optional[str] = None
        self._ready = threading.Event()
        self._stopped = threading.Event()
        self._thread = threading.Thread(target=self._run, name="ferrule-model-worker", daemon=True)
        self.steps = 0

    # ------------------------------------------------------------------ lifecycle
    def start(self, timeout: float = 600.0) -> "ModelWorker":
        self._thread.start()
        if not self._ready.wait(timeout):
            raise WorkerError("model worker did not become ready")
        if self._fatal:
            raise WorkerError(self._fatal)
        return self

    def stop(self, timeout: float = 30.0) -> None:
        try:
            self._cmds.put(("shutdown",), timeout=1.0)
        except queue.Full:
            pass
        self.hub.notify()
        self._stopped.wait(timeout)

    @property
    def healthy(self) -> bool:
        return self._ready.is_set() and self._fatal is None and not self._stopped.is_set()

    # ------------------------------------------------------------------ API for HTTP tasks
    async def submit(self, *, text: Optional[str], token_ids: Optional[List[int]], max_tokens: int, stop: List[str],
                     ignore_eos: bool = False, session_id: Optional[str] = None,
                     request_id: Optional[str] = None) -> RequestStream:
        if self._fatal:
            raise WorkerError(f"model worker failed: {self._fatal}", 503, "worker_failed")
        if self._stopped.is_set():
            raise WorkerError("model worker is stopped", 503, "worker_stopped")
        rid = request_id or uuid.uuid4().hex
        stream = RequestStream(rid, asyncio.get_running_loop(), self.cfg.event_queue, self)
        reply: asyncio.Future = asyncio.get_running_loop().create_future()
        cmd = ("submit", rid, text, token_ids, max_tokens, stop, ignore_eos, session_id, stream, reply)
        deadline = time.monotonic() + self.cfg.admission_timeout_s
        while True:
            try:
                self._cmds.put_nowait(cmd)
                break
            except queue.Full:
                if time.monotonic() > deadline:
                    raise WorkerError("server is overloaded: admission timed out", 503, "admission_timeout")
                await asyncio.sleep(0.005)
        self.hub.notify()
        try:
            n_prompt = await asyncio.wait_for(reply, self.cfg.admission_timeout_s)
        except asyncio.TimeoutError:
            stream.close()
            raise WorkerError("server is overloaded: admission timed out", 503, "admission_timeout")
        stream.prompt_tokens = n_prompt
        return stream

    def cancel(self, request_id: str) -> None:
        try:
            self._cmds.put_nowait(("cancel", request_id))
        except queue.Full:
            pass            # the disconnect guard will be noticed at the next event offer
        self.hub.notify()

    def tokenize(self, text: str) -> List[int]:
        return self.tokenizer.encode(text)

    def stats(self) -> Dict[str, Any]:
        e = self.engine
        return {"healthy": self.healthy, "live_requests": len(self._live), "steps": self.steps,
                "engine": e.snapshot_stats() if e is not None else None}

    # ------------------------------------------------------------------ worker thread
    def _reply(self, fut: asyncio.Future, stream: RequestStream, value=None, exc: Optional[BaseException] = None) -> None:
        def setter():
            if fut.done():
                return
            if exc is not None:
                fut.set_exception(exc)
            else:
                fut.set_result(value)
        try:
            stream.loop.call_soon_threadsafe(setter)
        except RuntimeError:
            pass

    def _handle(self, cmd) -> bool:
        op = cmd[0]
        if op == "shutdown":
            return False
        if op == "cancel":
            lv = self._live.get(cmd[1])
            if lv is not None and not lv.done:
                self.engine.cancel_request(cmd[1])
                self._tick_log.append(("cancel", cmd[1]))
            return True
        _, rid, text, token_ids, max_tokens, stop, ignore_eos, session_id, stream, reply = cmd
        try:
            ids = list(token_ids) if token_ids is not None else self.tokenizer.encode(text or "")
            if not ids:
                raise WorkerError("prompt is empty", 400, "empty_prompt")
            if any((t < 0 or t >= self.engine.runner.vocab_size) for t in ids):
                raise WorkerError("prompt holds a token id outside the vocabulary", 400, "bad_token")
            self.engine.submit(GenerateRequest(rid, ids, max_new_tokens=max_tokens, stop=stop, ignore_eos=ignore_eos,
                                               session_id=session_id, retain_session=session_id is not None))
        except WorkerError as e:
            self._reply(reply, stream, exc=e)
            return True
        except ValueError as e:
            self._reply(reply, stream, exc=WorkerError(str(e), 400, "invalid_request"))
            return True
        except Exception as e:  # noqa: BLE001 - the caller must get an answer and the worker must live on
            self._reply(reply, stream, exc=WorkerError(f"internal error: {type(e).__name__}: {e}", 500,
                                                       "internal_error"))
            return True
        self._tick_log.append(("submit", rid, ids, max_tokens, list(stop or []), ignore_eos, session_id))
        self._live[rid] = _Live(stream, IncrementalDecodeState(self.tokenizer), time.monotonic())
        METRICS.add(requests_started=1, prompt_tokens=len(ids))
        log_event(REQUEST_LOG, "admitted", request_id=rid, prompt_tokens=len(ids), max_tokens=max_tokens)
        self._reply(reply, stream, value=len(ids))
        return True

    def _emit(self, ev) -> None:
        lv = self._live.get(ev.request_id)
        if lv is None:
            return
        if isinstance(ev, TokenEvent):
            delta = ev.text if self.engine.detokenize is not None else lv.decoder.push(ev.token)
            lv.tokens += 1
            METRICS.add(generated_tokens=1)
            if not lv.stream.offer(StreamEvent("token", text=delta, token=ev.token)):
                # slow or vanished consumer
                if self.mirror is None:
                    self.engine.cancel_request(ev.request_id)
                else:                                            # through the command stream, so every rank sees it
                    try:
                        self._cmds.put_nowait(("cancel", ev.request_id))
                    except queue.Full:
                        self._deferred_cancels.append(ev.request_id)
        elif isinstance(ev, FinishEvent):
            lv.done = True
            tail = ev.tail if self.engine.detokenize is not None else lv.decoder.finish()
            if tail:
                lv.stream.offer(StreamEvent("token", text=tail))
            lv.stream.offer(StreamEvent("finish", reason=ev.reason, prompt_tokens=ev.prompt_tokens,
                                        completion_tokens=ev.generated_tokens))
            del self._live[ev.request_id]
            if ev.reason == FinishReason.CANCELLED:
                METRICS.add(requests_cancelled=1)
            elif ev.reason == FinishReason.ERROR:
                METRICS.add(requests_failed=1)
            else:
                METRICS.add(requests_finished=1, ttft_sum_s=ev.ttft_s, tpot_sum_s=ev.tpot_s,
                            e2e_sum_s=time.monotonic() - lv.t_submit)
            log_event(REQUEST_LOG, "terminal", request_id=ev.request_id, reason=ev.reason.value,
                      generated=ev.generated_tokens)

    def _fail_all(self, message: str) -> None:
        self._fatal = message
        for rid, lv in list(self._live.items()):
            lv.stream.offer(StreamEvent("error", message=message))
        self._live.clear()

    def _run(self) -> None:
        try:
            self.engine = self._factory()
            if self.engine.detokenize is None:
                # the engine needs text for stop strings; deltas then come from the engine itself
                self.engine.detokenize = self.tokenizer.decode
        except BaseException as exc:  # noqa: BLE001 - reported through start()
            self._fatal = f"engine construction failed: {exc}"
            self._ready.set()
            self._stopped.set()
            return
        self._ready.set()
        running = True
        while running:
            ticket = self.hub.listen()
            took = 0
            while took < self.cfg.commands_per_tick:
                try:
                    cmd = self._cmds.get_nowait()
                except queue.Empty:
                    break
                took += 1
                if not self._handle(cmd):
                    running = False
                    break
            if not running:
                break
            while self._deferred_cancels:
                self._handle(("cancel", self._deferred_cancels.pop()))
            progressed = False
            stepping = self._fatal is None
            if self.mirror is not None:
                # followers step exactly when the leader does: skip the idle polls, publish the rest
                stepping = stepping and (bool(self._tick_log) or self.engine.has_work())
                if stepping:
                    self.mirror.publish(self._tick_log)
            self._tick_log = []
            if stepping:
                try:
                    progressed = self.engine.step(self._emit)
                    self.steps += 1
                except BaseException as exc:  # noqa: BLE001 - latch: the engine state is unknown now
                    log.exception("engine step failed")
                    self._fail_all(f"engine failure: {exc}")
            METRICS.set(queue_depth=len(self.engine.scheduler.waiting))
            if not progressed and took == 0 and not self.engine.has_work():
                self.hub.wait(ticket, self.cfg.idle_wait_s)
        # drain: cancel everything, let transactions end
        if self.mirror is not None:
            try:
                self.mirror.shutdown()
            except Exception:  # noqa: BLE001 - the other ranks may be gone already
                log.exception("mirror shutdown failed")
        try:
            for _ in range(1000):
                if self.engine.shutdown():
                    break
            for rid, lv in list(self._live.items()):
                lv.stream.offer(StreamEvent("finish", reason=FinishReason.CANCELLED))
        finally:
            self._stopped.set()
