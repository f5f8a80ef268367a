"""CompletionHub: one epoch counter and one waiter, for "something finished, run the owner loop".

Producers (I/O threads, CUDA host callbacks, HTTP handlers) call `notify()`.  The owner takes a
`listen()` ticket *before* it looks at its queues, does its work, and then `wait(ticket)` returns
at once if anything was notified in between, so no wake-up is lost between "looked" and "slept".
Works from threads (`wait`) and from asyncio (`wait_async`).

Counterpart of crates/ferrule-common/src/async_wake.rs:40-150.
"""
from __future__ import annotations

import asyncio
import threading
from typing import Optional


class CompletionHub:
    def __init__(self):
        self._cv = threading.Condition()
        self._epoch = 0
        self._loop: Optional[asyncio.AbstractEventLoop] = None
        self._async_event: Optional[asyncio.Event] = None
        self.notifications = 0

    def notify(self) -> None:
        with self._cv:
            self._epoch += 1
            self.notifications += 1
            self._cv.notify_all()
        loop, ev = self._loop, self._async_event
        if loop is not None and ev is not None:
            try:
                loop.call_soon_threadsafe(ev.set)
            except RuntimeError:
                pass            # loop already closed

    def listen(self) -> int:
        with self._cv:
            return self._epoch

    def wait(self, ticket: int, timeout: Optional[float] = None) -> bool:
        """True if notified since `ticket` (possibly before the call)."""
        with self._cv:
            return self._cv.wait_for(lambda: self._epoch != ticket, timeout)

    async def wait_async(self, ticket: int, timeout: Optional[float] = None) -> bool:
        if self._loop is None:
            self._loop = asyncio.get_running_loop()
            self._async_event = asyncio.Event()
        while True:
            with self._cv:
                if self._epoch != ticket:
                    return True
            self._async_event.clear()
            with self._cv:
                if self._epoch != ticket:
                    return True
            try:
                await asyncio.wait_for(self._async_event.wait(), timeout)
            except asyncio.TimeoutError:
                return False
