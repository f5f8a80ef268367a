"""Python face of the native positioned-read engine (csrc/host/direct_reader.cpp).

`NativeDirectReader.submit(source, dst, done)` has the interface the expert-streaming provider
expects: one request per tensor slice of the expert, `done(ok, bytes)` called from the poller
thread when all slices have landed.  Aligned requests bypass the page cache (O_DIRECT).
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Callable, Dict

import torch

from ..ops._lib import get_lib


def _declare(lib) -> None:
    vp, ull, i = C.c_void_p, C.c_ulonglong, C.c_int
    lib.fb_reader_create.argtypes, lib.fb_reader_create.restype = [i], vp
    lib.fb_reader_destroy.argtypes, lib.fb_reader_destroy.restype = [vp], None
    lib.fb_reader_submit.argtypes, lib.fb_reader_submit.restype = [vp, ull, C.c_char_p, ull, ull, vp], i
    lib.fb_reader_cancel.argtypes, lib.fb_reader_cancel.restype = [vp, ull], i
    lib.fb_reader_poll.argtypes = [vp, C.POINTER(ull), C.POINTER(C.c_longlong), i, i]
    lib.fb_reader_poll.restype = i
    lib.fb_reader_stats.argtypes, lib.fb_reader_stats.restype = [vp, C.POINTER(ull)], None


class NativeDirectReader:
    def __init__(self, threads: int = 4):
        lib = get_lib(required=True)
        _declare(lib)
        self.lib = lib
        self.h = lib.fb_reader_create(threads)
        self._next = 1
        self._lock = threading.Lock()
        self._groups: Dict[int, dict] = {}          # tag -> group record
        self._stop = False
        self._poller = threading.Thread(target=self._pump, name="ferrule-read-pump", daemon=True)
        self._poller.start()

    def read(self, path: str, offset: int, length: int, dst: torch.Tensor, done: Callable[[bool, int], None]) -> int:
        """One positioned read into `dst` (a host tensor that stays alive until `done`)."""
        with self._lock:
            tag = self._next
            self._next += 1
            self._groups[tag] = {"left": 1, "bytes": 0, "ok": True, "done": done, "want": length, "keep": dst}
        self.lib.fb_reader_submit(self.h, tag, path.encode(), offset, length, dst.data_ptr())
        return tag

    def submit(self, src, dst: torch.Tensor, done: Callable[[bool, int], None]) -> None:
        """All tensor slices of an expert source -> their payload offsets inside `dst`."""
        group = {"left": len(src.slices), "bytes": 0, "ok": True, "done": done, "want": None, "keep": dst,
                 "total": src.payload_bytes}
        base = dst.data_ptr()
        with self._lock:
            tags = []
            for s in src.slices:
                tag = self._next
                self._next += 1
                self._groups[tag] = dict(group=group, want=s.length)
                tags.append((tag, s))
        for tag, s in tags:
            self.lib.fb_reader_submit(self.h, tag, s.file.encode(), s.offset, s.length, C.c_void_p(base + s.payload_offset))

    def _pump(self) -> None:
        tags = (C.c_ulonglong * 64)()
        res = (C.c_longlong * 64)()
        while not self._stop:
            n = self.lib.fb_reader_poll(self.h, tags, res, 64, 50)
            for i in range(n):
                with self._lock:
                    rec = self._groups.pop(int(tags[i]), None)
                if rec is None:
                    continue
                g = rec.get("group", rec)
                want = rec["want"]
                r = int(res[i])
                g["ok"] &= (r == want)
                g["bytes"] += max(r, 0)
                g["left"] -= 1
                if g["left"] == 0:
                    total = g.get("total", g["bytes"])
                    g["done"](g["ok"], total if g["ok"] else g["bytes"])

    def stats(self) -> Dict[str, int]:
        out = (C.c_ulonglong * 5)()
        self.lib.fb_reader_stats(self.h, out)
        return dict(zip(("submitted", "completed", "bytes", "direct_reads", "queued"), (int(v) for v in out)))

    def close(self) -> None:
        self._stop = True
        self._poller.join(timeout=2)
        if self.h:
            self.lib.fb_reader_destroy(self.h)
            self.h = None
