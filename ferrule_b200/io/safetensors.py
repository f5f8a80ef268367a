"""safetensors files and HuggingFace sharded checkpoints (`model.safetensors.index.json`).

File layout: 8-byte little-endian header length, JSON header `{name: {dtype, shape, data_offsets}}`
(+ optional `__metadata__`), then the raw tensor bytes; data offsets are relative to the end of the
header.  Dtypes handled: F32, BF16, F16, F8_E4M3, F8_E8M0 (kept as uint8), I8 (packed FP4), U8,
I32, I64.  Reads are bounded (`max_bytes`) and go through mmap, so a checkpoint larger than host
memory can still be bound and sliced.

Counterpart of crates/ferrule-model/src/gguf/safetensors.rs:19-240, checkpoint/tensor.rs:16-64,
checkpoint/source.rs:24-170 and read_plan.rs:19-170 in the reference.
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_DTYPES = {
    "F32": (torch.float32, 4), "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2),
    "F8_E4M3": (torch.uint8, 1), "F8_E8M0": (torch.uint8, 1), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}
_REV = {torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.int8: "I8", torch.uint8: "U8",
        torch.int32: "I32", torch.int64: "I64", torch.bool: "BOOL"}


def fails_closed(fn):
    """Loader entry points answer a damaged checkpoint (missing tensors, a config with impossible values, shapes
    that do not fit) with CheckpointError, whatever the first symptom was."""
    import functools

    @functools.wraps(fn)
    def wrapper(*args, **kw):
        try:
            return fn(*args, **kw)
        except CheckpointError:
            raise
        except (KeyError, TypeError, ValueError, RuntimeError, AttributeError, IndexError, ZeroDivisionError, OSError) as exc:
            raise CheckpointError(f"{fn.__name__}: the checkpoint does not fit the model it describes "
                                  f"({type(exc).__name__}: {exc})") from exc
    return wrapper


class CheckpointError(RuntimeError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    start: int          # absolute byte offset in the file
    end: int
    file: str

    @property
    def nbytes(self) -> int:
        return self.end - self.start

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsFile:
    def __init__(self, path):
        self.path = str(path)
        self._f = open(self.path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise CheckpointError(f"{path}: too small to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise CheckpointError(f"{path}: header length {hlen} is out of range")
        try:
            header = json.loads(self._f.read(hlen))
        except ValueError as exc:
            raise CheckpointError(f"{path}: header is not JSON") from exc
        if not isinstance(header, dict):
            raise CheckpointError(f"{path}: header is not a JSON object")
        self.metadata = header.pop("__metadata__", {})
        base = 8 + hlen
        self.tensors: Dict[str, TensorInfo] = {}
        for name, d in header.items():
            # every field is checked before use: a damaged header is a CheckpointError, never a stray exception
            if not isinstance(d, dict) or not {"dtype", "shape", "data_offsets"} <= set(d):
                raise CheckpointError(f"{path}: tensor {name} lacks dtype / shape / data_offsets")
            if not isinstance(d["dtype"], str) or d["dtype"] not in _DTYPES:
                raise CheckpointError(f"{path}: tensor {name} has unsupported dtype {d['dtype']!r}")
            shape, offs = d["shape"], d["data_offsets"]
            if not (isinstance(shape, list) and all(isinstance(x, int) and not isinstance(x, bool) and x >= 0 for x in shape)):
                raise CheckpointError(f"{path}: tensor {name} has a malformed shape {shape!r}")
            if not (isinstance(offs, list) and len(offs) == 2
                    and all(isinstance(x, int) and not isinstance(x, bool) and x >= 0 for x in offs)):
                raise CheckpointError(f"{path}: tensor {name} has malformed data_offsets {offs!r}")
            s, e = offs
            info = TensorInfo(name, d["dtype"], tuple(shape), base + s, base + e, self.path)
            if info.end > size or s > e:
                raise CheckpointError(f"{path}: tensor {name} reaches past the end of the file")
            if info.numel * _DTYPES[info.dtype][1] != info.nbytes:
                raise CheckpointError(f"{path}: tensor {name} byte size does not match its shape")
            self.tensors[name] = info
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self.tensors)

    def read(self, name: str, max_bytes: Optional[int] = None) -> torch.Tensor:
        info = self.tensors.get(name)
        if info is None:
            raise CheckpointError(f"{self.path}: no tensor {name}")
        if max_bytes is not None and info.nbytes > max_bytes:
            raise CheckpointError(f"tensor {name} has {info.nbytes} bytes, limit is {max_bytes}")
        dt, _ = _DTYPES[info.dtype]
        buf = bytearray(self._mm[info.start:info.end])
        if not buf:
            return torch.empty(info.shape, dtype=dt)
        return torch.frombuffer(buf, dtype=dt).reshape(info.shape)

    def read_rows(self, name: str, row_lo: int, row_hi: int) -> torch.Tensor:
        """Bounded slice along dim 0 without touching the rest of the tensor."""
        info = self.tensors[name]
        dt, es = _DTYPES[info.dtype]
        row_bytes = (info.numel // max(info.shape[0], 1)) * es
        buf = bytearray(self._mm[info.start + row_lo * row_bytes:info.start + row_hi * row_bytes])
        return torch.frombuffer(buf, dtype=dt).reshape((row_hi - row_lo,) + info.shape[1:])

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path, dtype_names: Optional[Dict[str, str]] = None,
              metadata: Optional[Dict[str, str]] = None) -> None:
    """Write a safetensors file.  `dtype_names` overrides the header dtype of byte tensors
    (e.g. "F8_E4M3" / "F8_E8M0" for uint8 payloads)."""
    header, chunks, off = {}, [], 0
    for name in sorted(tensors):
        t = tensors[name].contiguous().cpu()
        dname = (dtype_names or {}).get(name) or _REV.get(t.dtype)
        if dname is None:
            raise CheckpointError(f"cannot store dtype {t.dtype}")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        pad = (-len(raw)) % 8
        header[name] = {"dtype": dname, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        chunks.append(raw + b"\0" * pad)
        off += len(raw) + pad
    if metadata:
        header["__metadata__"] = metadata
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((-len(hj)) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for c in chunks:
            f.write(c)


class ShardedCheckpoint:
    """HF directory: config.json + model.safetensors.index.json (weight_map) + shards."""

    def __init__(self, directory):
        self.dir = Path(directory)
        idx = self.dir / "model.safetensors.index.json"
        if idx.exists():
            self.weight_map: Dict[str, str] = json.loads(idx.read_text())["weight_map"]
        else:
            single = sorted(self.dir.glob("*.safetensors"))
            if not single:
                raise CheckpointError(f"{directory}: no safetensors files")
            self.weight_map = {}
            for p in single:
                f = SafetensorsFile(p)
                for n in f.names():
                    self.weight_map[n] = p.name
                f.close()
        self._files: Dict[str, SafetensorsFile] = {}

    def _file(self, shard: str) -> SafetensorsFile:
        f = self._files.get(shard)
        if f is None:
            f = self._files[shard] = SafetensorsFile(self.dir / shard)
        return f

    def names(self) -> List[str]:
        return list(self.weight_map)

    def has(self, name: str) -> bool:
        return name in self.weight_map

    def info(self, name: str) -> TensorInfo:
        return self._file(self.weight_map[name]).tensors[name]

    def read(self, name: str, max_bytes: Optional[int] = None) -> torch.Tensor:
        if name not in self.weight_map:
            raise CheckpointError(f"tensor {name} is not in the checkpoint")
        return self._file(self.weight_map[name]).read(name, max_bytes)

    def source_identity(self) -> bytes:
        """Hash of (file name, size, mtime) of every shard: changes when the checkpoint on disk does."""
        h = hashlib.sha256()
        for shard in sorted(set(self.weight_map.values())):
            st = os.stat(self.dir / shard)
            h.update(f"{shard}:{st.st_size}:{int(st.st_mtime_ns)}".encode())
        return h.digest()

    def content_hash(self, names: Iterable[str]) -> bytes:
        """Hash over the identities (file, offsets, dtype, shape) of the tensors forming one payload."""
        h = hashlib.sha256()
        for n in names:
            i = self.info(n)
            h.update(f"{n}|{Path(i.file).name}|{i.start}|{i.end}|{i.dtype}|{i.shape}".encode())
        return h.digest()

    def read_plan(self, names: Iterable[str], gap: int = 1 << 16, align: int = 4096) -> List[Tuple[str, int, int]]:
        """Coalesced positioned reads (file, offset, length) covering the tensors; ranges closer than
        `gap` bytes merge, and every range is widened to `align` for direct I/O."""
        per_file: Dict[str, List[Tuple[int, int]]] = {}
        for n in names:
            i = self.info(n)
            per_file.setdefault(i.file, []).append((i.start, i.end))
        plan = []
        for file, spans in per_file.items():
            spans.sort()
            cur_s, cur_e = spans[0]
            for s, e in spans[1:]:
                if s - cur_e <= gap:
                    cur_e = max(cur_e, e)
                else:
                    plan.append((file, cur_s, cur_e))
                    cur_s, cur_e = s, e
            plan.append((file, cur_s, cur_e))
        out = []
        for file, s, e in plan:
            s2 = s // align * align
            e2 = (e + align - 1) // align * align
            out.append((file, s2, e2 - s2))
        return out

    def close(self) -> None:
        for f in self._files.values():
            f.close()
        self._files.clear()


def write_sharded(tensors: Dict[str, torch.Tensor], directory, shard_bytes: int = 1 << 30,
                  dtype_names: Optional[Dict[str, str]] = None) -> None:
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    for n in sorted(tensors):
        nb = tensors[n].numel() * tensors[n].element_size()
        if size and size + nb > shard_bytes:
            shards.append({})
            size = 0
        shards[-1][n] = tensors[n]
        size += nb
    weight_map = {}
    total = 0
    for i, sh in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(sh, d / fname, dtype_names)
        for n, t in sh.items():
            weight_map[n] = fname
            total += t.numel() * t.element_size()
    (d / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}, indent=1))
