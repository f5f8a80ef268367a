"""GGUF container reader for inspection: header, metadata key/values, tensor directory, and a decoder
for Q4_K blocks (the format most community checkpoints of small models use).  Nothing here feeds the
execution path: GGUF files are listed and summarised (`inspect-weightpack`), HuggingFace safetensors
are what the engine loads.

Layout (little endian): magic "GGUF", version u32, tensor count u64, kv count u64, then `kv count`
pairs (string key, u32 type, value), then `tensor count` records (string name, u32 n_dims, u64 dims[],
u32 ggml type, u64 offset); tensor data starts at the next multiple of `general.alignment` (32).

Counterpart of crates/ferrule-model/src/gguf/mod.rs:35-70 (metadata) and
crates/ferrule-model/src/quant/gguf_quant.rs:11-100 (Q4_K decode).
"""
from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Any, BinaryIO, Dict, List, Tuple

import numpy as np

from ..utils.errors import quant_type

_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
T_STRING, T_ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass(frozen=True)
class GgufTensorInfo:
    name: str
    shape: Tuple[int, ...]
    ggml_type: int
    offset: int                 # relative to the start of the data section

    @property
    def type_name(self) -> str:
        return quant_type(self.ggml_type).name


@dataclass
class GgufFile:
    version: int
    metadata: Dict[str, Any]
    tensors: List[GgufTensorInfo]
    data_offset: int

    def summary(self) -> Dict[str, Any]:
        by_type: Dict[str, int] = {}
        for t in self.tensors:
            by_type[t.type_name] = by_type.get(t.type_name, 0) + 1
        return {"version": self.version, "architecture": self.metadata.get("general.architecture"),
                "tensors": len(self.tensors), "tensor_types": by_type,
                "metadata_keys": len(self.metadata)}


def _read(f: BinaryIO, fmt: str):
    size = struct.calcsize(fmt)
    raw = f.read(size)
    if len(raw) != size:
        raise GgufError("unexpected end of file")
    return struct.unpack(fmt, raw)[0]


def _read_string(f: BinaryIO) -> str:
    n = _read(f, "<Q")
    if n > 1 << 24:
        raise GgufError("string length is implausible")
    raw = f.read(n)
    if len(raw) != n:
        raise GgufError("unexpected end of file")
    return raw.decode("utf-8", errors="replace")


def _read_value(f: BinaryIO, typ: int, depth: int = 0):
    if typ in _SCALARS:
        return _read(f, _SCALARS[typ])
    if typ == T_STRING:
        return _read_string(f)
    if typ == T_ARRAY:
        if depth > 2:
            raise GgufError("arrays nest too deep")
        inner = _read(f, "<I")
        n = _read(f, "<Q")
        if n > 1 << 26:
            raise GgufError("array length is implausible")
        return [_read_value(f, inner, depth + 1) for _ in range(n)]
    raise GgufError(f"unknown metadata value type {typ}")


def read_gguf(path: str) -> GgufFile:
    with open(path, "rb") as f:
        if f.read(4) != b"GGUF":
            raise GgufError("not a GGUF file (bad magic)")
        version = _read(f, "<I")
        if version not in (2, 3):
            raise GgufError(f"unsupported GGUF version {version}")
        n_tensors, n_kv = _read(f, "<Q"), _read(f, "<Q")
        if n_tensors > 1 << 20 or n_kv > 1 << 20:
            raise GgufError("header counts are implausible")
        meta: Dict[str, Any] = {}
        for _ in range(n_kv):
            key = _read_string(f)
            meta[key] = _read_value(f, _read(f, "<I"))
        tensors = []
        for _ in range(n_tensors):
            name = _read_string(f)
            nd = _read(f, "<I")
            if nd > 8:
                raise GgufError("tensor rank is implausible")
            dims = tuple(_read(f, "<Q") for _ in range(nd))
            typ, off = _read(f, "<I"), _read(f, "<Q")
            tensors.append(GgufTensorInfo(name, dims, typ, off))
        align = meta.get("general.alignment", 32)
        if isinstance(align, bool) or not isinstance(align, int) or not 1 <= align <= 1 << 20 or align & (align - 1):
            raise GgufError(f"general.alignment is not a power of two: {align!r}")
        pos = f.tell()
        return GgufFile(version, meta, tensors, (pos + align - 1) // align * align)


# ---------------------------------------------------------------------------------------- Q4_K
Q4K_BLOCK_BYTES, Q4K_BLOCK_ELEMS = 144, 256


def _q4k_scale_min(j: int, sc: np.ndarray) -> Tuple[int, int]:
    if j < 4:
        return int(sc[j] & 63), int(sc[j + 4] & 63)
    return int((sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4)), int((sc[j + 4] >> 4) | ((sc[j] >> 6) << 4))


def decode_q4_k(raw: bytes, n_elems: int) -> np.ndarray:
    """Q4_K super-blocks of 256 values: fp16 d, fp16 dmin, 12 bytes of packed 6-bit (scale, min) pairs for 8
    sub-blocks of 32, 128 bytes of 4-bit codes.  value = d * scale * q - dmin * min."""
    if n_elems % Q4K_BLOCK_ELEMS or len(raw) < n_elems // Q4K_BLOCK_ELEMS * Q4K_BLOCK_BYTES:
        raise GgufError("Q4_K payload size does not match the element count")
    out = np.empty(n_elems, dtype=np.float32)
    for b in range(n_elems // Q4K_BLOCK_ELEMS):
        blk = raw[b * Q4K_BLOCK_BYTES:(b + 1) * Q4K_BLOCK_BYTES]
        d, dmin = np.frombuffer(blk[:4], dtype=np.float16).astype(np.float32)
        sc = np.frombuffer(blk[4:16], dtype=np.uint8)
        qs = np.frombuffer(blk[16:], dtype=np.uint8)
        o = b * Q4K_BLOCK_ELEMS
        for pair in range(4):                       # 64 values per pair of sub-blocks share 32 bytes
            q = qs[pair * 32:(pair + 1) * 32]
            s1, m1 = _q4k_scale_min(2 * pair, sc)
            s2, m2 = _q4k_scale_min(2 * pair + 1, sc)
            out[o:o + 32] = d * s1 * (q & 0x0F) - dmin * m1
            out[o + 32:o + 64] = d * s2 * (q >> 4) - dmin * m2
            o += 64
    return out
