"""ctypes binding of libferrule_b200.so.

The library is loaded lazily.  On a machine with a CUDA device a missing or stale
library is an error (ops never fall back to PyTorch silently); on a CPU-only machine
`get_lib()` returns None and callers use the fp32 PyTorch reference path, which is
the oracle the CUDA kernels are tested against.

Mirrors the role of the reference's FFI layer between its device runtime and native
kernels (crates/ferrule-backend/src/cuda/kernels.rs:523-545, cutlass.rs:30-75).
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

from .. import _build

FB_OK = 0
_ERR_NAMES = {
    1: "FB_ERR_SHAPE (launcher rejected the arguments)",
    2: "FB_ERR_ALIGN (pointer or stride not 16-byte aligned)",
    3: "FB_ERR_DRIVER (driver entry point missing / tensor map encode failed)",
    4: "FB_ERR_LAUNCH (kernel launch failed)",
    5: "FB_ERR_RUNTIME (CUDA runtime error)",
    6: "FB_ERR_LIMIT (size beyond a fixed capacity)",
}


class NativeLibraryError(RuntimeError):
    pass


class GemmArgs(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("x", C.c_void_p), ("out", C.c_void_p),
        ("ldw", C.c_longlong), ("w_group_stride", C.c_longlong), ("ldx", C.c_longlong),
        ("ldo", C.c_longlong),
        ("n_out", C.c_int), ("k", C.c_int), ("groups", C.c_int), ("w_rows_per_group", C.c_int),
        ("x_rows", C.c_int), ("ntok", C.c_int), ("epilogue", C.c_int), ("dual_offset", C.c_int),
        ("out_fp32", C.c_int), ("max_tok_tiles", C.c_int), ("x_group_koff", C.c_int),
        ("out_group_coff", C.c_int), ("force_split", C.c_int),
        ("tile_group", C.c_void_p), ("tile_row0", C.c_void_p), ("tile_rows", C.c_void_p),
        ("num_tok_tiles", C.c_void_p), ("dst_row", C.c_void_p), ("row_scale", C.c_void_p),
        ("act_limit", C.c_float), ("rank", C.c_int), ("world", C.c_int), ("rows_cap", C.c_int),
        ("flag_capacity", C.c_int),
        ("peer_recv", C.c_void_p * 8), ("peer_flags", C.c_void_p * 8),
        ("local_ctr", C.c_void_p), ("residual", C.c_void_p), ("ldr", C.c_longlong),
        ("peer_wait_ns", C.c_ulonglong), ("status", C.c_void_p), ("trace", C.c_void_p),
        ("ar_payload_bf16", C.c_int),
        ("remap_rank", C.c_void_p), ("remap_row", C.c_void_p), ("mc_recv", C.c_void_p),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("kv", C.c_void_p), ("out", C.c_void_p),
        ("block_table", C.c_void_p), ("row_seq", C.c_void_p), ("row_pos", C.c_void_p),
        ("sink", C.c_void_p), ("part_o", C.c_void_p), ("part_ml", C.c_void_p),
        ("status", C.c_void_p),
        ("ldq", C.c_longlong), ("ldo", C.c_longlong), ("pool_rows", C.c_longlong),
        ("rows", C.c_int), ("heads", C.c_int), ("kv_lora", C.c_int), ("rope_dim", C.c_int),
        ("num_seqs", C.c_int), ("max_blocks", C.c_int), ("page_size", C.c_int),
        ("group_rows", C.c_int), ("splits", C.c_int), ("split_tokens", C.c_int),
        ("softmax_scale", C.c_float), ("merge_ctr", C.c_void_p),
        ("selection", C.c_void_p), ("sel_width", C.c_int), ("trace", C.c_void_p),
        ("decode_only", C.c_int),
    ]


class PrefillAttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("kv", C.c_void_p), ("out", C.c_void_p), ("tiles", C.c_void_p),
        ("block_table", C.c_void_p), ("sink", C.c_void_p), ("status", C.c_void_p),
        ("ldq", C.c_longlong), ("ldo", C.c_longlong), ("pool_rows", C.c_longlong),
        ("n_tiles", C.c_int), ("rows", C.c_int), ("heads", C.c_int), ("kv_lora", C.c_int), ("rope_dim", C.c_int),
        ("num_seqs", C.c_int), ("max_blocks", C.c_int), ("page_size", C.c_int), ("softmax_scale", C.c_float),
    ]


_lock = threading.Lock()
_lib: Optional[C.CDLL] = None
_tried = False


def _declare(lib: C.CDLL) -> None:
    vp, i, ll, f = C.c_void_p, C.c_int, C.c_longlong, C.c_float
    lib.fb_status_bytes.restype = i
    lib.fb_gemm_bf16.argtypes = [C.POINTER(GemmArgs), vp]
    lib.fb_mla_attention.argtypes = [C.POINTER(AttnArgs), vp]
    lib.fb_mla_prefill_tc.argtypes = [C.POINTER(PrefillAttnArgs), vp]
    lib.fb_mla_prefill_tc.restype = i
    lib.fb_embedding.argtypes = [vp, vp, vp, i, i, i, vp, vp]
    lib.fb_add_rmsnorm.argtypes = [vp, ll, vp, ll, vp, vp, ll, vp, ll, i, i, f, vp]
    lib.fb_mla_prep.argtypes = [vp, ll, i, vp, ll, i, i, i, vp, f, vp, vp, i, vp, vp, vp, ll, vp,
                                ll, i, vp, vp]
    lib.fb_router_topk.argtypes = [vp, ll, vp, vp, vp, i, i, i, i, i, i, i, f, vp, vp, vp]
    lib.fb_moe_plan.argtypes = [vp, vp, i, i, i, i, i, i, vp, vp, vp, vp, vp, vp, i, vp, vp, vp, vp]
    lib.fb_gather_rows.argtypes = [vp, ll, vp, vp, vp, ll, i, i, i, vp, vp]
    lib.fb_moe_reduce.argtypes = [vp, i, i, vp, i, i, vp, ll, vp, ll, vp, ll, i, i, i, vp]
    lib.fb_argmax.argtypes = [vp, ll, i, i, vp, vp, vp]
    lib.fb_topk_logits.argtypes = [vp, ll, i, i, i, vp, vp, vp]
    lib.fb_copy_pages.argtypes = [vp, ll, ll, vp, i, i, i, vp, vp]
    for name in ("fb_gemm_bf16", "fb_mla_attention", "fb_embedding", "fb_add_rmsnorm",
                 "fb_mla_prep", "fb_router_topk", "fb_moe_plan", "fb_gather_rows", "fb_moe_reduce",
                 "fb_argmax", "fb_topk_logits", "fb_copy_pages"):
        getattr(lib, name).restype = i
    # optional groups, declared by their own modules when present
    from . import _lib_ext
    _lib_ext.declare(lib)


def get_lib(required: Optional[bool] = None) -> Optional[C.CDLL]:
    """Return the loaded native library, building it if the tree has sources but no .so.

    required=None means "required iff a CUDA device is present".
    """
    global _lib, _tried
    if required is None:
        required = torch.cuda.is_available()
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if _tried and not required:
            return None
        _tried = True
        path = _build.LIB_PATH
        try:
            if not path.exists():
                if os.environ.get("FERRULE_NO_BUILD"):
                    raise NativeLibraryError(f"{path} is missing and FERRULE_NO_BUILD is set")
                _build.build()
            lib = C.CDLL(str(path))
            _declare(lib)
            _lib = lib
            return lib
        except Exception as exc:  # noqa: BLE001 - surfaced below
            if required:
                raise NativeLibraryError(
                    f"native library unavailable on a CUDA machine ({exc}); "
                    "run `python -m ferrule_b200._build`") from exc
            return None


def native_available() -> bool:
    return torch.cuda.is_available() and get_lib(required=False) is not None


LAUNCHES = [0]      # native kernel-launching calls that returned FB_OK (one launch each)


def check(rc: int, what: str) -> None:
    if rc != FB_OK:
        raise NativeLibraryError(f"{what}: {_ERR_NAMES.get(rc, rc)}")
    LAUNCHES[0] += 1


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ---------------------------------------------------------------------------
# device status word: one per device, checked by the engine between steps
# ---------------------------------------------------------------------------
_status = {}

_STATUS_NAMES = {1: "pipeline barrier timeout", 2: "peer flag timeout", 3: "index out of range",
                 4: "shape/capacity rejected on device"}


def status_tensor(device=None) -> torch.Tensor:
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.type == "cuda" and dev.index is None:          # "cuda" and "cuda:N" must name the same status word
        dev = torch.device("cuda", torch.cuda.current_device())
    t = _status.get(dev)
    if t is None:
        # words 0..3: status {code, site, detail0, detail1}; 4..5: ns spent waiting on peer flags; 6: waits that spun
        t = torch.zeros(8, dtype=torch.int32, device=dev)
        _status[dev] = t
    return t


def read_status(device=None, reset: bool = True):
    """Synchronising read of the status word -> (code, where, d0, d1)."""
    t = status_tensor(device)
    vals = [int(v) & 0xFFFFFFFF for v in t[:4].tolist()]
    if reset and vals[0] != 0:
        t[:4].zero_()
    return tuple(vals)


def read_peer_wait(device=None, reset: bool = True):
    """(nanoseconds kernels of this device spent spinning on peer flags, number of such waits) since the last reset."""
    t = status_tensor(device)
    w = [int(v) & 0xFFFFFFFF for v in t[4:7].tolist()]
    if reset:
        t[4:7].zero_()
    return (w[1] << 32) | w[0], w[2]


def raise_on_status(device=None) -> None:
    code, where, d0, d1 = read_status(device)
    if code != 0:
        raise NativeLibraryError(
            f"device status: {_STATUS_NAMES.get(code, code)} at site 0x{where:x} (detail {d0}, {d1})")
