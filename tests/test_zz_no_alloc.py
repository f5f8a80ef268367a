"""The allocation-free arg-max entry point, called through its exported C symbol.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.  The entry point serves callers that may not allocate device memory (fixed
memory budgets, no tolerance for cudaMalloc's device-wide synchronisation); its scratch is a fixed
array inside the library image, shared by all calls, so two calls in a row must not see each
other's leftovers.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ferrule_b200.ops import _lib
    lib = _lib.get_lib(required=True)
    fn = lib.fb_argmax_noalloc                      # the exported C symbol itself
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    return lib, fn


def _reference(K, logits):
    sc = K.ArgmaxScratch.allocate(logits.shape[0], "cuda")
    ids = torch.empty(logits.shape[0], dtype=torch.int32, device="cuda")
    vals = torch.empty(logits.shape[0], device="cuda")
    K.argmax_chunked(logits, sc, ids, vals)         # the existing entry point (caller-provided scratch)
    return ids, vals


def test_no_alloc_argmax_matches_existing_entry_point_twice():
    from ferrule_b200.ops import kernels as K
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device="cuda").manual_seed(123)
    # two calls in a row with different shapes: the second must not be disturbed by what the first
    # left in the shared scratch (more rows and chunks' worth of candidates, counters at 64)
    for call, (rows, vocab) in enumerate(((37, 102400), (5, 1000), (37, 102400))):
        logits = torch.randn(rows, vocab, generator=g, device="cuda")
        logits[0, 3] = logits[0, vocab - 1] = 77.0          # tie -> lower index
        logits[1] = float("nan")                            # no finite candidate -> -1
        ids = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        vals = torch.zeros(rows, device="cuda")
        # torch's counter only sees torch's own allocator; the driver's free-byte count (cudaMemGetInfo) also
        # sees a raw cudaMalloc.  The first call on a device resolves the scratch address (and may make the driver
        # load the module), so the driver-level comparison starts with the second call.
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(logits.data_ptr(), logits.stride(0), rows, vocab, ids.data_ptr(), vals.data_ptr(), stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() <= before      # (frees deferred by earlier tests may land meanwhile)
        if call > 0:
            assert torch.cuda.mem_get_info()[0] >= free_before
        ref_ids, ref_vals = _reference(K, logits)
        torch.cuda.synchronize()
        assert torch.equal(ids.cpu(), ref_ids.cpu())
        assert int(ids[0]) == 3 and int(ids[1]) == -1
        ok = ref_ids.cpu() >= 0
        assert torch.equal(vals.cpu()[ok], ref_vals.cpu()[ok])


def test_no_alloc_argmax_refuses_sizes_beyond_its_scratch():
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    rows = 257                                              # FB_NOALLOC_ARGMAX_MAX_ROWS is 256
    logits = torch.zeros(rows, 64, device="cuda")
    ids = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    rc = fn(logits.data_ptr(), logits.stride(0), rows, 64, ids.data_ptr(), None, stream)
    assert rc == 6                                          # FB_ERR_LIMIT
    torch.cuda.synchronize()
    assert int(ids.min()) == -7 and int(ids.max()) == -7    # nothing ran
    assert fn(None, 4, 1, 64, ids.data_ptr(), None, stream) == 1          # FB_ERR_SHAPE
