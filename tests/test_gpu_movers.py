"""Data-mover kernels against plain PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fill_iota_pack_saxpy():
    from ferrule_b200.ops import movers as M
    t = torch.full((1000,), 7, dtype=torch.int32, device="cuda")
    assert int(M.fill_(t, 0).abs().sum()) == 0
    assert torch.equal(M.iota_(t, 5, 3).cpu(), torch.arange(1000, dtype=torch.int32) * 3 + 5)
    ids = torch.arange(17, dtype=torch.int32, device="cuda")
    vals = torch.randn(17, device="cuda")
    p = M.pack_pairs(ids, vals)
    assert torch.equal(p[:, 0], ids) and torch.equal(p[:, 1].view(torch.float32), vals)
    y, x = torch.randn(5000, device="cuda"), torch.randn(5000, device="cuda")
    want = y + 0.5 * x
    assert torch.allclose(M.saxpy_(y, x, 0.5), want, atol=1e-6)


def test_index_fills_match_torch():
    from ferrule_b200.ops import movers as M
    B, window, k, nmax = 5, 16, 12, 20
    pos = torch.tensor([0, 3, 15, 16, 40], dtype=torch.int32, device="cuda")
    base = torch.arange(B, device="cuda", dtype=torch.int64) * 1000
    sel = torch.full((B, window + k + nmax), -7, dtype=torch.int32, device="cuda")
    M.window_index_fill(sel, 0, window, pos, base)
    wpos = pos.long()[:, None] - torch.arange(window - 1, -1, -1, device="cuda")[None]
    assert torch.equal(sel[:, :window].long(), torch.where(wpos >= 0, base[:, None] + wpos, torch.full_like(wpos, -1)))
    idx = torch.randint(-1, 50, (B, k), dtype=torch.int32, device="cuda")
    M.offset_index_fill(sel, window, idx, base + 500)
    assert torch.equal(sel[:, window:window + k].long(),
                       torch.where(idx >= 0, base[:, None] + 500 + idx.long(), torch.full_like(idx, -1).long()))
    counts = torch.tensor([0, 1, 20, 7, 19], dtype=torch.int32, device="cuda")
    M.count_index_fill(sel, window + k, nmax, counts, base)
    j = torch.arange(nmax, device="cuda")[None]
    assert torch.equal(sel[:, window + k:].long(), torch.where(j < counts[:, None], base[:, None] + j, torch.full_like(j, -1)))


def test_row_moves_and_paged_scatter():
    from ferrule_b200.ops import _lib, movers as M
    src = torch.randn(40, 576, device="cuda").bfloat16()
    dst = torch.zeros(100, 576, dtype=torch.bfloat16, device="cuda")
    M.copy_rows(dst, 13, src)
    assert torch.equal(dst[13:53], src) and float(dst[:13].abs().sum()) == 0
    idx = torch.tensor([3, 39, 0, 3], dtype=torch.int32, device="cuda")
    out = torch.zeros(4, 576, dtype=torch.bfloat16, device="cuda")
    assert torch.equal(M.gather_rows(src, idx, out), src[idx.long()])
    acc = torch.zeros(6, 64, device="cuda")
    s = torch.randn(10, 64, device="cuda")
    ii = torch.tensor([0, 1, 1, 5, 5, 5, 2, 2, 0, 3], dtype=torch.int32, device="cuda")
    M.scatter_add_rows(acc, ii, s)
    assert torch.allclose(acc, torch.zeros(6, 64, device="cuda").index_add_(0, ii.long(), s), atol=1e-5)
    # paged scatter: 3 sequences, pages of 4 rows
    pool = torch.zeros(10 * 4, 64, dtype=torch.bfloat16, device="cuda")
    bt = torch.tensor([[2, 5, -1], [7, 1, 3], [0, -1, -1]], dtype=torch.int32, device="cuda")
    seq = torch.tensor([0, 1, 1, 2, 0], dtype=torch.int32, device="cuda")
    pos = torch.tensor([5, 0, 9, 3, -1], dtype=torch.int32, device="cuda")
    rows = torch.randn(5, 64, device="cuda").bfloat16()
    M.paged_row_scatter(pool, bt, seq, pos, rows, 4)
    torch.cuda.synchronize()
    assert torch.equal(pool[5 * 4 + 1], rows[0]) and torch.equal(pool[7 * 4], rows[1])
    assert torch.equal(pool[3 * 4 + 1], rows[2]) and torch.equal(pool[3], rows[3])
    assert int((pool.abs().sum(-1) > 0).sum()) == 4
    assert _lib.read_status()[0] == 0


def test_ring_to_logical_matches_host_resolver():
    from ferrule_b200.models.sparse_layout import CombinedRing
    from ferrule_b200.ops import movers as M
    window = 8
    ring = CombinedRing(window)
    last = [3, 8, 21]
    ncomp = [0, 2, 5]
    slots = torch.tensor([[0, 3, 4, 7, 8, 9], [0, 1, 7, 8, 9, 10], [5, 6, 0, 12, 13, 8]], dtype=torch.int32, device="cuda")
    idx, plane = M.ring_to_logical(slots, window, torch.tensor(last, dtype=torch.int32, device="cuda"),
                                   torch.tensor(ncomp, dtype=torch.int32, device="cuda"))
    for r in range(3):
        for j in range(6):
            s = int(slots[r, j])
            if s < window:
                p = ring.logical_of_slot(s, last[r])
                want = (p, 0) if p is not None else (-1, -1)
            else:
                c = s - window
                want = (c, 1) if c < ncomp[r] else (-1, -1)
            assert (int(idx[r, j]), int(plane[r, j])) == want, (r, j, s)
