"""Numerics of every CUDA kernel against the plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

from ferrule_b200.ops import reference as ref

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from ferrule_b200.ops import kernels
    return kernels


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    if torch.cuda.is_available():
        from ferrule_b200.ops import _lib
        torch.cuda.synchronize()
        code = _lib.read_status()
        assert code[0] == 0, f"device status word set: {code}"


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    assert not bad.any(), f"{int(bad.sum())}/{bad.numel()} mismatches, max err {float(err.max()):.4g}, ref max {float(b.abs().max()):.4g}"


@pytest.mark.parametrize("rows,n,k", [(1, 128, 64), (7, 128, 512), (32, 576, 2048), (32, 2048, 1408),
                                      (100, 3648, 2048), (300, 2048, 2048), (16, 64, 2048),
                                      (700, 1000, 1024)])
def test_gemm_dense(K, rows, n, k):
    x, w = rnd(rows, k), rnd(n, k, scale=0.05)
    out = K.gemm(x, w)
    close(out, x.float() @ w.float().T)


@pytest.mark.parametrize("split", [1, 2, 4, 8])
@pytest.mark.parametrize("rows,n,k", [(32, 2048, 2048), (5, 576, 1024), (32, 128, 1408)])
def test_gemm_split_k_cluster(K, split, rows, n, k):
    """Split-K over a thread-block cluster (DSMEM reduction) gives the same result for every factor."""
    x, w = rnd(rows, k), rnd(n, k, scale=0.05)
    out = K.gemm(x, w, split_k=split)
    close(out, x.float() @ w.float().T)
    # the SwiGLU variant keeps two accumulators per peer in the leader's shared memory: only run the
    # factors whose reduction area fits beside a two-stage pipeline
    ntok = K.pick_ntok(rows, dual=True)
    red_bytes = (split - 1) * 2 * ntok * 512
    stage_bytes = 2 * 16384 + ntok * 128
    if red_bytes + 2 * stage_bytes + 2048 <= 227 * 1024:
        w13 = rnd(2 * 256, k, scale=0.05)
        out2 = K.gemm(x, w13, epilogue=K.EPI_SWIGLU, split_k=split)
        y = x.float() @ w13.float().T
        close(out2, ref.swiglu(y[:, :256], y[:, 256:]))


def test_gemm_fp32_out_and_strided_x(K):
    big = rnd(40, 4096)
    x = big[:, 1024:3072]           # row stride 4096, 16-byte aligned start
    w = rnd(64, 2048, scale=0.05)
    out = K.gemm(x, w, out_dtype=torch.float32)
    assert out.dtype == torch.float32
    close(out, x.float() @ w.float().T, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("rows,inter,k", [(32, 1408, 2048), (5, 256, 512), (200, 352, 2048)])
def test_gemm_swiglu_dense(K, rows, inter, k):
    x, w13 = rnd(rows, k), rnd(2 * inter, k, scale=0.05)
    out = K.gemm(x, w13, epilogue=K.EPI_SWIGLU)
    y = x.float() @ w13.float().T
    close(out, ref.swiglu(y[:, :inter], y[:, inter:]))


def test_gemm_swiglu_clamp(K):
    x, w13 = rnd(8, 512, scale=2.0), rnd(256, 512, scale=0.3)
    out = K.gemm(x, w13, epilogue=K.EPI_SWIGLU, act_limit=7.0)
    y = x.float() @ w13.float().T
    close(out, ref.swiglu(y[:, :128], y[:, 128:], limit=7.0))


def test_gemm_batched_heads(K):
    heads, nope, lat, rows = 16, 128, 512, 33
    q = rnd(rows, heads * 192)
    w = rnd(heads, lat, nope, scale=0.05)
    out = torch.zeros(rows, heads * 576, dtype=torch.bfloat16, device="cuda")
    K.gemm(q, w, out=out, x_group_koff=192, out_group_coff=576)
    qv = q.view(rows, heads, 192)[:, :, :nope].float()
    expect = torch.einsum("rhk,hnk->rhn", qv, w.float())
    close(out.view(rows, heads, 576)[:, :, :lat], expect)
    assert float(out.view(rows, heads, 576)[:, :, lat:].abs().max()) == 0.0


def _route_setup(K, T, E, topk, e_lo, e_hi, ntok, seed=1):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn(T, E, generator=g, device="cuda")
    idx, w = ref.route(logits, topk, ref.SCORE_SOFTMAX)
    plan = K.MoePlan.allocate(T * topk, e_hi - e_lo, ntok, "cuda")
    K.moe_plan(idx, w, plan, e_lo, e_hi)
    return idx, w, plan


@pytest.mark.parametrize("T,E,topk,e_lo,e_hi,ntok", [(32, 64, 6, 0, 64, 32), (32, 64, 6, 8, 16, 16),
                                                      (257, 16, 2, 0, 16, 64), (4, 8, 2, 0, 8, 16),
                                                      (2048, 64, 6, 0, 64, 128), (1500, 64, 6, 16, 48, 64)])
def test_moe_plan(K, T, E, topk, e_lo, e_hi, ntok):
    idx, w, plan = _route_setup(K, T, E, topk, e_lo, e_hi, ntok)
    torch.cuda.synchronize()
    flat = idx.flatten().cpu()
    local = (flat >= e_lo) & (flat < e_hi)
    n_rows = int(local.sum())
    tiles, rows = plan.meta.cpu().tolist()
    assert rows == n_rows
    counts = torch.bincount(flat[local] - e_lo, minlength=e_hi - e_lo)
    assert plan.counts.cpu().tolist() == counts.tolist()
    assert tiles == int(((counts + ntok - 1) // ntok).sum())
    dst = plan.dst_row.cpu()[:n_rows]
    # expert-major, ascending route id inside an expert
    experts_sorted = flat[dst.long()]
    assert (experts_sorted[1:] >= experts_sorted[:-1]).all()
    for e in range(e_lo, e_hi):
        seg = dst[experts_sorted == e]
        assert (seg[1:] > seg[:-1]).all()
    assert sorted(dst.tolist()) == torch.nonzero(local).flatten().tolist()
    assert torch.equal(plan.src_token.cpu()[:n_rows], dst // topk)
    assert torch.allclose(plan.row_scale.cpu()[:n_rows], w.flatten().cpu()[dst.long()])
    # tile table
    tg, t0, tr = (t.cpu()[:tiles] for t in (plan.tile_group, plan.tile_row0, plan.tile_rows))
    assert int(tr.sum()) == n_rows and int(tr.max() if tiles else 0) <= ntok
    off = torch.cumsum(counts, 0) - counts
    for g_, r0, r in zip(tg.tolist(), t0.tolist(), tr.tolist()):
        assert off[g_] <= r0 and r0 + r <= off[g_] + counts[g_]


@pytest.mark.parametrize("T,E,topk,e_lo,e_hi,ntok,H,I", [(32, 64, 6, 0, 64, 32, 2048, 1408),
                                                          (32, 64, 6, 16, 24, 16, 512, 256),
                                                          (300, 8, 2, 0, 8, 128, 512, 384)])
def test_moe_grouped_pipeline(K, T, E, topk, e_lo, e_hi, ntok, H, I):
    """gather -> grouped gate/up SwiGLU -> grouped down with weighted scatter -> reduce."""
    idx, w, plan = _route_setup(K, T, E, topk, e_lo, e_hi, ntok)
    L = e_hi - e_lo
    x = rnd(T, H)
    w13 = rnd(L, 2 * I, H, scale=0.03)
    w2 = rnd(L, H, I, scale=0.03)
    xg = torch.zeros(T * topk, H, dtype=torch.bfloat16, device="cuda")
    K.gather_rows(x, plan, xg)
    hmid = torch.zeros(T * topk, I, dtype=torch.bfloat16, device="cuda")
    K.gemm(xg, w13, out=hmid, epilogue=K.EPI_SWIGLU, plan=plan)
    slots = topk + 1
    route_out = torch.zeros(T * slots, H, dtype=torch.bfloat16, device="cuda")
    # route r = t*topk + s lands in row t*slots + s
    ro_view = route_out.view(T, slots, H)
    K.moe_plan(idx, w, plan, e_lo, e_hi, dst_slots=slots)
    K.gemm(hmid, w2, out=route_out, epilogue=K.EPI_SCATTER, plan=plan)
    extra = rnd(T, H)
    resid = rnd(T, H)
    ro_view[:, topk] = extra
    out = K.moe_reduce(route_out, slots, topk, idx, e_lo, e_hi, T, H, residual=resid)
    # reference
    expect = resid.float() + extra.float()
    xf = x.float()
    for t in range(T):
        for s in range(topk):
            e = int(idx[t, s])
            if e_lo <= e < e_hi:
                y = w13[e - e_lo].float() @ xf[t]
                h = ref.bf16_round(ref.swiglu(y[:I], y[I:]))
                expect[t] += ref.bf16_round((w2[e - e_lo].float() @ h) * w[t, s])
    close(out, expect, rtol=3e-2, atol=3e-2)


def test_moe_retile_gives_the_scatter_gemm_taller_tiles(K):
    """A second tile table (256-row tiles) over a 128-row plan: same expert-major rows, fewer tiles, and the
    scatter GEMM over it writes exactly what it writes over the original table."""
    T, E, topk, H, I = 700, 8, 2, 512, 384
    idx, w, plan = _route_setup(K, T, E, topk, 0, E, 128)
    slots = topk + 1
    K.moe_plan(idx, w, plan, 0, E, dst_slots=slots)
    tall = K.moe_retile(plan, 256)
    counts = plan.counts.cpu()
    n2 = int(tall.meta[0])
    assert n2 == int(((counts + 255) // 256).sum()) and int(tall.meta[1]) == int(counts.sum())
    assert int(tall.tile_rows[:n2].sum()) == int(counts.sum()) and n2 < int(plan.meta[0])
    hmid = rnd(T * topk, I)
    w2 = rnd(E, H, I, scale=0.03)
    a = torch.zeros(T * slots, H, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros_like(a)
    K.gemm(hmid, w2, out=a, epilogue=K.EPI_SCATTER, plan=plan)
    K.gemm(hmid, w2, out=b, epilogue=K.EPI_SCATTER, plan=tall)
    assert torch.equal(a, b)
    again = K.moe_retile(plan, 256, tall)
    assert again is tall and int(tall.meta[0]) == n2


@pytest.mark.parametrize("score_fn,bias,groups,tg,norm", [(0, False, 1, 1, False), (1, True, 8, 4, True),
                                                         (2, True, 1, 1, True), (1, False, 1, 1, True)])
def test_router_topk(K, score_fn, bias, groups, tg, norm):
    T, E, k = 37, 256 if groups > 1 else 64, 8 if groups > 1 else 6
    g = torch.Generator(device="cuda").manual_seed(3)
    logits = torch.randn(T, E, generator=g, device="cuda")
    b = torch.randn(E, generator=g, device="cuda") * 0.1 if bias else None
    idx, w = K.router_topk(logits, k, score_fn, bias=b, n_groups=groups, topk_groups=tg, normalize=norm,
                           route_scale=2.5)
    ridx, rw = ref.route(logits, k, score_fn, bias=b, n_groups=groups, topk_groups=tg, normalize=norm,
                         route_scale=2.5)
    assert torch.equal(idx.cpu(), ridx.cpu())
    assert torch.allclose(w, rw, rtol=1e-4, atol=1e-6)


def test_router_hash_and_ties(K):
    T, E, k, V = 9, 64, 6, 50
    logits = torch.zeros(T, E, device="cuda")            # all tied -> lowest ids win
    idx, w = K.router_topk(logits, k, 0)
    assert idx.cpu().tolist() == [list(range(k))] * T
    g = torch.Generator(device="cuda").manual_seed(4)
    logits = torch.randn(T, E, generator=g, device="cuda")
    table = torch.randint(0, E, (V, k), generator=g, device="cuda", dtype=torch.int64)
    toks = torch.randint(0, V, (T,), generator=g, device="cuda", dtype=torch.int32)
    idx, w = K.router_topk(logits, k, 2, hash_table=table, token_ids=toks, normalize=True, route_scale=1.5)
    ridx, rw = ref.route(logits, k, 2, hash_table=table, token_ids=toks, normalize=True, route_scale=1.5)
    assert torch.equal(idx.cpu(), ridx.cpu())
    assert torch.allclose(w, rw, rtol=1e-4, atol=1e-6)


def test_add_rmsnorm_and_embedding(K):
    rows, dim = 33, 2048
    x, d, w = rnd(rows, dim), rnd(rows, dim), rnd(dim)
    res, nrm = K.add_rmsnorm(x, w, 1e-6, delta=d)
    r = ref.bf16_round(x.float() + d.float())
    close(res, r, rtol=0, atol=0)
    close(nrm, ref.rmsnorm(r, w, 1e-6), rtol=1e-2, atol=1e-2)
    _, nrm2 = K.add_rmsnorm(x, w, 1e-6)
    close(nrm2, ref.rmsnorm(x, w, 1e-6), rtol=1e-2, atol=1e-2)
    table = rnd(1000, 512)
    ids = torch.randint(0, 1000, (17,), device="cuda", dtype=torch.int32)
    assert torch.equal(K.embedding(ids, table), table[ids.long()])


def test_argmax_topk(K):
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(6, 102400, generator=g, device="cuda")
    logits[0, 7] = logits[0, 90000] = 50.0          # tie -> lower id
    logits[1] = float("nan")
    logits[2, 5] = float("nan")
    ids = K.argmax(logits)
    assert torch.equal(ids.cpu(), ref.greedy_argmax(logits).cpu())
    assert int(ids[0]) == 7 and int(ids[1]) == -1
    ti, tv = K.topk_logits(logits[3:], 40)
    ri, rv = ref.topk_logits(logits[3:], 40)
    assert torch.equal(ti.cpu(), ri.cpu()) and torch.allclose(tv, rv)


def _attn_case(K, heads, dl, dr, page, ctx_lens, q_per_seq, splits, split_tokens, sink=False, seed=0,
               merge_in_kernel=True, cluster=False):
    D = dl + dr
    S = len(ctx_lens)
    max_blocks = (max(ctx_lens) + page - 1) // page + 1
    n_pages = S * max_blocks + 3
    g = torch.Generator(device="cuda").manual_seed(seed)
    pool = (torch.randn(n_pages * page, D, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    perm = torch.randperm(n_pages, generator=g, device="cuda")[: S * max_blocks].to(torch.int32)
    bt = perm.view(S, max_blocks).contiguous()
    row_seq, row_pos = [], []
    for s, n in enumerate(ctx_lens):
        for j in range(q_per_seq):
            row_seq.append(s)
            row_pos.append(n - q_per_seq + j)
    rows = len(row_seq)
    row_seq = torch.tensor(row_seq, dtype=torch.int32, device="cuda")
    row_pos = torch.tensor(row_pos, dtype=torch.int32, device="cuda")
    q = (torch.randn(rows, heads, D, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    sk = torch.randn(heads, generator=g, device="cuda") if sink else None
    out = torch.zeros(rows, heads, dl, dtype=torch.bfloat16, device="cuda")
    ws = None
    if splits > 1 and not cluster:
        ws = K.AttnWorkspace(torch.zeros(rows, splits, heads, dl, device="cuda"),
                             torch.zeros(rows, splits, heads, 2, device="cuda"), rows, splits,
                             torch.zeros(rows * ((heads + 15) // 16), dtype=torch.int32, device="cuda")
                             if merge_in_kernel else None)
    scale = 1.0 / math.sqrt(dl // 4 + dr)
    K.mla_attention(q, pool, bt, row_seq, row_pos, page, dl, dr, scale, out, splits=splits,
                    split_tokens=split_tokens, ws=ws, sink=sk)
    expect = ref.mla_paged_attention(q, pool, bt, row_seq, row_pos, page, dl, scale, sink=sk)
    close(out, expect, rtol=2e-2, atol=1e-2)


@pytest.mark.parametrize("heads,dl,dr,page,ctx,qps,splits,st,sink", [
    (16, 512, 64, 64, [1, 64, 65, 700], 1, 1, 1 << 20, False),
    (16, 512, 64, 64, [513, 768, 40], 1, 4, 256, False),
    (16, 512, 64, 16, [100, 300], 3, 2, 192, True),
    (4, 64, 16, 16, [17, 64, 33], 2, 1, 1 << 20, False),
    (2, 512, 64, 64, [130], 1, 3, 64, True),
    (16, 512, 64, 64, [640] * 5, 1, 8, 128, True),
    (32, 512, 64, 64, [200, 90], 1, 1, 1 << 20, False),
    (128, 512, 64, 64, [150], 1, 2, 128, False),
])
def test_mla_attention(K, heads, dl, dr, page, ctx, qps, splits, st, sink):
    _attn_case(K, heads, dl, dr, page, ctx, qps, splits, st, sink)
    if splits > 1:
        _attn_case(K, heads, dl, dr, page, ctx, qps, splits, st, sink, merge_in_kernel=False)
    if splits in (2, 4, 8):
        _attn_case(K, heads, dl, dr, page, ctx, qps, splits, st, sink, cluster=True)


@pytest.mark.parametrize("heads,page,segs,sink", [
    (16, 64, [(0, 200), (37, 129), (500, 64), (0, 5)], False),      # (context before the chunk, chunk rows)
    (16, 16, [(0, 70), (100, 33)], True),
    (8, 64, [(64, 300)], False),
    (128, 64, [(0, 40), (90, 7)], False),
    (32, 128, [(300, 260), (0, 1)], True),
])
def test_mla_prefill_tc_matches_reference_and_the_row_tile_kernel(K, heads, page, segs, sink):
    """tcgen05 prefill attention (128-row tiles, P from TMEM, V as the MN-major view of the KV tile) against the
    fp32 reference; chunks that start mid-sequence, partial tiles, pages smaller and larger than the KV tile."""
    dl, dr = 512, 64
    D = dl + dr
    S = len(segs)
    total = [c + n for c, n in segs]
    max_blocks = (max(total) + page - 1) // page + 1
    n_pages = S * max_blocks + 3
    g = torch.Generator(device="cuda").manual_seed(11)
    pool = (torch.randn(n_pages * page, D, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    bt = torch.randperm(n_pages, generator=g, device="cuda")[: S * max_blocks].to(torch.int32).view(S, max_blocks)
    # pages past a sequence's end hold ids that must never be dereferenced
    for s_, t in enumerate(total):
        bt[s_, (t + page - 1) // page:] = -1
    bt = bt.contiguous()
    row_seq, row_pos, segments, r0 = [], [], [], 0
    for s_, (c, n) in enumerate(segs):
        segments.append((s_, r0, n, c))
        row_seq += [s_] * n
        row_pos += list(range(c, c + n))
        r0 += n
    rows = r0
    row_seq = torch.tensor(row_seq, dtype=torch.int32, device="cuda")
    row_pos = torch.tensor(row_pos, dtype=torch.int32, device="cuda")
    q = (torch.randn(rows, heads, D, generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    sk = torch.randn(heads, generator=g, device="cuda") if sink else None
    scale = 1.0 / math.sqrt(dl // 4 + dr)
    tiles_np, rest = K.prefill_tiles(segments, heads)
    assert rest == [] and K.prefill_tc_supported(heads, dl, dr, page)
    tiles = torch.from_numpy(tiles_np).cuda()
    out = torch.full((rows, heads, dl), 7.0, dtype=torch.bfloat16, device="cuda")
    K.mla_prefill_tc(q, pool, bt, tiles, tiles.shape[0], page, dl, dr, scale, out, sink=sk)
    assert K._lib.read_status()[0] == 0
    expect = ref.mla_paged_attention(q, pool, bt.clamp(min=0), row_seq, row_pos, page, dl, scale, sink=sk)
    close(out, expect, rtol=2e-2, atol=1e-2)
    legacy = torch.zeros_like(out)
    K.mla_attention(q, pool, bt, row_seq, row_pos, page, dl, dr, scale, legacy, sink=sk)
    close(out, legacy, rtol=2e-2, atol=1e-2)
    # a row's result does not depend on its tile mates: cut the same rows into other tiles
    tiles2_np, _ = K.prefill_tiles([(s_, r, 1, p_) for s_, r_, n, p_0 in segments[:1]
                                    for r, p_ in zip(range(r_, r_ + min(n, 9)), range(p_0, p_0 + min(n, 9)))], heads)
    out2 = torch.zeros_like(out)
    t2 = torch.from_numpy(tiles2_np).cuda()
    K.mla_prefill_tc(q, pool, bt, t2, t2.shape[0], page, dl, dr, scale, out2, sink=sk)
    n9 = min(segs[0][1], 9)
    assert torch.equal(out2[:n9], out[:n9])


def test_mla_prep(K):
    rows, heads, qhd, lora, rope = 11, 16, 192, 512, 64
    D = lora + rope
    q = rnd(rows, heads * qhd)
    ckv = rnd(rows, D)
    wn = rnd(lora)
    cos, sin = (t.cuda() for t in ref.rope_tables(4096, rope, 10000.0))
    pos = torch.randint(0, 4096, (rows,), device="cuda", dtype=torch.int32)
    pool = torch.zeros(64 * 4, D, dtype=torch.bfloat16, device="cuda")
    slots = torch.randperm(64 * 4, device="cuda")[:rows].to(torch.int64)
    slots[3] = -1                                      # "do not write" marker
    q_out = torch.zeros(rows, heads, D, dtype=torch.bfloat16, device="cuda")
    K.mla_prep(q, qhd, ckv, heads, lora, rope, wn, 1e-6, cos, sin, pos, slots, pool, q_out.view(rows, -1))
    c, s = cos[pos.long()], sin[pos.long()]
    qr = ref.apply_rope(q.view(rows, heads, qhd)[:, :, qhd - rope:], c[:, None, :], s[:, None, :])
    close(q_out[:, :, lora:], qr, rtol=1e-2, atol=1e-2)
    kvn = ref.rmsnorm(ckv[:, :lora], wn, 1e-6)
    kr = ref.apply_rope(ckv[:, lora:], c, s)
    for r in range(rows):
        if int(slots[r]) < 0:
            continue
        close(pool[int(slots[r]), :lora], kvn[r], rtol=1e-2, atol=1e-2)
        close(pool[int(slots[r]), lora:], kr[r], rtol=1e-2, atol=1e-2)
    written = torch.zeros(pool.shape[0], dtype=torch.bool, device="cuda")
    written[slots[slots >= 0]] = True
    assert float(pool[~written].abs().max()) == 0.0


def test_copy_pages(K):
    pool = rnd(3, 10, 16, 80)
    before = pool.clone()
    pairs = torch.tensor([[1, 7], [2, 9]], dtype=torch.int32, device="cuda")
    K.copy_pages(pool, pairs)
    assert torch.equal(pool[:, 7], before[:, 1]) and torch.equal(pool[:, 9], before[:, 2])
    assert torch.equal(pool[:, :7], before[:, :7])


def test_argmax_chunked(K):
    g = torch.Generator(device="cuda").manual_seed(9)
    logits = torch.randn(5, 102400, generator=g, device="cuda")
    logits[0, 11] = logits[0, 70001] = 60.0
    logits[1] = float("nan")
    logits[2, 102399] = 99.0
    sc = K.ArgmaxScratch.allocate(8, "cuda")
    ids = torch.zeros(5, dtype=torch.int32, device="cuda")
    vals = torch.zeros(5, device="cuda")
    for _ in range(2):                       # the row counters must be reusable
        K.argmax_chunked(logits, sc, ids, vals)
        assert torch.equal(ids.cpu(), ref.greedy_argmax(logits).cpu())
    assert int(ids[0]) == 11 and int(ids[1]) == -1 and int(ids[2]) == 102399
    odd = torch.randn(3, 1000, generator=g, device="cuda")
    K.argmax_chunked(odd, sc, ids[:3], vals[:3])
    assert torch.equal(ids[:3].cpu(), ref.greedy_argmax(odd).cpu())


@pytest.mark.parametrize("T,E,k,H,score,groups,tg", [(32, 64, 6, 2048, 0, 1, 1), (5, 256, 8, 1024, 1, 8, 4),
                                                      (200, 16, 4, 512, 2, 1, 1)])
def test_router_plan_fused(K, T, E, k, H, score, groups, tg):
    x = rnd(T, H)
    w = rnd(E, H, scale=0.05)
    bias = torch.randn(E, device="cuda") * 0.01 if score else None
    e_lo, e_hi = E // 4, E // 2
    plan = K.MoePlan.allocate(T * k, e_hi - e_lo, 16, "cuda")
    idx = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(T, k, device="cuda")
    ctr = torch.zeros(4, dtype=torch.int32, device="cuda")
    for _ in range(2):
        K.router_plan_fused(x, w, k, score, plan, e_lo, e_hi, idx, wts, ctr, bias=bias, n_groups=groups,
                            topk_groups=tg, normalize=True, route_scale=1.5, dst_slots=k + 1)
    torch.cuda.synchronize()
    logits = x.float() @ w.float().T
    ridx, rw = ref.route(logits, k, score, bias=bias, n_groups=groups, topk_groups=tg, normalize=True, route_scale=1.5)
    # fp32 summation order differs from the reference matmul: compare on tokens without near ties
    sel = ref.route(logits, min(k + 1, E), score, bias=bias, normalize=False)[1] if groups == 1 else None
    same = (idx.cpu() == ridx.cpu()).all(-1)
    assert float(same.float().mean()) > 0.9
    assert torch.allclose(wts[same.cuda()], rw[same.cuda()], rtol=2e-3, atol=1e-5)
    # the plan describes exactly the routes the kernel chose
    plan2 = K.MoePlan.allocate(T * k, e_hi - e_lo, 16, "cuda")
    K.moe_plan(idx, wts, plan2, e_lo, e_hi, dst_slots=k + 1)
    torch.cuda.synchronize()
    n = int(plan2.meta[1])
    assert plan.meta.cpu().tolist() == plan2.meta.cpu().tolist()
    assert torch.equal(plan.dst_row[:n].cpu(), plan2.dst_row[:n].cpu())
    assert torch.equal(plan.src_token[:n].cpu(), plan2.src_token[:n].cpu())
    assert torch.equal(plan.counts.cpu(), plan2.counts.cpu())


@pytest.mark.parametrize("T,E,k,H,I", [(32, 64, 6, 2048, 1408), (5, 64, 6, 2048, 1408), (64, 32, 8, 1024, 512)])
def test_router_append_static_plan(K, T, E, k, H, I):
    """Static one-tile-per-expert plan: same routes as the planned path, and the grouped GEMM pair over it (with
    empty experts skipped) gives the same per-route outputs."""
    x = rnd(T, H)
    w = rnd(E, H, scale=0.05)
    e_lo, e_hi = E // 4, E
    el = e_hi - e_lo
    nt = 16 if T <= 16 else (32 if T <= 32 else 64)
    w13 = rnd(el, 2 * I, H, scale=0.03)
    w2 = rnd(el, H, I, scale=0.03)
    slots = k + 1
    cnt = torch.zeros(2, el, dtype=torch.int32, device="cuda")
    base = K.static_plan(nt, el, cnt[0])
    plan = K.static_plan(nt, el, cnt[1], base)
    idx = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    wts = torch.zeros(T, k, device="cuda")
    xg = torch.zeros(el * nt, H, dtype=torch.bfloat16, device="cuda")
    hmid = torch.zeros(el * nt, I, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(T * slots, H, dtype=torch.bfloat16, device="cuda")
    for _ in range(2):
        cnt.zero_()
        K.router_append(x, w, k, 0, plan, e_lo, e_hi, idx, wts, xg, normalize=True, route_scale=1.5, dst_slots=slots)
        K.gemm(xg, w13, out=hmid, epilogue=K.EPI_SWIGLU, plan=plan)
        K.gemm(hmid, w2, out=out, epilogue=K.EPI_SCATTER, plan=plan, scatter_rows=T * slots)
    torch.cuda.synchronize()
    from ferrule_b200.ops import _lib
    assert _lib.read_status()[0] == 0
    # planned path on the same routes
    plan2 = K.MoePlan.allocate(T * k, el, 16, "cuda")
    K.moe_plan(idx, wts, plan2, e_lo, e_hi, dst_slots=slots)
    xg2 = torch.zeros(T * k, H, dtype=torch.bfloat16, device="cuda")
    K.gather_rows(x, plan2, xg2, cap_rows=T * k)
    hmid2 = torch.zeros(T * k, I, dtype=torch.bfloat16, device="cuda")
    out2 = torch.zeros(T * slots, H, dtype=torch.bfloat16, device="cuda")
    K.gemm(xg2, w13, out=hmid2, epilogue=K.EPI_SWIGLU, plan=plan2)
    K.gemm(hmid2, w2, out=out2, epilogue=K.EPI_SCATTER, plan=plan2, scatter_rows=T * slots)
    torch.cuda.synchronize()
    assert torch.equal(cnt[1].cpu(), plan2.counts.cpu()) and int(cnt[0].sum()) == 0
    assert int(cnt[1].sum()) == int(((idx >= e_lo) & (idx < e_hi)).sum())
    local = ((idx >= e_lo) & (idx < e_hi)).cpu()
    o1 = out.view(T, slots, H)[:, :k].float().cpu()
    o2 = out2.view(T, slots, H)[:, :k].float().cpu()
    assert torch.equal(o1[local], o2[local])


@pytest.mark.parametrize("T,E,k,H,with_delta", [(32, 64, 6, 2048, True), (7, 64, 6, 2048, False), (16, 256, 8, 7168, True)])
def test_router_append_with_norm_prologue_is_bit_equal_to_norm_then_router(K, T, E, k, H, with_delta):
    """Residual add + RMSNorm folded into the router kernel: same residual stream, same normalised rows, same
    routes and weights, and the same gathered rows as add_rmsnorm followed by router_append."""
    h = rnd(T, H)
    delta = rnd(T, H, scale=0.3) if with_delta else None
    nw = rnd(H)
    w = rnd(E, H, scale=0.05)
    e_lo, e_hi = 0, E
    nt = 16 if T <= 16 else 32
    outs = []
    for fused in (False, True):
        cnt = torch.zeros(E, dtype=torch.int32, device="cuda")
        plan = K.static_plan(nt, E, cnt)
        idx = torch.zeros(T, k, dtype=torch.int32, device="cuda")
        wts = torch.zeros(T, k, device="cuda")
        xg = torch.zeros(E * nt, H, dtype=torch.bfloat16, device="cuda")
        res = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
        xn = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
        if fused:
            K.router_append(h, w, k, 0, plan, e_lo, e_hi, idx, wts, xg, normalize=True, dst_slots=k + 1,
                            norm_w=nw, eps=1e-6, delta=delta, res_out=res if with_delta else None, norm_out=xn)
        else:
            if with_delta:
                K.add_rmsnorm(h, nw, 1e-6, delta=delta, res_out=res, norm_out=xn)
            else:
                K.add_rmsnorm(h, nw, 1e-6, norm_out=xn)
            K.router_append(xn, w, k, 0, plan, e_lo, e_hi, idx, wts, xg, normalize=True, dst_slots=k + 1)
        torch.cuda.synchronize()
        # rows of one expert land in the order of the atomics: compare them keyed by their source token
        rows = {}
        c = cnt.cpu().tolist()
        src = plan.src_token.cpu().tolist()
        for e in range(E):
            for j in range(c[e]):
                r = e * nt + j
                rows[(e, src[r])] = xg[r].cpu()
        outs.append((idx.cpu(), wts.cpu(), xn.cpu(), res.cpu(), rows))
    a, b = outs
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])
    assert a[4].keys() == b[4].keys() and len(a[4]) == T * k
    assert all(torch.equal(a[4][key], b[4][key]) for key in a[4])
    from ferrule_b200.ops import _lib
    assert _lib.read_status()[0] == 0


@pytest.mark.parametrize("T,k,H", [(32, 6, 2048), (5, 8, 7168)])
def test_moe_reduce_norm_is_bit_equal_to_reduce_then_norm(K, T, k, H):
    slots = k + 1
    ro = rnd(T * slots, H)
    idx = torch.randint(0, 16, (T, k), dtype=torch.int32, device="cuda")
    res = rnd(T, H)
    w = rnd(H)
    out1 = torch.zeros(T, H, dtype=torch.bfloat16, device="cuda")
    K.moe_reduce(ro, slots, k, idx, 4, 12, T, H, residual=res, out=out1)
    _, n1 = K.add_rmsnorm(out1, w, 1e-6)
    out2 = torch.zeros_like(out1)
    n2 = torch.zeros_like(out1)
    K.moe_reduce_norm(ro, slots, k, idx, 4, 12, T, H, res, out2, w, n2, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(out1, out2) and torch.equal(n1, n2)


def test_bounded_wait_reports_timeout_and_context_stays_usable():
    """Failure detection on the device: a wait on a flag that nothing sets gives up after its limit, records a
    status word (no trap, no hang) and later kernels still run."""
    from ferrule_b200.ops import _lib
    lib = _lib.get_lib(True)
    flag = torch.zeros(4, dtype=torch.int32, device="cuda")
    result = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    _lib.read_status()                                        # start clean
    st = _lib.status_tensor()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.fb_flag_wait_probe(flag.data_ptr(), 1, 50_000_000, st.data_ptr(), result.data_ptr(), _lib.stream_ptr())
    t1.record()
    assert rc == 0
    torch.cuda.synchronize()
    assert 30.0 <= t0.elapsed_time(t1) <= 1000.0              # waited about the 50 ms limit, then returned
    assert int(result[0]) == 0                                # the wait reported failure to its caller
    code, where, seen, target = _lib.read_status()
    assert code == 2 and target == 1 and seen == 0           # "peer flag timeout"
    assert _lib.read_status()[0] == 0                         # reading cleared it
    x = torch.arange(8, device="cuda").float()
    assert float((x * 2).sum()) == 56.0                       # the context is alive
    flag[0] = 1                                               # now the same wait succeeds at once
    lib.fb_flag_wait_probe(flag.data_ptr(), 1, 50_000_000, st.data_ptr(), result.data_ptr(), _lib.stream_ptr())
    torch.cuda.synchronize()
    assert int(result[0]) == 1 and _lib.read_status()[0] == 0
