"""Quantisation kernels against the host codecs (io/encoding.py)."""
import pytest
import torch

from ferrule_b200.io import encoding as enc

pytestmark = pytest.mark.gpu


def rnd(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def test_fp8_row_quant_matches_host_codec_bitwise():
    from ferrule_b200.ops import quant as Q
    x = rnd(37, 512, scale=3.0)
    x[0, :128] = 0            # exercises the amax floor
    x[1, 5] = 1000.0          # saturation inside a block is impossible after scaling, large scale instead
    q, s = Q.quant_fp8_rows(x)
    rq, rs = enc.act_quant_fp8(x.float().cpu())
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(q.cpu(), rq)
    y = x.clone()
    Q.fp8_qat_(y)
    assert torch.equal(y.float().cpu(), enc.fp8_qat(x.float().cpu()))


def test_fp8_block_and_mxfp4_dequant_and_quant():
    from ferrule_b200.ops import quant as Q
    w = (torch.randn(300, 512) * 0.05)
    qw, sw = enc.weight_quant_fp8_block(w)
    d = Q.dequant_fp8_block(qw.cuda(), sw.cuda())
    assert torch.equal(d.float().cpu(), enc.weight_dequant_fp8_block(qw, sw).bfloat16().float())
    x = rnd(19, 256, scale=2.0, seed=3)
    p, s = Q.quant_mxfp4_rows(x)
    rp, rs = enc.weight_quant_mxfp4(x.float().cpu())
    assert torch.equal(s.cpu(), rs)
    assert torch.equal(p.cpu(), rp)
    d4 = Q.dequant_mxfp4(p, s)
    assert torch.equal(d4.float().cpu(), enc.weight_dequant_mxfp4(rp, rs).bfloat16().float())


def test_hadamard_rows():
    from ferrule_b200.ops import quant as Q
    x = rnd(7, 512, seed=5)
    y = x.clone()
    Q.hadamard_(y)
    ref = enc.hadamard(x.float().cpu())
    assert float((y.float().cpu() - ref).abs().max()) <= 0.02 * float(ref.abs().max()) + 1e-3


def _fp8_inputs(rows, n, k, seed):
    from ferrule_b200.ops import quant as Q
    x = rnd(rows, k, scale=1.5, seed=seed)
    xq, xs = Q.quant_fp8_rows(x)
    w = (torch.randn(n, k, generator=torch.Generator().manual_seed(seed + 1)) * 0.05)
    wq, ws = enc.weight_quant_fp8_block(w)
    xd = enc.act_dequant_fp8(xq.cpu(), xs.cpu())
    wd = enc.weight_dequant_fp8_block(wq, ws)
    return xq, xs, wq.cuda(), ws.cuda(), xd, wd


@pytest.mark.parametrize("rows,n,k", [(32, 2048, 2048), (5, 576, 1536), (64, 256, 7168), (16, 128, 128)])
def test_gemm_fp8_block_scaled_dense(rows, n, k):
    from ferrule_b200.ops import quant as Q
    xq, xs, wq, ws, xd, wd = _fp8_inputs(rows, n, k, 11)
    out = Q.gemm_fp8(xq, xs, wq, ws, out_dtype=torch.float32)
    ref = xd @ wd.T
    err = (out.cpu() - ref).abs().max()
    assert float(err) <= 2e-3 * float(ref.abs().max()) + 1e-4, float(err)


def test_gemm_fp8_swiglu_and_grouped_scatter():
    from ferrule_b200.ops import kernels as K
    from ferrule_b200.ops import quant as Q
    from ferrule_b200.ops import reference as ref
    rows, inter, k = 32, 256, 1024
    xq, xs, wq, ws, xd, wd = _fp8_inputs(rows, 2 * inter, k, 21)
    out = Q.gemm_fp8(xq, xs, wq, ws, epilogue=1, out_dtype=torch.float32)
    y = xd @ wd.T
    r = ref.swiglu(y[:, :inter], y[:, inter:])
    assert float((out.cpu() - r).abs().max()) <= 3e-3 * float(r.abs().max()) + 1e-4
    # grouped: 8 experts, routes in expert-major order
    T, E, topk, H, I = 24, 8, 2, 512, 256
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(T, E, generator=g, device="cuda")
    idx, wts = ref.route(logits, topk, 0)
    plan = K.MoePlan.allocate(T * topk, E, 16, "cuda")
    K.moe_plan(idx, wts, plan, 0, E)
    x = rnd(T, H, seed=31)
    xg = torch.zeros(T * topk, H, dtype=torch.bfloat16, device="cuda")
    K.gather_rows(x, plan, xg)
    xgq, xgs = Q.quant_fp8_rows(xg)
    w2 = torch.randn(E, I, H, generator=torch.Generator().manual_seed(9)) * 0.05
    packs = [enc.weight_quant_fp8_block(w2[e]) for e in range(E)]
    w2q = torch.stack([p[0] for p in packs]).cuda()
    w2s = torch.stack([p[1] for p in packs]).cuda()
    out = torch.zeros(T * topk, I, dtype=torch.float32, device="cuda")
    Q.gemm_fp8(xgq, xgs, w2q, w2s, out=out, epilogue=2, plan=plan)
    torch.cuda.synchronize()
    n = int(plan.meta[1])
    xgd = enc.act_dequant_fp8(xgq.cpu(), xgs.cpu())
    flat = idx.flatten().cpu()
    dst = plan.dst_row.cpu()[:n]
    exp = torch.zeros(T * topk, I)
    for pos in range(n):
        route = int(dst[pos])
        e = int(flat[route])
        wd = enc.weight_dequant_fp8_block(*packs[e])
        exp[route] = (wd @ xgd[pos]) * float(wts.flatten()[route])
    assert float((out.cpu() - exp).abs().max()) <= 3e-3 * float(exp.abs().max()) + 1e-4


@pytest.mark.parametrize("rows,dim", [(32, 2048), (5, 7168), (3, 128), (17, 1536)])
def test_add_rmsnorm_writes_the_fp8_form_of_its_output(rows, dim):
    """norm -> FP8 in one kernel: codes and scales are bit-equal to the row quantiser run on the bf16 output."""
    from ferrule_b200.ops import kernels as K
    from ferrule_b200.ops import quant as Q
    x, d, w = rnd(rows, dim, seed=1), rnd(rows, dim, seed=2), rnd(dim, seed=3)
    q = torch.zeros(rows + 2, dim, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(rows + 2, dim // 128, dtype=torch.uint8, device="cuda")
    res, nrm = K.add_rmsnorm(x, w, 1e-6, delta=d, quant_out=(q, sc))
    res2, nrm2 = K.add_rmsnorm(x, w, 1e-6, delta=d)
    assert torch.equal(res, res2) and torch.equal(nrm, nrm2)
    q2, s2 = Q.quant_fp8_rows(nrm2)
    assert torch.equal(q[:rows], q2) and torch.equal(sc[:rows], s2)
    assert int(q[rows:].sum()) == 0 and int(sc[rows:].sum()) == 0
    # 1 x 32 blocks (MXFP8) for the linears that run on the block-scaled MMA
    q3 = torch.zeros(rows, dim, dtype=torch.uint8, device="cuda")
    s3 = torch.zeros(rows, dim // 32, dtype=torch.uint8, device="cuda")
    K.add_rmsnorm(x, w, 1e-6, delta=d, quant_out=(q3, s3), quant_block=32)
    q4, s4 = Q.quant_mxfp8_rows(nrm2)
    assert torch.equal(q3, q4) and torch.equal(s3, s4)


@pytest.mark.parametrize("rows,n,k,dual", [(32, 2048, 2048, False), (5, 576, 1536, False), (64, 256, 7168, False),
                                           (16, 128, 128, False), (32, 256, 1024, True), (100, 384, 512, False)])
def test_fp8_block_weights_on_the_block_scaled_mma(rows, n, k, dual):
    """e4m3 weights with 128 x 128 block scales replicated into the per-32 scale layout: the tensor core applies
    the scales, the products are those of the checkpoint format (fp32 oracle over the dequantised operands)."""
    from ferrule_b200.ops import quant as Q
    from ferrule_b200.ops import reference as ref
    x = rnd(rows, k, scale=1.5, seed=51)
    xq, xs = Q.quant_mxfp8_rows(x)
    n_w = 2 * n if dual else n
    w = torch.randn(n_w, k, generator=torch.Generator().manual_seed(52)) * 0.05
    wq, ws_ = enc.weight_quant_fp8_block(w)
    wd = enc.weight_dequant_fp8_block(wq, ws_)
    sf = Q.fp8_block_sf(ws_.cuda(), n_w, k)
    out = Q.gemm_mxfp4(xq, xs, wq.cuda(), sf, out_dtype=torch.float32, epilogue=1 if dual else 0, w_fp8=True,
                       ntok=None if rows <= 64 else 64)
    xd = _mx_dequant_rows(xq.cpu(), xs.cpu())
    y = xd @ wd.T
    want = ref.swiglu(y[:, :n], y[:, n:]) if dual else y
    err = (out.cpu() - want).abs().max()
    assert float(err) <= 2e-3 * float(want.abs().max()) + 1e-4, float(err)


@pytest.mark.parametrize("slot,counts", [(32, [3, 0, 32, 1, 0, 0, 17, 9]), (64, [40, 0, 64, 1, 33, 0, 0, 32]),
                                         (16, [16, 0, 0, 0, 2, 0, 0, 0])])
def test_gemm_fp8_static_slots_skip_empty_experts_and_requantise(slot, counts):
    """Slot mode of the FP8 GEMM (group g owns rows [g * slot, (g + 1) * slot), counts[g] filled): the SwiGLU
    epilogue's FP8 output equals the row quantiser applied to the bf16 result, rows outside the counts are not
    touched, and the slot walk gives the result of the same GEMM over an explicit tile table."""
    from ferrule_b200.ops import kernels as K
    from ferrule_b200.ops import quant as Q
    E, H, I = len(counts), 512, 256
    ntok = min(slot, 32)
    x = rnd(E * slot, H, scale=1.5, seed=41)
    xq, xs = Q.quant_fp8_rows(x)
    w13 = torch.randn(E, 2 * I, H, generator=torch.Generator().manual_seed(42)) * 0.05
    packs = [enc.weight_quant_fp8_block(w13[e]) for e in range(E)]
    wq = torch.stack([p_[0] for p_ in packs]).cuda()
    ws_ = torch.stack([p_[1] for p_ in packs]).cuda()
    cnt = torch.tensor(counts, dtype=torch.int32, device="cuda")
    # explicit table: slot // ntok tiles per expert
    tg, t0, tr = [], [], []
    for e, c in enumerate(counts):
        for sub in range(slot // ntok):
            tg.append(e)
            t0.append(e * slot + sub * ntok)
            tr.append(max(0, min(ntok, c - sub * ntok)))
    i32 = dict(dtype=torch.int32, device="cuda")
    plan = K.MoePlan(ntok, len(tg), E * slot, torch.zeros(E * slot, **i32), torch.arange(E * slot, **i32),
                     torch.ones(E * slot, device="cuda"), torch.tensor(tg, **i32), torch.tensor(t0, **i32),
                     torch.tensor(tr, **i32), cnt, torch.tensor([len(tg), sum(counts)], **i32))
    want = torch.full((E * slot, I), 7.0, dtype=torch.bfloat16, device="cuda")
    Q.gemm_fp8(xq, xs, wq, ws_, out=want, epilogue=1, plan=plan, act_limit=7.0)
    got = torch.full((E * slot, I), 7.0, dtype=torch.bfloat16, device="cuda")
    Q.gemm_fp8(xq, xs, wq, ws_, out=got, epilogue=1, slots=(cnt, slot), act_limit=7.0)
    assert torch.equal(got, want)
    oq = torch.full((E * slot, I), 9, dtype=torch.uint8, device="cuda")
    os_ = torch.full((E * slot, I // 128), 9, dtype=torch.uint8, device="cuda")
    Q.gemm_fp8(xq, xs, wq, ws_, epilogue=1, slots=(cnt, slot), act_limit=7.0, out_q=(oq, os_))
    q2, s2 = Q.quant_fp8_rows(want)
    for e, c in enumerate(counts):
        r0 = e * slot
        assert torch.equal(oq[r0:r0 + c], q2[r0:r0 + c]) and torch.equal(os_[r0:r0 + c], s2[r0:r0 + c])
        assert int((oq[r0 + c:r0 + slot] != 9).sum()) == 0 and float((got[r0 + c:r0 + slot].float() - 7).abs().sum()) == 0
    # the down projection over the quantised rows, scatter epilogue through the same slots
    w2 = torch.randn(E, H, I, generator=torch.Generator().manual_seed(43)) * 0.05
    p2 = [enc.weight_quant_fp8_block(w2[e]) for e in range(E)]
    w2q, w2s = torch.stack([p_[0] for p_ in p2]).cuda(), torch.stack([p_[1] for p_ in p2]).cuda()
    a = torch.zeros(E * slot, H, dtype=torch.bfloat16, device="cuda")
    b_ = torch.zeros_like(a)
    Q.gemm_fp8(q2, s2, w2q, w2s, out=a, epilogue=2, plan=plan)
    Q.gemm_fp8(oq, os_, w2q, w2s, out=b_, epilogue=2, plan=plan, slots=(cnt, slot))
    assert torch.equal(a, b_)


@pytest.mark.parametrize("slot,sub,counts,w_fp8", [(64, 16, [40, 0, 64, 1, 33, 0, 0, 17], True),
                                                   (32, 16, [3, 0, 32, 1, 0, 0, 16, 9], False),
                                                   (64, 32, [0, 0, 5, 0, 64, 0, 31, 33], False)])
def test_block_scaled_gemm_walks_static_slots_in_short_tiles(slot, sub, counts, w_fp8):
    """Slot mode of the block-scaled GEMM: a `slot`-row slot per expert walked in `sub`-row tiles gives bit for bit
    the result of one `slot`-row tile per expert over an explicit table (gate|up with MXFP8 requant, then the
    scatter GEMM), touches nothing outside the filled rows, and skips experts and sub-tiles without rows."""
    from ferrule_b200.ops import kernels as K
    from ferrule_b200.ops import quant as Q
    E, H, I = len(counts), 512, 256
    x = rnd(E * slot, H, scale=1.5, seed=61)
    xq, xs = Q.quant_mxfp8_rows(x)
    w13 = rnd(E, 2 * I, H, scale=0.05, seed=62)
    w2 = rnd(E, H, I, scale=0.05, seed=63)
    if w_fp8:
        def prep(w):
            packs = [enc.weight_quant_fp8_block(w[e].float().cpu()) for e in range(E)]
            q = torch.stack([p_[0] for p_ in packs]).cuda()
            sc = torch.stack([p_[1] for p_ in packs]).cuda()
            return q, Q.fp8_block_sf(sc, w.shape[1], w.shape[2])
    else:
        def prep(w):
            G, O, Kk = w.shape
            packed, sb = Q.quant_mxfp4_rows(w.reshape(G * O, Kk).contiguous())
            return packed.view(G, O, Kk // 2), Q.mxfp4_prepare_sf(sb.view(G, O, Kk // 32))
    (c13, sf13), (c2, sf2) = prep(w13), prep(w2)
    cnt = torch.tensor(counts, dtype=torch.int32, device="cuda")
    i32 = dict(dtype=torch.int32, device="cuda")
    ar = torch.arange(E, **i32)
    plan = K.MoePlan(slot, E, E * slot, torch.zeros(E * slot, **i32), torch.arange(E * slot, **i32),
                     torch.ones(E * slot, device="cuda"), ar, ar * slot, cnt, cnt, torch.tensor([E, E * slot], **i32))

    def run(**kw):
        hq = torch.full((E * slot, I), 9, dtype=torch.uint8, device="cuda")
        hs = torch.full((E * slot, I // 32), 9, dtype=torch.uint8, device="cuda")
        Q.gemm_mxfp4(xq, xs, c13, sf13, epilogue=1, plan=plan, act_limit=7.0, out_mx=(hq, hs), w_fp8=w_fp8, **kw)
        out = torch.full((E * slot, H), 3.0, dtype=torch.bfloat16, device="cuda")
        Q.gemm_mxfp4(hq, hs, c2, sf2, out=out, epilogue=2, plan=plan, w_fp8=w_fp8, **kw)
        return hq, hs, out
    hq0, hs0, out0 = run()
    hq1, hs1, out1 = run(slots=(cnt, slot), ntok=sub)
    assert torch.equal(hq0, hq1) and torch.equal(hs0, hs1) and torch.equal(out0, out1)
    for e, c in enumerate(counts):
        r0 = e * slot
        assert int((hq1[r0 + c:r0 + slot] != 9).sum()) == 0 and float((out1[r0 + c:r0 + slot].float() - 3).abs().sum()) == 0
        if c:
            assert float(out1[r0:r0 + c].float().abs().max()) > 0 and float((out1[r0:r0 + c].float() - 3).abs().min()) >= 0


@pytest.mark.parametrize("rows,n,k,dual", [(32, 1408, 2048, False), (7, 256, 512, True), (32, 2048, 1408 - 1408 % 128, False)])
def test_gemm_mxfp4_weights_group_scaled(rows, n, k, dual):
    """MXFP4 weights (e2m1 + UE8M0 per 32) expanded to e4m3 containers, FP8 activations."""
    from ferrule_b200.ops import quant as Q
    from ferrule_b200.ops import reference as ref
    x = rnd(rows, k, scale=1.5, seed=41)
    xq, xs = Q.quant_fp8_rows(x)
    w = torch.randn(n * (2 if dual else 1), k, generator=torch.Generator().manual_seed(42)) * 0.05
    packed, sb = enc.weight_quant_mxfp4(w)
    wq = Q.mxfp4_to_e4m3_containers(packed).cuda()
    out = Q.gemm_fp8(xq, xs, wq, sb.cuda(), epilogue=1 if dual else 0, out_dtype=torch.float32, group32=True)
    xd = enc.act_dequant_fp8(xq.cpu(), xs.cpu())
    wd = enc.weight_dequant_mxfp4(packed, sb)
    y = xd @ wd.T
    r = ref.swiglu(y[:, :n], y[:, n:]) if dual else y
    assert float((out.cpu() - r).abs().max()) <= 3e-3 * float(r.abs().max()) + 1e-4


def _mx_dequant_rows(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    v = enc.e4m3_decode(q.cpu())
    sc = enc.e8m0_decode(s.cpu())
    return (v.view(v.shape[0], -1, 32) * sc.unsqueeze(-1)).view(v.shape)


def test_mxfp8_row_quant_matches_host_codec():
    from ferrule_b200.ops import quant as Q
    x = rnd(37, 512, scale=3.0, seed=71)
    x[3] = 0
    q, s = Q.quant_mxfp8_rows(x)
    xf = x.float().cpu()
    amax = xf.view(37, -1, 32).abs().amax(-1).clamp_min(1e-4)
    sb = enc.e8m0_encode_ceil(amax / 448.0)
    assert torch.equal(s.cpu(), sb)
    qref = enc.e4m3_encode((xf.view(37, -1, 32) / enc.e8m0_decode(sb).unsqueeze(-1)).view(37, -1))
    assert torch.equal(q.cpu(), qref)


def test_mxfp4_scale_blocks_layout():
    from ferrule_b200.ops import quant as Q
    G, rows, k = 2, 200, 512
    sc = torch.randint(100, 140, (G, rows, k // 32), dtype=torch.uint8, device="cuda")
    prep = Q.mxfp4_prepare_sf(sc).cpu()
    assert prep.shape == (G, 2, k // 128, 512)
    s = sc.cpu()
    for g, rt, kb, r, gg, kk in [(0, 0, 0, 0, 0, 0), (1, 0, 3, 31, 3, 2), (0, 1, 1, 5, 1, 3), (1, 1, 2, 7, 2, 0)]:
        row = rt * 128 + gg * 32 + r
        want = int(s[g, row, kb * 4 + kk]) if row < rows else 0x7f
        assert int(prep[g, rt, kb, r * 16 + gg * 4 + kk]) == want


@pytest.mark.parametrize("rows,n,k,dual", [(32, 256, 512, False), (7, 128, 128, False), (16, 256, 1024, True),
                                           (64, 384, 2048, False), (128, 256, 512, False), (32, 2048, 7168, True),
                                           (50, 1408, 2048, False)])
def test_gemm_mxfp4_native_block_scaled(rows, n, k, dual):
    """Packed e2m1 weights + UE8M0/32 scales against MXFP8 activations on the block-scaled tensor-core path,
    compared with the fp32 product of the dequantised operands."""
    from ferrule_b200.ops import _lib
    from ferrule_b200.ops import quant as Q
    from ferrule_b200.ops import reference as ref
    x = rnd(rows, k, scale=1.5, seed=41)
    xq, xs = Q.quant_mxfp8_rows(x)
    w = torch.randn(n * (2 if dual else 1), k, generator=torch.Generator().manual_seed(42)) * 0.05
    parts = [enc.weight_quant_mxfp4(w[r:r + 512]) for r in range(0, w.shape[0], 512)]
    packed, sb = torch.cat([a for a, _ in parts]), torch.cat([b for _, b in parts])
    sf = Q.mxfp4_prepare_sf(sb.cuda())
    out = Q.gemm_mxfp4(xq, xs, packed.cuda(), sf, epilogue=1 if dual else 0, out_dtype=torch.float32)
    # the same weights stored tile-major give the same bits
    out_t = Q.gemm_mxfp4(xq, xs, Q.mxfp4_tile_major(packed.cuda()), sf, epilogue=1 if dual else 0,
                         out_dtype=torch.float32, w_rows=packed.shape[0])
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    assert torch.equal(out, out_t)
    xd = _mx_dequant_rows(xq, xs)
    wd = enc.weight_dequant_mxfp4(packed, sb).float()
    y = xd @ wd.T
    r = ref.swiglu(y[:, :n], y[:, n:]) if dual else y
    err = float((out.cpu() - r).abs().max())
    assert err <= 2e-3 * float(r.abs().max()) + 1e-4, err


def test_gemm_mxfp4_grouped_pipeline_with_requantised_hidden():
    """gate|up (SwiGLU, epilogue re-quantises to MXFP8) -> down (weighted scatter) over a static expert plan with
    empty experts, against the same chain on dequantised operands."""
    from ferrule_b200.ops import _lib
    from ferrule_b200.ops import kernels as K
    from ferrule_b200.ops import quant as Q
    from ferrule_b200.ops import reference as ref
    T, E, topk, H, I, nt = 24, 8, 2, 512, 256, 32
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = torch.randn(T, E, generator=g, device="cuda")
    logits[:, 3] = -1e9                                     # expert 3 receives nothing
    idx, wts = ref.route(logits, topk, 0)
    cnt = torch.zeros(E, dtype=torch.int32, device="cuda")
    plan = K.static_plan(nt, E, cnt)
    x = rnd(T, H, seed=31)
    # place the rows by hand in the static layout (expert e owns rows e * nt ...)
    xg = torch.zeros(E * nt, H, dtype=torch.bfloat16, device="cuda")
    src, dst, scl = plan.src_token.cpu(), plan.dst_row.cpu(), plan.row_scale.cpu()
    counts = [0] * E
    for t in range(T):
        for s_ in range(topk):
            e = int(idx[t, s_])
            r = e * nt + counts[e]
            counts[e] += 1
            xg[r] = x[t]
            src[r], dst[r], scl[r] = t, t * topk + s_, float(wts[t, s_])
    plan.src_token.copy_(src)
    plan.dst_row.copy_(dst)
    plan.row_scale.copy_(scl)
    cnt.copy_(torch.tensor(counts, dtype=torch.int32))
    gen = torch.Generator().manual_seed(9)
    w13 = torch.randn(E, 2 * I, H, generator=gen) * 0.05
    w2 = torch.randn(E, H, I, generator=gen) * 0.05
    p13 = [enc.weight_quant_mxfp4(w13[e]) for e in range(E)]
    p2 = [enc.weight_quant_mxfp4(w2[e]) for e in range(E)]
    w13p, w13s = torch.stack([a for a, _ in p13]).cuda(), Q.mxfp4_prepare_sf(torch.stack([b for _, b in p13]).cuda())
    w2p, w2s = torch.stack([a for a, _ in p2]).cuda(), Q.mxfp4_prepare_sf(torch.stack([b for _, b in p2]).cuda())
    xgq, xgs = Q.quant_mxfp8_rows(xg)
    hq = torch.zeros(E * nt, I, dtype=torch.uint8, device="cuda")
    hs = torch.zeros(E * nt, I // 32, dtype=torch.uint8, device="cuda")
    Q.gemm_mxfp4(xgq, xgs, w13p, w13s, epilogue=1, plan=plan, out_mx=(hq, hs))
    out = torch.zeros(T * topk, H, dtype=torch.float32, device="cuda")
    Q.gemm_mxfp4(hq, hs, w2p, w2s, out=out, epilogue=2, plan=plan, scatter_rows=T * topk)
    torch.cuda.synchronize()
    assert _lib.read_status()[0] == 0
    xd = _mx_dequant_rows(xgq, xgs)
    exp = torch.zeros(T * topk, H)
    for e in range(E):
        if counts[e] == 0:
            continue
        rows = slice(e * nt, e * nt + counts[e])
        w13d = enc.weight_dequant_mxfp4(*p13[e]).float()
        w2d = enc.weight_dequant_mxfp4(*p2[e]).float()
        y = xd[rows] @ w13d.T
        h = enc.bf16_round(ref.swiglu(y[:, :I], y[:, I:]))
        amax = h.view(h.shape[0], -1, 32).abs().amax(-1).clamp_min(1e-4)
        sb = enc.e8m0_decode(enc.e8m0_encode_ceil(amax / 448.0)).unsqueeze(-1)
        hd = (enc.e4m3_decode(enc.e4m3_encode((h.view(h.shape[0], -1, 32) / sb).view(h.shape))).view(h.shape[0], -1, 32) * sb).view(h.shape)
        o = hd @ w2d.T
        for j in range(counts[e]):
            r = e * nt + j
            exp[int(dst[r])] = o[j] * float(scl[r])
    err = float((out.cpu() - exp).abs().max())
    assert err <= 4e-3 * float(exp.abs().max()) + 1e-4, err

