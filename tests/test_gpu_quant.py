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
