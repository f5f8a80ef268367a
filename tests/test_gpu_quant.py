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
