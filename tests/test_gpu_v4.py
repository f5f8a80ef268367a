"""DeepSeek-V4 operator kernels against their fp32 PyTorch oracles."""
import pytest
import torch

from ferrule_b200.models import v4
from ferrule_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("hc,hidden,tokens", [(4, 4096, 5), (2, 256, 3)])
def test_hc_pre_post_match_reference(hc, hidden, tokens):
    from ferrule_b200.ops import v4 as K
    torch.manual_seed(0)
    cfg = v4.HcConfig(hc=hc, hidden=hidden, sinkhorn_iters=20)
    state = torch.randn(tokens, hc, hidden, device=DEV).bfloat16()
    fn = torch.randn(cfg.mix, hc * hidden, device=DEV) * 0.02
    scale = torch.tensor([0.7, 1.1, 0.9], device=DEV)
    base = torch.randn(cfg.mix, device=DEV) * 0.3
    hidden_ref, (pre, post, comb) = v4.hc_pre(state, fn, scale, base, cfg)
    got, coeff = K.hc_pre(state, fn, scale, base, cfg, out_fp32=True)
    torch.cuda.synchronize()
    assert torch.allclose(coeff[:, :hc], pre, atol=2e-5, rtol=1e-4)
    assert torch.allclose(coeff[:, hc:2 * hc], post, atol=2e-5, rtol=1e-4)
    assert torch.allclose(coeff[:, 2 * hc:].view(tokens, hc, hc), comb, atol=2e-5, rtol=1e-4)
    assert torch.allclose(got, hidden_ref, atol=1e-4, rtol=1e-4)
    hid_bf = got.bfloat16()
    out = K.hc_post(hid_bf, state, coeff)
    want = v4.hc_post(hid_bf, state, post, comb)
    assert torch.allclose(out.float(), want, atol=2e-2, rtol=1e-2)
    head_fn = fn[:hc].contiguous()
    hgot, _ = K.hc_pre(state, head_fn, scale, base, cfg, out_fp32=True, head_only=True)
    hwant = v4.hc_head(state, head_fn, scale, base, cfg)
    assert torch.allclose(hgot, hwant, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("ratio,overlap", [(4, True), (128, False)])
def test_compressor_pool_matches_reference(ratio, overlap):
    from ferrule_b200.ops import v4 as K
    torch.manual_seed(1)
    tokens, D = ratio * 5, 512
    od = D * (2 if overlap else 1)
    kv, gate = torch.randn(tokens, od, device=DEV), torch.randn(tokens, od, device=DEV) * 2
    ape = torch.randn(ratio, od, device=DEV)
    got = K.compressor_pool(kv, gate, ape, ratio, overlap)
    want = v4.compressor_pool(kv, gate, ape, ratio, overlap)
    assert got.shape == want.shape == (5, D)
    assert torch.allclose(got.float(), want, atol=1e-2, rtol=1e-2)
    exact = (got.float() == want).float().mean().item()
    assert exact > 0.98       # bf16 rounding of an fp32 sum: only last-ulp ties may differ


def test_rope_rows_forward_then_inverse_is_identity():
    from ferrule_b200.ops import v4 as K
    torch.manual_seed(2)
    cos, sin = ref.rope_tables(64, 64, 10000.0)
    cos, sin = cos.to(DEV), sin.to(DEV)
    x = torch.randn(7, 3, 192, device=DEV).bfloat16()
    pos = torch.tensor([0, 5, 9, 63, 1, 2, 33], dtype=torch.int32, device=DEV)
    y = x.clone()
    K.rope_rows(y, pos, cos, sin, off=128, rdim=64)
    want = x.float().clone()
    want[..., 128:] = ref.apply_rope(x[..., 128:], cos[pos.long()][:, None], sin[pos.long()][:, None])
    assert torch.allclose(y.float(), want, atol=2e-2, rtol=1e-2)
    assert torch.equal(y[..., :128], x[..., :128])
    K.rope_rows(y, pos, cos, sin, off=128, rdim=64, inverse=True)
    assert torch.allclose(y.float(), x.float(), atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("use_gemm", [False, True])
def test_indexer_scores_and_topk_match_reference(use_gemm):
    from ferrule_b200.ops import v4 as K
    torch.manual_seed(3)
    Q, H, d, n, k = 3, 64, 128, 3000, 512
    q = torch.randn(Q, H, d, device=DEV).bfloat16()
    plane = torch.randn(n, d, device=DEV).bfloat16()
    w = torch.randn(Q, H, device=DEV)
    scores = K.indexer_scores(q, plane, w, use_gemm=use_gemm)       # SIMT kernel / tcgen05 GEMM + head reduction
    vis = torch.tensor([n, 700, 100], dtype=torch.int32, device=DEV)
    idx = K.indexer_topk(scores, k, vis)
    torch.cuda.synchronize()
    for i in range(Q):
        _, s_ref = v4.indexer_topk(q[i], plane, w[i], k, int(vis[i]))
        # scores: fp32 accumulation order differs -> allow one bf16 ulp on a small share
        close = torch.isclose(scores[i], s_ref, rtol=1.6e-2, atol=1e-2)
        assert close.float().mean() > 0.999
        # top-k exactness is checked on the kernel's own scores (the selection contract)
        cand = scores[i, :int(vis[i])]
        order = torch.sort(cand, descending=True, stable=True).indices[:k].int()
        want = torch.full((k,), -1, dtype=torch.int32, device=DEV)
        want[:order.numel()] = order
        assert torch.equal(idx[i], want)


def test_indexer_topk_ties_and_nonfinite():
    from ferrule_b200.ops import v4 as K
    s = torch.zeros(1, 2000, device=DEV)
    s[0, 5] = float("nan")
    s[0, 100:110] = 2.0
    s[0, 7] = float("inf")
    s[0, 1500] = -1.0
    idx = K.indexer_topk(s, 16)
    assert idx[0].tolist() == list(range(100, 110)) + [0, 1, 2, 3, 4, 6]


@pytest.mark.parametrize("splits", [1, 4])
def test_selection_attention_matches_reference(splits):
    from ferrule_b200.ops import v4 as K
    torch.manual_seed(4)
    rows, heads, DL, DR, n, W = 5, 16, 512, 64, 4096, 640
    D = DL + DR
    table = (torch.randn(n, D, device=DEV) * 0.5).bfloat16()
    q = (torch.randn(rows, heads, D, device=DEV) * 0.5).bfloat16()
    sel = torch.stack([torch.randperm(n, device=DEV)[:W] for _ in range(rows)]).int()
    sel[:, 17] = -1
    sel[2, 300:] = -1
    sink = torch.randn(heads, device=DEV)
    got = K.sparse_sink_attention(q, table, sel, DL, DR, 0.07, sink=sink, splits=splits)
    want = v4.sparse_sink_attention(q, table, sel, DL, 0.07, sink=sink)
    torch.cuda.synchronize()
    assert torch.allclose(got.float(), want, atol=2e-2, rtol=2e-2)


def test_v4_model_decode_matches_reference():
    """The assembled DeepSeek-V4 layer stack (hyper-connections, window + compressed + indexed attention, grouped
    output projection, hash / sqrt-softplus MoE): CUDA decode steps of two ragged sequences against the oracle."""
    from ferrule_b200.models import v4_model as M
    from ferrule_b200.ops import _lib
    cfg = M.tiny_v4()
    w_cpu = M.random_v4_weights(cfg, device="cpu", seed=0)
    w_gpu = M.random_v4_weights(cfg, device=DEV, seed=0)
    ref_model = M.V4Reference(w_cpu)
    caches = [M.V4SeqCache(cfg), M.V4SeqCache(cfg)]
    cuda_model = M.V4Cuda(w_gpu, max_seqs=2, max_len=64)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (2, 30), generator=g)
    worst = 0.0
    agree = total = 0
    for t in range(30):
        seqs = [0, 1] if t < 22 else [0]                      # the second sequence stops early
        want = torch.stack([ref_model.step(caches[s], int(toks[s, t])) for s in seqs])
        nxt, logits = cuda_model.step(seqs, [int(toks[s, t]) for s in seqs])
        torch.cuda.synchronize()
        err = float((logits.cpu() - want).abs().max())
        scale = float(want.abs().max())
        worst = max(worst, err / scale)
        top2 = want.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 3 * err
        agree += int((nxt.cpu()[clear].long() == want.argmax(-1)[clear]).sum())
        total += int(clear.sum())
    _lib.raise_on_status()
    assert worst <= 0.08, worst
    assert agree == total and total > 20
    # the compressed tables were filled: ratio-4 layer has 30 // 4 rows, ratio-8 layer 30 // 8
    assert len(caches[0].comp[1]) == 7 and len(caches[0].comp[2]) == 3
    got = cuda_model.tables[1][0, 64:64 + 7].float().cpu()
    assert torch.allclose(got, torch.stack(caches[0].comp[1]), atol=0.08, rtol=0.05)


def test_v4_prompt_chunks_in_one_pass_match_token_by_token():
    """Two prompt chunks and a decode row as ONE batch of rows through the kernels against the same rows fed one
    at a time: same tables (window, compressed, indexer plane), same next tokens."""
    from ferrule_b200.models import v4_model as M
    from ferrule_b200.ops import _lib
    cfg = M.tiny_v4()
    w = M.random_v4_weights(cfg, device=DEV, seed=1)
    g = torch.Generator().manual_seed(3)
    a, b, c = (torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (21, 13, 9))
    one = M.V4Cuda(w, max_seqs=3, max_len=64)
    many = M.V4Cuda(w, max_seqs=3, max_len=64, max_rows=64)
    for m in (one, many):
        for t in c[:8]:
            m.step([2], [t])
        for t in a[:6]:
            m.step([0], [t])
    last = {}
    for t in a[6:]:
        last[0] = one.step([0], [t])[1][0].clone()
    for t in b:
        last[1] = one.step([1], [t])[1][0].clone()
    last[2] = one.step([2], [c[8]])[1][0].clone()
    seqs = [0] * 15 + [1] * 13 + [2]
    pos = list(range(6, 21)) + list(range(13)) + [8]
    nxt, logits = many.step_rows(seqs, a[6:] + b + [c[8]], pos, want_rows=[14, 27, 28])
    torch.cuda.synchronize()
    _lib.raise_on_status()
    assert logits.shape[0] == 3 and many.positions == one.positions == [21, 13, 9]
    for k in range(3):
        scale = float(last[k].abs().max())
        assert float((logits[k] - last[k]).abs().max()) <= 0.03 * scale
        top2 = last[k].topk(2).values
        if float(top2[0] - top2[1]) > 0.1 * scale:
            assert int(nxt[k]) == int(last[k].argmax())
    for layer in range(cfg.n_layers):
        assert torch.allclose(many.tables[layer].float(), one.tables[layer].float(), atol=0.03, rtol=0.03)
    assert torch.allclose(many.iplane[1].float(), one.iplane[1].float(), atol=0.03, rtol=0.03)
    assert float(many.tables[1][0, 64:64 + 5].abs().max()) > 0 and float(many.iplane[1][1, :3].abs().max()) > 0


def test_v4_decode_with_qat_steps_on_the_kernels():
    """QAT checkpoints: the rows the kernels read are the quantised ones (FP8 window / compressed rows, FP4
    indexer plane), batched and one-at-a-time decoding agree, and the stream follows the oracle's wherever the
    oracle's choice is clear."""
    from ferrule_b200.io import encoding as enc
    from ferrule_b200.models import v4_model as M
    from ferrule_b200.ops import _lib
    cfg = M.tiny_v4().with_(qat=True)
    w_cpu = M.random_v4_weights(cfg, device="cpu", seed=0)
    w_gpu = M.random_v4_weights(cfg, device=DEV, seed=0)
    ref_model = M.V4Reference(w_cpu)
    caches = [M.V4SeqCache(cfg), M.V4SeqCache(cfg)]
    both = M.V4Cuda(w_gpu, max_seqs=2, max_len=64)
    solo = M.V4Cuda(w_gpu, max_seqs=1, max_len=64)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (2, 24), generator=g)
    agree = total = 0
    for t in range(24):
        want = torch.stack([ref_model.step(caches[s], int(toks[s, t])) for s in (0, 1)])
        nxt, logits = both.step([0, 1], [int(toks[0, t]), int(toks[1, t])])
        one, _ = solo.step([0], [int(toks[0, t])])
        torch.cuda.synchronize()
        assert torch.isfinite(logits).all()
        assert int(one[0]) == int(nxt[0]), "a sequence decodes the same alone and in a batch"
        top2 = want.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 0.25 * float(want.abs().max())
        agree += int((nxt.cpu()[clear].long() == want.argmax(-1)[clear]).sum())
        total += int(clear.sum())
    _lib.raise_on_status()
    assert agree == total
    rd = cfg.rope_dim
    for layer in range(cfg.n_layers):
        rows = both.tables[layer][0, :24].float().cpu()
        assert torch.equal(v4.qat_kv_rows(rows, rd), rows), "window rows are stored quantised"
    comp = both.tables[1][0, 64:64 + 6].float().cpu()
    assert torch.equal(v4.qat_kv_rows(comp, rd), comp) and float(comp.abs().max()) > 0
    plane = both.iplane[1][0, :6].float().cpu()
    assert torch.equal(enc.fp4_qat(plane, 32), plane) and float(plane.abs().max()) > 0


def test_markov_head_and_mean_taps_match_reference():
    from ferrule_b200.ops import v4 as K
    torch.manual_seed(5)
    vocab, rank, gamma = 129280, 64, 5
    logits = torch.randn(gamma, vocab, device=DEV)
    w1 = (torch.randn(vocab, rank, device=DEV) * 0.3).bfloat16()
    w2 = (torch.randn(vocab, rank, device=DEV) * 0.3).bfloat16()
    anchor = torch.tensor([1234], dtype=torch.int32, device=DEV)
    ids, vals = K.markov_head(logits, w1, w2, anchor)
    want_ids, want_vals = v4.markov_head(logits, w1, w2, 1234)
    torch.cuda.synchronize()
    assert ids.tolist() == want_ids
    assert torch.allclose(vals.cpu(), torch.tensor(want_vals), atol=1e-3)
    state = torch.randn(7, 4, 256, device=DEV).bfloat16()
    taps = torch.zeros(7, 3 * 256, dtype=torch.bfloat16, device=DEV)
    K.hc_mean_scatter(state, taps, 1)
    want = v4.hc_mean_taps([state], 4)
    assert torch.equal(taps[:, 256:512].float(), want) and float(taps[:, :256].abs().max()) == 0.0
