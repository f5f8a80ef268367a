"""DeepSeek-V4 proposal attachment: block protocol, the non-causal block attention over context window + block
rows, the Markov / confidence heads, and speculative decoding through the engine (the stream must stay the
greedy stream whatever the drafts are worth)."""
import pytest
import torch

from ferrule_b200.models import v4
from ferrule_b200.models.v4_model import V4Reference, V4SeqCache, random_v4_weights, tiny_v4
from ferrule_b200.models.v4_runner import V4Runner
from ferrule_b200.ops import reference as ref
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.runner import Proposal
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest


def _cfg(**kw):
    return tiny_v4().with_(n_proposal_stages=2, proposal_target_layers=(0, 2), proposal_noise_token=3,
                           proposal_markov_rank=16, **kw)


def _fed(w, n, seed=0):
    r = V4Reference(w)
    c = V4SeqCache(w.cfg)
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, w.cfg.vocab_size, (n,), generator=g).tolist()
    for t in toks:
        logits = r.step(c, t)
    return r, c, toks, logits


def test_block_protocol_rows():
    w = random_v4_weights(_cfg(), seed=1)
    p = V4Reference(w).proposal
    assert p.gamma == 5 and p.draft_input_ids(41) == [41, 3, 3, 3, 3]
    assert p.target_rows_for_drafts(5) == 6 and p.target_rows_for_drafts(0) == 1
    with pytest.raises(ValueError):
        p.target_rows_for_drafts(6)
    bad = random_v4_weights(_cfg(), seed=1)
    bad.proposal.main_proj = bad.proposal.main_proj[:, :-1]
    with pytest.raises(ValueError):
        V4Reference(bad)


def test_every_target_row_leaves_one_context_row_per_stage():
    w = random_v4_weights(_cfg(), seed=2)
    r, c, toks, _ = _fed(w, 13)
    assert [len(rows) for rows in c.pctx] == [13, 13]
    # the row is stage wkv -> norm -> RoPE of the projected taps: recompute position 0 from scratch
    c0 = V4SeqCache(w.cfg)
    r.step(c0, toks[0])
    assert torch.equal(c0.pctx[1][0], c.pctx[1][0])
    # two stages have different wkv: different rows
    assert not torch.equal(c.pctx[0][5], c.pctx[1][5])


def test_block_attention_sees_window_of_context_and_the_whole_block():
    w = random_v4_weights(_cfg(), seed=3)
    cfg = w.cfg
    r, c, _, _ = _fed(w, 20)
    p = r.proposal
    ctx = [torch.stack(rows) for rows in c.pctx]
    ids = p.draft_input_ids(17)
    base = p.block_hidden(ctx, 20, ids)
    assert base.shape == (5, cfg.hidden)
    # not causal: the LAST block token changes the FIRST row
    other = p.block_hidden(ctx, 20, ids[:-1] + [9])
    assert not torch.equal(other[0], base[0])
    # context rows older than the window are not read ...
    old = [t.clone() for t in ctx]
    for t in old:
        t[:20 - cfg.window] = 7.0
    assert torch.equal(p.block_hidden(old, 20, ids), base)
    # ... rows inside it are ...
    near = [t.clone() for t in ctx]
    near[0][19] += 1.0
    assert not torch.equal(p.block_hidden(near, 20, ids), base)
    # ... and rows at or past the committed length (a rejected draft's leftovers) are not
    longer = [torch.cat([t, torch.full((3, t.shape[1]), 5.0)]) for t in ctx]
    assert torch.equal(p.block_hidden(longer, 20, ids), base)


def test_block_attention_matches_a_plain_softmax_with_sink():
    w = random_v4_weights(_cfg(), seed=4)
    cfg = w.cfg
    r, c, _, _ = _fed(w, 6)
    p = r.proposal
    lw = w.proposal.stages[0]
    g = torch.Generator().manual_seed(5)
    xn = ref.bf16_round(torch.randn(5, cfg.hidden, generator=g))
    ctx = torch.stack(c.pctx[0])
    pos = torch.arange(6, 11)
    got = p._attention(lw, xn, ctx, pos)
    # the same thing, row by row, with explicit tensors
    rnd = ref.bf16_round
    hd, rd, nh = cfg.head_dim, cfg.rope_dim, cfg.n_heads
    cos, sin = p.rope
    keys = []
    for j in range(5):
        kv = rnd(ref.rmsnorm(rnd(xn[j] @ lw.wkv.float().T)[None], lw.kv_norm, cfg.norm_eps))[0]
        kv = kv.clone()
        kv[-rd:] = ref.apply_rope(kv[-rd:], cos[6 + j], sin[6 + j])
        keys.append(rnd(kv))
    table = torch.cat([ctx, torch.stack(keys)])
    for j in range(5):
        qn = rnd(ref.rmsnorm(rnd(xn[j] @ lw.wq_a.float().T)[None], lw.q_norm, cfg.norm_eps))[0]
        q = rnd(ref.rmsnorm(rnd(qn @ lw.wq_b.float().T).view(nh, hd), None, cfg.norm_eps)).clone()
        q[:, -rd:] = ref.apply_rope(q[:, -rd:], cos[6 + j], sin[6 + j])
        q = rnd(q)
        logit = q @ table.T * cfg.softmax_scale
        full = torch.cat([logit, lw.sink.float()[:, None]], dim=1)
        prob = rnd(torch.softmax(full, -1)[:, :-1])
        o = rnd(prob @ table).clone()
        o[:, -rd:] = ref.apply_rope(o[:, -rd:], cos[6 + j], sin[6 + j], inverse=True)
        o = rnd(o)
        lat = rnd(torch.einsum("gk,gnk->gn", o.reshape(cfg.o_groups, cfg.group_in), lw.wo_a.float())).reshape(-1)
        want = rnd(lat @ lw.wo_b.float().T)
        assert torch.allclose(got[j], want, atol=2e-2 * float(want.abs().max()) + 1e-3)


def test_markov_chain_and_confidence_heads():
    w = random_v4_weights(_cfg(), seed=6)
    cfg = w.cfg
    p = V4Reference(w).proposal
    g = torch.Generator().manual_seed(7)
    hn = ref.bf16_round(torch.randn(5, cfg.hidden, generator=g))
    drafts, conf = p.heads(hn, anchor=11)
    logits = hn @ w.lm_head.float().T
    prev = 11
    cw = w.proposal.confidence_proj.float()[0]
    for j in range(5):
        biased = logits[j] + w.proposal.markov_w2.float() @ w.proposal.markov_w1[prev].float()
        assert drafts[j] == int(torch.argmax(biased))
        want = float(hn[j] @ cw[:cfg.hidden] + w.proposal.markov_w1[prev].float() @ cw[cfg.hidden:])
        assert abs(conf[j] - want) < 1e-4
        prev = drafts[j]
    # the chain matters: another anchor moves the first draft's bias
    assert p.heads(hn, anchor=12)[1][0] != conf[0]
    assert v4.markov_head(logits, w.proposal.markov_w1, w.proposal.markov_w2, 11)[0] == drafts


def _greedy(w, prompt, n_new):
    r = V4Reference(w)
    c = V4SeqCache(w.cfg)
    for t in prompt:
        logits = r.step(c, t)
    out = []
    for _ in range(n_new):
        t = int(torch.argmax(logits))
        out.append(t)
        logits = r.step(c, t)
    return out


def _spec_engine(w, **kw):
    runner = V4Runner(w, n_pages=48, page_size=16, max_seqs=4, max_seq_len=128, max_rows=64)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=12,
                            ctx_size=128)
    cfg = EngineConfig(scheduler=sched, kv_pages=48, page_size=16, speculative=True, max_draft=5,
                       confidence_threshold=0.0, **kw)
    return Engine(runner, cfg), runner


def _run(eng, prompts, n_new):
    for i, p in enumerate(prompts):
        eng.submit(GenerateRequest(f"r{i}", p, max_new_tokens=n_new, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=5000)
    return [[e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == f"r{i}"] for i in range(len(prompts))]


def test_speculative_v4_stream_is_the_greedy_stream_on_cpu():
    w = random_v4_weights(_cfg(), device="cpu", seed=3)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, w.cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 20, 14)]
    eng, runner = _spec_engine(w)
    got = _run(eng, prompts, 10)
    for p, toks in zip(prompts, got):
        assert toks == _greedy(w, p, 10)
    m = eng.spec.metrics
    assert m.cycles > 0 and m.drafted > 0 and runner.proposal_blocks > 0
    assert m.emitted == sum(len(t) for t in got) - len(prompts)      # the first token of a request comes from prefill
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0


@pytest.mark.parametrize("good", [0, 2, 5])
def test_partly_accepted_blocks_rewind_the_slot_state(good):
    """Drafts that are right for `good` tokens and wrong after: the accepted rows stay, the rejected rows'
    window / compressor / proposal-context entries are overwritten when their positions run again."""
    w = random_v4_weights(_cfg(), device="cpu", seed=5)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, w.cfg.vocab_size, (11,), generator=g).tolist()
    want = _greedy(w, prompt, 16)
    eng, runner = _spec_engine(w)

    def teacher(slots, anchors, positions, views, max_draft):
        k = positions[0] - len(prompt)                 # the anchor is want[k]
        assert anchors[0] == want[k]
        truth = want[k + 1:k + 1 + max_draft]
        drafts = [t if j < good else (t + 1) % w.cfg.vocab_size for j, t in enumerate(truth)]
        return [Proposal(drafts, [9.0] * len(drafts))]

    runner.propose = teacher
    got = _run(eng, [prompt], 16)[0]
    assert got == want
    m = eng.spec.metrics
    if good:
        assert m.accepted > 0 and max(m.accepted_prefix_hist) == good
    else:
        assert m.accepted == 0
    # the oracle cache of the slot ended exactly at the committed length (nothing of a rejected row survives)
    assert eng.kv.stats().used_pages == 0


@pytest.mark.gpu
def test_speculative_v4_stream_is_the_greedy_stream_on_the_kernels():
    w = random_v4_weights(_cfg(), device="cuda", seed=3)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, w.cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 20, 14)]
    eng, runner = _spec_engine(w)
    got = _run(eng, prompts, 10)
    plain_runner = V4Runner(w, n_pages=48, page_size=16, max_seqs=4, max_seq_len=128, max_rows=64)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=12,
                            ctx_size=128)
    plain = Engine(plain_runner, EngineConfig(scheduler=sched, kv_pages=48, page_size=16))
    assert got == _run(plain, prompts, 10)
    m = eng.spec.metrics
    assert m.cycles > 0 and m.drafted > 0 and runner.proposal_blocks > 0
    from ferrule_b200.ops import _lib
    assert _lib.read_status()[0] == 0


# ---------------------------------------------------------------------------------------------- QAT steps
def test_qat_row_operators():
    from ferrule_b200.io import encoding as enc
    g = torch.Generator().manual_seed(11)
    rows = ref.bf16_round(torch.randn(3, 192, generator=g) * 3)
    out = v4.qat_kv_rows(rows, rope_dim=64)
    assert torch.equal(out[:, 128:], rows[:, 128:]), "the rotary tail is not quantised"
    assert torch.equal(out[:, :128], enc.fp8_qat(rows[:, :128], 64))
    assert torch.equal(v4.qat_kv_rows(out, 64), out), "quantising representable values changes nothing"
    # 48 non-rotary features do not divide into blocks of 64: one scale per row
    odd = ref.bf16_round(torch.randn(2, 64, generator=g))
    assert torch.equal(v4.qat_kv_rows(odd, 16)[:, :48], enc.fp8_qat(odd[:, :48], 48))
    # power-of-two scale from ceil(log2(amax / 448)): a block whose amax is 448 * 2^k keeps it exactly
    blk = torch.zeros(1, 64)
    blk[0, 0], blk[0, 1] = 448.0 * 4, 3.0
    assert torch.equal(enc.fp8_qat(blk, 64), blk)
    x = ref.bf16_round(torch.randn(4, 32, generator=g))
    y = v4.qat_indexer_rows(x)
    want = enc.fp4_qat(enc.bf16_round(enc.hadamard(x)), 32)
    assert torch.equal(y, want)
    # every value is an e2m1 magnitude times the row's power-of-two scale
    mags = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    for r in range(4):
        scale = 2.0 ** torch.ceil(torch.log2(want[r].abs().max() / 6.0))
        assert all(bool(((v.abs() / scale)[None] == mags).any()) for v in want[r])
    lin = ref.bf16_round(torch.randn(2, 256, generator=g))
    assert torch.equal(v4.qat_linear_input(lin), enc.fp8_qat(lin, 128))


def test_qat_steps_run_inside_the_v4_step():
    cfg = _cfg(qat=True)
    w = random_v4_weights(cfg, seed=8)
    r, c, toks, logits = _fed(w, 17)
    plain = V4Reference(random_v4_weights(_cfg(), seed=8))
    c2 = V4SeqCache(plain.cfg)
    for t in toks:
        logits2 = plain.step(c2, t)
    # same weights, another function: close, not equal
    assert not torch.equal(logits, logits2)
    assert float((logits - logits2).abs().max()) < 0.35 * float(logits2.abs().max())
    rd = cfg.rope_dim
    from ferrule_b200.io import encoding as enc
    for layer in range(cfg.n_layers):
        kv = torch.stack(c.kv[layer])
        assert torch.equal(v4.qat_kv_rows(kv, rd), kv), "window rows are stored quantised"
        if c.comp[layer]:
            comp = torch.stack(c.comp[layer])
            assert torch.equal(v4.qat_kv_rows(comp, rd), comp)
        if c.icomp[layer]:
            ic = torch.stack(c.icomp[layer])
            assert torch.equal(enc.fp4_qat(ic, 32), ic), "the indexer plane holds FP4 values"
    for rows in c.pctx:
        ctx = torch.stack(rows)
        assert torch.equal(v4.qat_kv_rows(ctx, rd), ctx)
    assert not torch.equal(torch.stack(c.kv[0]), torch.stack(c2.kv[0]))


def test_speculative_v4_with_qat_is_the_greedy_stream_on_cpu():
    w = random_v4_weights(_cfg(qat=True), device="cpu", seed=3)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, w.cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 13)]
    eng, runner = _spec_engine(w)
    got = _run(eng, prompts, 8)
    for p, toks in zip(prompts, got):
        assert toks == _greedy(w, p, 8)
    assert eng.spec.metrics.drafted > 0
