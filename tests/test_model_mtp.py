"""MTP proposal head on the real model runner (CPU reference path): speculative decoding must emit
exactly the greedy stream, the MTP layer's KV rows must follow the published positions."""
import torch

from ferrule_b200.models import config as C
from ferrule_b200.models import weights as W
from ferrule_b200.models.runner import DeepSeekRunner
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest


def _engine(speculative: bool, w):
    runner = DeepSeekRunner(w, n_pages=48, page_size=16, max_rows=128, max_seqs=4, max_seq_len=256, device="cpu")
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=64, prefill_chunk_size=24,
                            ctx_size=256)
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=48, page_size=16, speculative=speculative,
                                       max_draft=1, confidence_threshold=0.0)), runner


def _run(eng, prompts, n_new):
    for i, p in enumerate(prompts):
        eng.submit(GenerateRequest(f"r{i}", p, max_new_tokens=n_new, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=5000)
    return {f"r{i}": [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == f"r{i}"]
            for i in range(len(prompts))}


def test_mtp_speculation_equals_greedy_on_tiny_fixture():
    cfg = C.tiny_fixture()
    w = W.random_weights(cfg, device="cpu", seed=0)
    assert w.mtp, "the fixture carries one MTP stage"
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (16, 37, 50)]
    base, _ = _engine(False, w)
    spec, runner = _engine(True, w)
    want = _run(base, prompts, 12)
    got = _run(spec, prompts, 12)
    assert got == want
    m = spec.spec.metrics
    assert m.drafted > 0 and runner.stats.mtp_proposals > 0
    assert m.accepted <= m.drafted
    spec.kv.check_invariants()
    assert spec.kv.stats().used_pages == 0


def test_mtp_rows_follow_published_positions():
    cfg = C.tiny_fixture()
    w = W.random_weights(cfg, device="cpu", seed=1)
    eng, runner = _engine(True, w)
    eng.submit(GenerateRequest("a", list(range(1, 30)), max_new_tokens=4, ignore_eos=True))
    seen = []
    orig = runner.propose

    def spy(slots, anchors, positions, views, max_draft):
        before = {s: (runner._mtp[s].next_pos, len(runner._mtp[s].tokens)) for s in slots if s in runner._mtp}
        out = orig(slots, anchors, positions, views, max_draft)
        for s, pos in zip(slots, positions):
            if s in before:
                seen.append((before[s], pos, runner._mtp[s].next_pos))
        return out

    runner.propose = spy
    eng.run_until_idle(lambda e: None, max_steps=2000)
    assert seen, "the engine asked for proposals"
    (first_pos0, first_n), pos, after = seen[0]
    assert first_pos0 == 0 and first_n == 29 and pos == 29 and after == 29     # whole prompt queued, then written
    for (p0, n), pos, after in seen[1:]:
        assert p0 + n == pos and after == pos                                  # contiguous afterwards


def test_zipf_router_bias_skews_expert_popularity():
    """`random_weights(router_zipf=s)`: unit-variance router logits plus a Zipf selection bias - the routed-expert
    histogram becomes skewed (the head of the popularity order takes most routes) while every token still
    chooses by its own logits (different tokens pick different experts)."""
    import torch
    from ferrule_b200.models import config as C, weights as W
    from ferrule_b200.models.weights import zipf_router_bias
    from ferrule_b200.ops import reference as ref
    b = zipf_router_bias(64, 1.1, seed=3)
    assert abs(float(b.mean())) < 1e-6 and float(b.abs().max()) <= 0.5 + 1e-6 and len(set(b.tolist())) == 64
    assert torch.equal(b, zipf_router_bias(64, 1.1, seed=3)) and not torch.equal(b, zipf_router_bias(64, 1.1, seed=4))
    cfg = C.deepseek_v2_lite().with_(n_layers=2, vocab_size=1024, score_fn=1, router_bias=True)
    w = W.random_weights(cfg, device="cpu", seed=0, router_zipf=1.1)
    lw = w.layers[1]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(2000, cfg.hidden, generator=g)
    x = x / x.pow(2).mean(-1, keepdim=True).sqrt()
    logits = x @ lw.router_w.float().T
    assert 0.8 < float(logits.std()) < 1.25
    idx, _ = ref.route(logits, cfg.topk, cfg.score_fn, bias=lw.router_bias)
    hist = torch.bincount(idx.flatten(), minlength=cfg.n_routed_experts).float()
    top = hist.sort(descending=True).values
    assert float(top[:8].sum() / hist.sum()) > 0.25 > 8 / 64 and int((hist > 0).sum()) > 32
    assert len({tuple(r) for r in idx[:50].tolist()}) > 25
