"""Randomised soak of the DeepSeek runner behind the engine (CPU reference path, real weights): ragged requests,
a retained session, shared prompt prefixes, cancellations, a small KV pool - crossed with speculative decoding
(MTP drafts), asynchronously streamed experts at half residency with transaction prefetch, the prompt-prefix cache
and auto-preemption.  Every request that ran to its length limit must have streamed exactly the tokens of the
plain resident model; nothing may be left behind (pages, slots, arena leases, continuations).

The streamed configurations are what exercises frame contention: several parked transactions that each lease
some frames and wait for one more (the engine rolls back all but the oldest), and loads that must not evict a
payload installed for a transaction that has not resumed yet."""
import random

import pytest
import torch

from ferrule_b200.models import config as C
from ferrule_b200.models import weights as W
from ferrule_b200.models.runner import DeepSeekRunner
from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest

cfg = C.tiny_fixture().with_(n_mtp_layers=1)
_cache = {}


def plain_engine():
    w = W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2)
    runner = DeepSeekRunner(w, n_pages=64, page_size=16, max_rows=64, max_seqs=4, max_seq_len=128, device="cpu", enable_mtp=False)
    sched = SchedulerConfig(max_active_sequences=1, max_decode_batch=1, max_batch_tokens=64, prefill_chunk_size=64, ctx_size=128)
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=64, page_size=16))


_ref = None


def greedy(prompt, n):
    global _ref
    key = (tuple(prompt), n)
    if key in _cache:
        return _cache[key]
    if _ref is None:
        _ref = plain_engine()
    _ref.submit(GenerateRequest("g", prompt, max_new_tokens=n, ignore_eos=True))
    ev = []
    _ref.run_until_idle(ev.append)
    out = [e.token for e in ev if isinstance(e, TokenEvent)]
    _cache[key] = out
    return out


def _soak(seed, spec, stream, prefix):
    rnd = random.Random(seed)
    w = W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2)
    runner = DeepSeekRunner(w, n_pages=14, page_size=16, max_rows=64, max_seqs=3, max_seq_len=128, device="cpu",
                            enable_mtp=spec, expert_residency=0.5 if stream else None, async_streaming=stream)
    sched = SchedulerConfig(max_active_sequences=3, max_decode_batch=3, max_batch_tokens=24, prefill_chunk_size=8, ctx_size=128)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=14, page_size=16, speculative=spec, max_draft=1,
                                      confidence_threshold=0.0, auto_preempt=rnd.random() < 0.5,
                                      prefix_cache_tokens=64 if prefix else 0, prefix_block=16,
                                      transaction_prefetch=2 if stream else 0),
                 registry=runner.make_registry() if stream else None)
    prompts, toks, fins, n = {}, {}, {}, 0
    ev = []
    base = [rnd.randrange(1, cfg.vocab_size) for _ in range(20)]
    for _ in range(100):
        a = rnd.random()
        if a < 0.3 and len(prompts) - len(fins) < 5:
            rid, n = f"r{n}", n + 1
            p = (base[:16] if rnd.random() < 0.4 else []) + [rnd.randrange(1, cfg.vocab_size) for _ in range(rnd.randrange(1, 14))]
            k = rnd.randrange(0, 6)
            sid = rnd.choice([None, None, None, "a"])
            try:
                eng.submit(GenerateRequest(rid, p, max_new_tokens=k, ignore_eos=True, session_id=sid, retain_session=bool(sid)))
                prompts[rid] = (p, k, sid)
            except ValueError:
                pass
        elif a < 0.34:
            live = [r for r in prompts if r not in fins]
            if live:
                eng.cancel_request(rnd.choice(live))
        elif a < 0.36:
            eng.reset_session("a")
        eng.step(ev.append)
        for e in ev:
            if isinstance(e, TokenEvent):
                toks.setdefault(e.request_id, []).append(e.token)
            elif isinstance(e, FinishEvent):
                fins[e.request_id] = e
        ev.clear()
        eng.kv.check_invariants()
    assert eng.run_until_idle(ev.append, max_steps=5000) < 5000
    for e in ev:
        if isinstance(e, TokenEvent):
            toks.setdefault(e.request_id, []).append(e.token)
        elif isinstance(e, FinishEvent):
            fins[e.request_id] = e
    assert eng.last_error is None or "KV pool" in str(eng.last_error) or getattr(eng.last_error, "retryable", False), eng.last_error
    for rid, (p, k, sid) in prompts.items():
        f = fins[rid]
        if sid is None and f.reason == FinishReason.MAX_TOKENS:
            assert toks.get(rid, []) == greedy(p, k), (seed, spec, stream, prefix, rid, toks.get(rid), greedy(p, k))
    for sid in list(eng._sessions):
        eng.reset_session(sid)
    assert eng.shutdown()
    st = eng.kv.stats()
    assert st.used_pages == 0, (st,)
    if stream:
        for la in runner.arena.layers.values():
            assert all(s.leases == 0 for s in la.coord.slots)
        assert eng.registry.residual().get("continuations", 0) == 0


@pytest.mark.parametrize("spec,stream", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("seed", [0, 5, 11])
def test_deepseek_soak(seed, spec, stream):
    _soak(seed, spec, stream, prefix=seed % 2 == 0)
