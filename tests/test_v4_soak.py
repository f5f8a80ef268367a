"""Randomised soak of the DeepSeek-V4 runner behind the engine (CPU oracle path): ragged requests, retained sessions
that keep their slot, cancellations, session resets, a pool small enough to stall, with and without speculative
decoding by the checkpoint's block drafter and with or without auto-preemption.  Every request that ran to its
length limit must have streamed exactly the oracle's greedy tokens, and nothing may be left behind."""
import random

import pytest
import torch

from ferrule_b200.models.v4_model import V4Reference, V4SeqCache, random_v4_weights, tiny_v4
from ferrule_b200.models.v4_runner import V4Runner
from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest

cfg = tiny_v4().with_(n_proposal_stages=1, proposal_target_layers=(0, 2), proposal_noise_token=3, proposal_markov_rank=8)
_cache = {}


def _weights():
    if "w" not in _cache:
        _cache["w"] = random_v4_weights(cfg, seed=3)
    return _cache["w"]


def greedy(prompt, n):
    key = (tuple(prompt), n)
    if key in _cache:
        return _cache[key]
    w = _weights()
    r, c = V4Reference(w), V4SeqCache(cfg)
    for t in prompt:
        logits = r.step(c, t)
    out = []
    for _ in range(n):
        out.append(int(torch.argmax(logits)))
        logits = r.step(c, out[-1])
    _cache[key] = out
    return out


def _soak(seed, spec):
    rnd = random.Random(seed)
    w = _weights()
    runner = V4Runner(w, n_pages=10, page_size=16, max_seqs=3, max_seq_len=96, max_rows=48)
    sched = SchedulerConfig(max_active_sequences=3, max_decode_batch=3, max_batch_tokens=24, prefill_chunk_size=8, ctx_size=96)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=10, page_size=16, speculative=spec, max_draft=5,
                                      confidence_threshold=0.0, auto_preempt=rnd.random() < 0.5))
    prompts, toks, fins, n = {}, {}, {}, 0
    ev = []
    for _ in range(120):
        a = rnd.random()
        if a < 0.3 and len(prompts) - len(fins) < 5:
            rid, n = f"r{n}", n + 1
            p = [rnd.randrange(1, cfg.vocab_size) for _ in range(rnd.randrange(1, 20))]
            k = rnd.randrange(0, 7)
            sid = rnd.choice([None, None, "a", "b"])
            try:
                eng.submit(GenerateRequest(rid, p, max_new_tokens=k, ignore_eos=True, session_id=sid, retain_session=bool(sid)))
                prompts[rid] = (p, k, sid)
            except ValueError:
                pass
        elif a < 0.35:
            live = [r for r in prompts if r not in fins]
            if live:
                eng.cancel_request(rnd.choice(live))
        elif a < 0.38:
            eng.reset_session(rnd.choice(["a", "b"]))
        eng.step(ev.append)
        for e in ev:
            if isinstance(e, TokenEvent):
                toks.setdefault(e.request_id, []).append(e.token)
            elif isinstance(e, FinishEvent):
                fins[e.request_id] = e
        ev.clear()
        eng.kv.check_invariants()
    assert eng.run_until_idle(ev.append, max_steps=3000) < 3000
    for e in ev:
        if isinstance(e, TokenEvent):
            toks.setdefault(e.request_id, []).append(e.token)
        elif isinstance(e, FinishEvent):
            fins[e.request_id] = e
    for rid, (p, k, sid) in prompts.items():
        f = fins[rid]
        if sid is None and f.reason == FinishReason.MAX_TOKENS:
            assert toks.get(rid, []) == greedy(p, k), (seed, spec, rid)
    for sid in list(eng._sessions):
        eng.reset_session(sid)
    eng.step(ev.append)
    st = eng.kv.stats()
    assert st.used_pages == 0 and eng.scheduler.slots.available == 3 and runner.seq_state == {}, (seed, spec, st, runner.seq_state)
    return sum(1 for f in fins.values() if f.reason == FinishReason.ERROR)


@pytest.mark.parametrize("spec", [False, True])
@pytest.mark.parametrize("seed", [1, 2])
def test_v4_soak(seed, spec):
    _soak(seed, spec)
