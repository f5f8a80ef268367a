"""DeepSeek-V4 behind the engine: the V4 runner must emit the oracle's greedy stream through the scheduler's
chunked prefill, batching and transaction protocol."""
import pytest
import torch

from ferrule_b200.models.v4_model import V4Reference, V4SeqCache, random_v4_weights, tiny_v4
from ferrule_b200.models.v4_runner import V4Runner
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest


def _greedy(w, prompt, n_new):
    ref = V4Reference(w)
    c = V4SeqCache(w.cfg)
    for t in prompt:
        logits = ref.step(c, t)
    out = []
    for _ in range(n_new):
        t = int(torch.argmax(logits))
        out.append(t)
        logits = ref.step(c, t)
    return out


def _engine(w, device):
    runner = V4Runner(w, n_pages=32, page_size=16, max_seqs=4, max_seq_len=128, max_rows=64)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=12,
                            ctx_size=128)
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=32, page_size=16)), runner


def _run(eng, prompts, n_new):
    for i, p in enumerate(prompts):
        eng.submit(GenerateRequest(f"r{i}", p, max_new_tokens=n_new, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=5000)
    return [[e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == f"r{i}"] for i in range(len(prompts))]


def test_v4_runner_serves_oracle_greedy_stream_on_cpu():
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cpu", seed=3)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 20, 14)]
    eng, runner = _engine(w, "cpu")
    got = _run(eng, prompts, 6)
    for p, toks in zip(prompts, got):
        assert toks == _greedy(w, p, 6)
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0
    assert runner.kv_schema().planes[0].name == "window_kv" and runner.steps > 0


def test_v4_runner_reexecutes_positions_after_abort_on_cpu():
    """An aborted transaction leaves rows past the committed length; the next batch overwrites them."""
    from ferrule_b200.runtime.execution import (ExecutionBatch, Intent, LogitsRequest, Phase, SequenceSlice)
    from ferrule_b200.runtime.runner import EndIntent
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cpu", seed=4)
    runner = V4Runner(w, n_pages=8, page_size=16, max_seqs=2, max_seq_len=64, max_rows=32)
    prompt = list(range(3, 13))

    def batch(tokens, ctx):
        n = len(tokens)
        return ExecutionBatch(tokens, list(range(ctx, ctx + n)), list(range(ctx, ctx + n)),
                              [LogitsRequest.none()] * (n - 1) + [LogitsRequest(kind=_topk_kind(), k=1)],
                              [SequenceSlice(0, Phase.PREFILL, 0, n, ctx, ctx + n, 0, 4)], [0, 1, 2, 3],
                              Intent.COMMITTED, 16)

    def run(tokens, ctx, intent):
        runner.prepare_batch(1, batch(tokens, ctx))
        out = runner.execute(1).output
        runner.end_transaction(1, intent)
        return out.rows[-1].token_ids[0]

    run(prompt[:6], 0, EndIntent.PUBLISH)
    run([99, 98, 97], 6, EndIntent.ABORT)                   # rows 6..8 written, then dropped
    got = run(prompt[6:], 6, EndIntent.PUBLISH)
    assert got == _greedy(w, prompt, 1)[0]


def _topk_kind():
    from ferrule_b200.runtime.execution import LogitsKind
    return [k for k in LogitsKind if k != LogitsKind.NONE][0]


@pytest.mark.gpu
def test_v4_runner_serves_on_the_kernels():
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cuda", seed=3)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 20, 14)]
    eng, runner = _engine(w, "cuda")
    got = _run(eng, prompts, 6)
    assert all(len(t) == 6 for t in got) and runner.steps > 0
    # the batched engine path equals the kernels' own one-sequence-at-a-time stream
    from ferrule_b200.models.v4_model import V4Cuda
    solo = V4Cuda(w, 1, 128)
    for p, toks in zip(prompts, got):
        solo.positions[0] = 0
        for t in p:
            nxt, _ = solo.step([0], [t])
        want = []
        for _ in range(6):
            t = int(nxt[0])
            want.append(t)
            nxt, _ = solo.step([0], [t])
        assert toks == want
    from ferrule_b200.ops import _lib
    assert _lib.read_status()[0] == 0


def test_v4_sequences_swap_out_and_return_under_page_pressure_on_cpu():
    """The pool admits the three prompts but not their growth: with `auto_preempt` the engine swaps a V4 sequence
    out (its slot tables stay in place, its pages go back) and brings it back later; the streams stay the
    oracle's.  Page sharing stays off for the slot-bound runner (no prefix-cache hit, no fork)."""
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cpu", seed=3)
    g = torch.Generator().manual_seed(2)
    base = torch.randint(0, cfg.vocab_size, (15,), generator=g).tolist()
    prompts = [base, base[:14] + [7], torch.randint(0, cfg.vocab_size, (15,), generator=g).tolist()]
    runner = V4Runner(w, n_pages=6, page_size=16, max_seqs=4, max_seq_len=128, max_rows=64)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=12,
                            ctx_size=128)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=6, page_size=16, auto_preempt=True,
                                      prefix_cache_tokens=256, prefix_block=16))
    got = _run(eng, prompts, 24)
    for p, toks in zip(prompts, got):
        assert toks == _greedy(w, p, 24)
    assert eng.stats.auto_preemptions >= 1 and eng.kv.stats().preemptions == eng.stats.auto_preemptions
    assert eng.stats.prefix_hits == 0 and eng.stats.prefix_entries == 0 and eng.kv.stats().forks == 0
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and not eng.scheduler.suspended
    assert runner.seq_state == {}, "finished sequences gave their slots (and the slot's cursor) back"


def test_v4_session_is_retained_in_its_slot_across_turns_on_cpu():
    """The V4 state of a sequence lives in its slot: a retained session keeps the slot out of the pool between
    requests, the continuation returns to it and feeds only the new tokens, and dropping the session gives the
    slot back."""
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cpu", seed=3)
    eng, runner = _engine(w, "cpu")
    g = torch.Generator().manual_seed(7)
    p1 = torch.randint(0, cfg.vocab_size, (9,), generator=g).tolist()
    p2 = torch.randint(0, cfg.vocab_size, (5,), generator=g).tolist()
    eng.submit(GenerateRequest("t1", p1, max_new_tokens=4, ignore_eos=True, session_id="s", retain_session=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=2000)
    first = [e.token for e in ev if isinstance(e, TokenEvent)]
    assert eng.scheduler.slots.available == 3, "the session holds its slot"
    steps_before = runner.steps
    eng.submit(GenerateRequest("t2", p2, max_new_tokens=4, ignore_eos=True, session_id="s", retain_session=True))
    ev2 = []
    eng.run_until_idle(ev2.append, max_steps=2000)
    second = [e.token for e in ev2 if isinstance(e, TokenEvent)]
    # the oracle over the whole conversation: first prompt, its reply, second prompt
    assert eng._sessions["s"].position == len(p1) + 4 + len(p2) + 4
    assert second == _greedy(w, p1 + first + p2, 4)
    assert runner.steps - steps_before <= len(p2) + 1 + 4, "only the new tokens ran"
    # another request gets a different slot while the session is held
    eng.submit(GenerateRequest("other", p2, max_new_tokens=2, ignore_eos=True))
    eng.run_until_idle(lambda e: None, max_steps=2000)
    assert eng.scheduler.slots.available == 3
    assert eng.reset_session("s") and eng.scheduler.slots.available == 4
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and runner.seq_state == {}


def test_idle_retained_sessions_give_their_slots_to_waiting_requests_on_cpu():
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cpu", seed=3)
    eng, runner = _engine(w, "cpu")                   # four slots
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, cfg.vocab_size, (6,), generator=g).tolist() for _ in range(6)]
    for i in range(4):
        eng.submit(GenerateRequest(f"s{i}", prompts[i], max_new_tokens=2, ignore_eos=True, session_id=f"sess{i}",
                                   retain_session=True))
    eng.run_until_idle(lambda e: None, max_steps=2000)
    assert eng.scheduler.slots.available == 0 and len(eng._sessions) == 4
    # two fresh requests: the two sessions retained longest are dropped for them, the others keep their state
    for i in (4, 5):
        eng.submit(GenerateRequest(f"n{i}", prompts[i], max_new_tokens=3, ignore_eos=True))
    ev = []
    steps = eng.run_until_idle(ev.append, max_steps=2000)
    assert steps < 2000
    for i in (4, 5):
        assert [e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == f"n{i}"] == _greedy(w, prompts[i], 3)
    assert eng.stats.session_evictions == 2 and sorted(eng._sessions) == ["sess2", "sess3"]
    # a kept session still continues from its cached state
    eng.submit(GenerateRequest("c", [7, 8], max_new_tokens=2, ignore_eos=True, session_id="sess3", retain_session=True))
    ev2 = []
    eng.run_until_idle(ev2.append, max_steps=2000)
    kept = eng._sessions["sess3"]
    assert [e.token for e in ev2 if isinstance(e, TokenEvent)] == _greedy(w, kept.tokens[:6 + 2 + 2], 2)
    for sid in list(eng._sessions):
        eng.reset_session(sid)
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0 and eng.scheduler.slots.available == 4


def test_v4_sessions_cannot_be_forked_by_sharing_pages():
    cfg = tiny_v4()
    w = random_v4_weights(cfg, device="cpu", seed=3)
    eng, runner = _engine(w, "cpu")
    eng.submit(GenerateRequest("t1", [5, 6, 7, 8], max_new_tokens=2, ignore_eos=True, session_id="s", retain_session=True))
    eng.run_until_idle(lambda e: None, max_steps=500)
    with pytest.raises(ValueError):
        eng.fork_session_exact("s", GenerateRequest("f", [9], max_new_tokens=1))
    assert eng.kv.stats().forks == 0
    assert eng.reset_session("s") and eng.kv.stats().used_pages == 0
