"""Randomised owner-loop soak (CPU, mock runner): requests with and without retained sessions, cancellations,
session resets, exact forks, scripted execute failures and delayed endings, a pool small enough to stall, with
and without speculation and auto-preemption.  After every step the page manager's invariants hold; at the end
every page and every slot is back."""
import random

import pytest

from ferrule_b200.runtime.engine import Engine, EngineConfig, FinishEvent
from ferrule_b200.runtime.io_protocol import MaterializationKey, ResourceId, ResourceKind
from ferrule_b200.runtime.provider import FakeMaterializationProvider
from ferrule_b200.runtime.registry import LoadRegistry
from ferrule_b200.runtime.runner import MockRunner
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import FinishReason, GenerateRequest


def _key(e: int) -> MaterializationKey:
    return MaterializationKey("m", b"s", bytes([e]), ResourceId(ResourceKind.ROUTED_EXPERT, 1, e), 1, "cuda", 0, 0, 0)


def _soak(seed: int, spec: bool) -> Engine:
    rnd = random.Random(seed)
    runner = MockRunner(page_size=16, draft_len=2 if spec else 0,
                        draft_accuracy=(lambda slot, j, nxt: nxt if rnd.random() < 0.6 else (nxt + 1) % 1000) if spec else None)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=48, prefill_chunk_size=16,
                            ctx_size=200)
    # half of the runs park transactions on materializations (scripted provider: failures, lost completions)
    prov = FakeMaterializationProvider(auto=True) if rnd.random() < 0.5 else None
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=24, page_size=16, speculative=spec, max_draft=2,
                                      auto_preempt=rnd.random() < 0.5,
                                      prefix_cache_tokens=rnd.choice([0, 64, 256]), prefix_block=16,
                                      materialization_timeout_s=0.01),
                 registry=LoadRegistry(prov) if prov is not None else None,
                 detokenize=lambda ids: "".join(str(t % 10) for t in ids))
    shared = [rnd.randrange(1, 900) for _ in range(40)]           # prompts often start with a common prefix
    live, n, ev, reasons = set(), 0, [], {}
    for _ in range(500):
        a = rnd.random()
        if a < 0.25 and len(live) < 10:
            rid, n = f"r{n}", n + 1
            sid = rnd.choice([None, None, "s1", "s2", "s3"])
            try:
                head = shared[:rnd.choice([0, 0, 16, 32, 40])]
                eng.submit(GenerateRequest(rid, head + [rnd.randrange(1, 900) for _ in range(rnd.randrange(1, 40))],
                                           max_new_tokens=rnd.randrange(0, 12), session_id=sid,
                                           stop=["7", "13"] if rnd.random() < 0.2 else [],
                                           retain_session=bool(sid) and rnd.random() < 0.7, ignore_eos=True))
                live.add(rid)
            except ValueError:
                pass                                   # busy session, or a continuation past the context window
        elif a < 0.31 and live:
            eng.cancel_request(rnd.choice(sorted(live)))
        elif a < 0.34:
            eng.reset_session(rnd.choice(["s1", "s2", "s3"]))
        elif a < 0.38 and eng._sessions and len(live) < 10:
            rid, n = f"f{n}", n + 1
            try:
                eng.fork_session_exact(rnd.choice(sorted(eng._sessions)),
                                       GenerateRequest(rid, [rnd.randrange(1, 900)], max_new_tokens=rnd.randrange(1, 5),
                                                       ignore_eos=True))
                live.add(rid)
            except (ValueError, RuntimeError, KeyError):
                pass
        elif a < 0.39:
            runner.fail_next_execute = 1
        elif a < 0.40:
            runner.fail_next_end = rnd.randrange(1, 3)
        elif a < 0.44:
            runner.pending_ends = rnd.randrange(0, 3)
        elif a < 0.46 and live:
            # manual swap-out / swap-in of a running request
            rid = rnd.choice(sorted(live))
            try:
                if rid in eng.scheduler.suspended:
                    eng.restore_session(rid)
                else:
                    eng.preempt_session(rid)
            except Exception:  # noqa: BLE001 - not preemptible right now (inside a transaction, nothing cached, no pages)
                pass
        elif a < 0.47:
            runner.no_candidate_rows = {rnd.randrange(0, 8)} if rnd.random() < 0.5 else set()
        elif a < 0.52 and prov is not None:
            runner.wait_next.append([_key(e) for e in rnd.sample(range(20), rnd.randrange(1, 3))])
            if rnd.random() < 0.25:
                # "stale" and "lose" leave the load without its completion: the parked transaction times out
                prov.script_next(rnd.choice(["fail", "short", "dup", "fail", "short", "dup", "stale", "lose"]))
        eng.step(ev.append)
        for e in ev:
            if isinstance(e, FinishEvent):
                live.discard(e.request_id)
                reasons[e.request_id] = e.reason
        ev.clear()
        eng.kv.check_invariants()
    runner.pending_ends = runner.fail_next_end = 0
    runner.no_candidate_rows = set()
    runner.wait_next.clear()
    for rid in list(eng.scheduler.suspended):
        try:
            eng.restore_session(rid)
        except Exception:  # noqa: BLE001 - no room yet: cancel it instead
            eng.cancel_request(rid)
    assert eng.run_until_idle(ev.append, max_steps=5000) < 5000, "the engine did not drain"
    for e in ev:
        if isinstance(e, FinishEvent):
            live.discard(e.request_id)
            reasons[e.request_id] = e.reason
    assert not live, f"requests without a finish event: {sorted(live)}"
    for sid in list(eng._sessions):
        eng.reset_session(sid)
    while eng._prefix_evict():
        pass
    eng.step(ev.append)
    eng.kv.check_invariants()
    st = eng.kv.stats()
    assert st.used_pages == 0 and st.quarantined_pages == 0, (seed, spec, st)
    assert eng.scheduler.slots.available == 4 and not eng._session_busy
    if prov is not None:
        assert eng.registry.residual().get("continuations", 0) == 0 and not eng._waiting
        assert not any(op.waiters or op.leases for op in eng.registry.ops.values())
    assert set(reasons.values()) <= {FinishReason.MAX_TOKENS, FinishReason.CANCELLED, FinishReason.ERROR,
                                     FinishReason.CONTEXT, FinishReason.STOP_STRING, FinishReason.NO_CANDIDATE}
    return eng


@pytest.mark.parametrize("spec", [False, True])
@pytest.mark.parametrize("seed", range(6))
def test_soak(seed, spec):
    eng = _soak(seed, spec)
    assert eng.stats.finished > 10
