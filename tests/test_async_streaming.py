"""Asynchronous expert streaming on the real model: a batch that routes to a non-resident expert parks as a
continuation, the load registry drives the arena provider, the transaction resumes at the layer it stopped at
and the token stream equals the fully resident model's."""
import pytest
import torch

from ferrule_b200.models import config as C
from ferrule_b200.models import weights as W
from ferrule_b200.models.runner import DeepSeekRunner
from ferrule_b200.runtime.engine import Engine, EngineConfig, TokenEvent
from ferrule_b200.runtime.scheduler import SchedulerConfig
from ferrule_b200.runtime.session import GenerateRequest


def _engine(w, device, residency=None, async_streaming=False):
    runner = DeepSeekRunner(w, n_pages=48, page_size=16, max_rows=64, max_seqs=4, max_seq_len=256, device=device,
                            enable_mtp=False, expert_residency=residency, async_streaming=async_streaming)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=8,
                            ctx_size=256)
    reg = runner.make_registry() if async_streaming else None
    return Engine(runner, EngineConfig(scheduler=sched, kv_pages=48, page_size=16), registry=reg), runner


def _run(eng, prompts, n_new):
    for i, p in enumerate(prompts):
        eng.submit(GenerateRequest(f"r{i}", p, max_new_tokens=n_new, ignore_eos=True))
    ev = []
    eng.run_until_idle(ev.append, max_steps=20000)
    return [[e.token for e in ev if isinstance(e, TokenEvent) and e.request_id == f"r{i}"] for i in range(len(prompts))]


def _check(device, residency=0.75):
    cfg = C.tiny_fixture()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 11)]
    dt = torch.bfloat16 if device == "cuda" else torch.float32
    want = _run(_engine(W.random_weights(cfg, device=device, dtype=dt, seed=2), device)[0], prompts, 8)
    eng, runner = _engine(W.random_weights(cfg, device=device, dtype=dt, seed=2), device, residency=residency,
                          async_streaming=True)
    got = _run(eng, prompts, 8)
    assert got == want
    assert eng.stats.waits > 0 and eng.stats.resumes > 0 and runner.stats.waits == eng.stats.waits
    a = runner.arena.stats
    assert a.uploads > 0 and a.evictions > 0, "fewer frames than experts: experts were evicted and reloaded"
    for la in runner.arena.layers.values():
        assert all(s.leases == 0 for s in la.coord.slots), "every lease was returned when its transaction ended"
    eng.kv.check_invariants()
    assert eng.kv.stats().used_pages == 0
    assert eng.registry.residual().get("continuations", 0) == 0
    obs = runner.observability()
    assert obs["expert_arena"]["uploads"] == a.uploads and "expert_telemetry" in obs
    assert "expert_predictor" not in obs, "nobody asked for prefetch candidates: no predictor, no observations"


def test_async_streaming_parks_and_resumes_on_cpu():
    _check("cpu")


def test_async_streaming_takes_layers_with_more_experts_than_frames_in_waves_on_cpu():
    """Two frames for eight experts: nearly every batch routes to more experts than frames.  The layer runs them
    in waves of two, parks whenever a wave misses an expert and resumes with the finished waves remembered -
    nothing streams inline, and the tokens are those of the resident model."""
    _check("cpu", residency=0.25)


@pytest.mark.gpu
@pytest.mark.parametrize("residency", [0.75, 0.25])
def test_async_streaming_parks_and_resumes_on_gpu(residency):
    _check("cuda", residency)
    from ferrule_b200.ops import _lib
    assert _lib.read_status()[0] == 0


def test_speculative_decoding_with_streamed_experts_drafts_on_resident_proposal_experts_on_cpu():
    """The proposal stage's experts stay on the device (drafting runs between transactions, where nothing can park
    for an upload): with asynchronous streaming and speculative decoding together no `ensure` call - the inline
    upload path - ever runs, and the stream is the resident, non-speculative model's."""
    cfg = C.tiny_fixture().with_(n_mtp_layers=1)
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 11)]
    want = _run(_engine(W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2), "cpu")[0], prompts, 8)
    w = W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2)
    runner = DeepSeekRunner(w, n_pages=48, page_size=16, max_rows=64, max_seqs=4, max_seq_len=256, device="cpu",
                            enable_mtp=True, expert_residency=0.5, async_streaming=True)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=8,
                            ctx_size=256)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=48, page_size=16, speculative=True, max_draft=1,
                                      confidence_threshold=0.0), registry=runner.make_registry())
    got = _run(eng, prompts, 8)
    assert got == want
    assert all(layer < cfg.n_layers for layer in runner.arena.layers), "the proposal stage is not in the arena"
    assert runner.stats.mtp_proposals > 0 and eng.spec.metrics.drafted > 0
    assert runner.arena.stats.ensure_calls == 0, "nothing was uploaded inline"
    assert eng.stats.waits > 0 and runner.arena.stats.uploads > 0
    for la in runner.arena.layers.values():
        assert all(s.leases == 0 for s in la.coord.slots)
    # a proposal stage inside the arena (the old arrangement) still works: its experts stream inline while drafting
    from ferrule_b200.models.expert_arena import ExpertArena
    w2 = W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2)
    assert cfg.n_layers in ExpertArena(w2, 0.5, replace_weights=False, mtp_resident=False).layers


def test_parked_transactions_prefetch_the_hot_experts_of_later_layers_on_cpu():
    """`transaction_prefetch`: while a transaction waits for the experts it must have, the engine requests - without
    a waiter - the most-routed non-resident experts of the layers that follow.  The requests are owned by the
    transaction, nothing of them is left when it ends, and the stream stays the resident model's."""
    cfg = C.tiny_fixture().with_(n_layers=4)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 11, 9)]
    want = _run(_engine(W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2), "cpu")[0], prompts, 10)
    w = W.random_weights(cfg, device="cpu", dtype=torch.float32, seed=2)
    runner = DeepSeekRunner(w, n_pages=48, page_size=16, max_rows=64, max_seqs=4, max_seq_len=256, device="cpu",
                            enable_mtp=False, expert_residency=0.5, async_streaming=True)
    sched = SchedulerConfig(max_active_sequences=4, max_decode_batch=4, max_batch_tokens=32, prefill_chunk_size=8,
                            ctx_size=256)
    eng = Engine(runner, EngineConfig(scheduler=sched, kv_pages=48, page_size=16, transaction_prefetch=3),
                 registry=runner.make_registry())
    got = _run(eng, prompts, 10)
    assert got == want
    assert eng.stats.waits > 0 and eng.stats.prefetch_requests > 0
    reg = eng.registry
    from ferrule_b200.runtime.registry import OwnerKind
    leftover = [op for op in reg.ops.values() if any(k == OwnerKind.TRANSACTION_PREFETCH for k, _ in op.owners)]
    assert not leftover, "every prefetch owner was detached when its transaction ended"
    assert reg.residual().get("continuations", 0) == 0
    for la in runner.arena.layers.values():
        assert all(s.leases == 0 for s in la.coord.slots)
    assert sum(runner.telemetry.tokens) > 0
    assert runner.predictor is not None and runner.observability()["expert_predictor"]["predictions"] > 0
    # candidates: only layers after the stop layer, only non-resident experts, at most n
    keys = runner.prefetch_candidates(1, 4)
    assert len(keys) <= 4 and all(k.resource.group > 1 for k in keys)
    assert all(runner.arena.layers[k.resource.group].coord.resolve(k.resource.item) is None for k in keys)
    assert runner.prefetch_candidates(max(runner.arena.layers), 4) == []
