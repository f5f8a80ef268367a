"""Arena pool and sequence-state core (CPU)."""
import pytest

from ferrule_b200.runtime.arena import (ExecutionStateError, PersistentArenaPool, SequenceStateCore)


def test_pool_reuses_exact_key_and_counts():
    pool = PersistentArenaPool()
    built = []

    def build(tag):
        def f():
            built.append(tag)
            return {"tag": tag}
        return f
    with pool.acquire((32, 8), build("a")) as a:
        assert a["tag"] == "a"
        with pytest.raises(ExecutionStateError):
            pool.acquire((32, 8), build("x"))          # one lease at a time
    assert pool.stats.misses == 1 and pool.stats.installs == 1 and (32, 8) in pool
    lease = pool.acquire((32, 8), build("b"))
    assert lease.reused and lease.arena["tag"] == "a" and (32, 8) not in pool
    lease.__exit__(None, None, None)
    assert pool.stats.hits == 1 and built == ["a"]
    # another key never coalesces
    c1 = pool.checkout((64, 8), build("c"))
    c2 = pool.checkout((64, 8), build("d"))               # same key, first one still out: builds a second
    pool.checkin(c1)
    pool.checkin(c2)
    assert pool.idle((64, 8)) == 2 and pool.stats.installs == 3
    with pytest.raises(ExecutionStateError):
        pool.checkin(c2)
    # a failed build publishes nothing
    def boom():
        raise MemoryError("no memory")
    with pytest.raises(MemoryError):
        pool.checkout((128, 8), boom)
    assert (128, 8) not in pool and pool.stats.misses == 4 and pool.stats.installs == 3
    pool.clear()
    assert len(pool) == 0 and pool.stats.hits == 1


def test_sequence_state_core_binding_rules():
    s = SequenceStateCore()
    b = s.begin_step()
    s.commit_step(b, 5)
    assert s.position == 5
    with pytest.raises(ExecutionStateError):
        s.commit_step(b, 1)                                # stale: position moved on
    b2 = s.begin_step()
    s.poison_step(b2)
    with pytest.raises(ExecutionStateError):
        s.begin_step()
    s.reset()
    assert s.position == 0 and s.generation == 1 and not s.poisoned
    b3 = s.begin_step()
    s.commit_step(b3, 7)
    child = s.forked()
    assert child.position == 7 and child.generation == s.generation + 1
    snap = SequenceStateCore(3)
    s.restore_from(snap)
    assert s.position == 3 and s.generation == 2
    s.commit_step(s.begin_step(), 4)
    s.rewind(5)
    assert s.position == 5 and s.generation == 3
    with pytest.raises(ExecutionStateError):
        s.rewind(9)


def test_policy_set_and_engine_plan():
    from ferrule_b200.models import config as C
    from ferrule_b200.models.support import (AttentionKind, EnginePlan, ParallelismPlan, PolicySet, RouterKind,
                                             SpeculationMode)
    cfg = C.deepseek_v3()
    p = PolicySet.from_config(cfg, "fp8_mxfp4", ParallelismPlan(tensor_parallel=8, expert_parallel=8, sequence_parallel=8))
    assert p.attention.kind == AttentionKind.MLA and p.router.kind == RouterKind.SIGMOID_GROUP_TOPK
    assert p.quant.activation_blocks == (128, 32) and p.speculation.mode == SpeculationMode.MULTI_TOKEN_PREDICTION
    assert p.parallelism.gpus == 8 and p.semantics == "deepseek-v3"
    plan = EnginePlan.from_policies(p, cfg.n_heads, cfg.n_routed_experts, cfg.n_layers, cfg.vocab_size)
    assert plan.is_executable
    bad = PolicySet.from_config(cfg, "bf16", ParallelismPlan(tensor_parallel=8, context_parallel=2))
    plan = EnginePlan.from_policies(bad, cfg.n_heads, cfg.n_routed_experts, cfg.n_layers, cfg.vocab_size)
    assert not plan.is_executable and plan.missing[0].area == "parallelism"
    odd = PolicySet.from_config(cfg, "bf16", ParallelismPlan(tensor_parallel=3))
    assert not EnginePlan.from_policies(odd, cfg.n_heads, cfg.n_routed_experts, cfg.n_layers, cfg.vocab_size).is_executable
    lite = PolicySet.from_config(C.deepseek_v2_lite())
    assert lite.router.kind == RouterKind.SOFTMAX_TOPK and lite.semantics == "deepseek-v2"
