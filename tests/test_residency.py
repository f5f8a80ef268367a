"""Expert residency coordinator, residency planning, prediction, telemetry (CPU)."""
import pytest

from ferrule_b200.runtime.expert_prediction import ExpertPredictor, ExpertTelemetry
from ferrule_b200.runtime.expert_residency import (ExpertResidencyController, ExpertResidencyCoordinator,
                                                   ResidencyError, plan_residency)


def install(c, e, required=True):
    t = c.prepare(e, required)
    c.activate(t)
    c.publish(t)
    return t


def test_two_phase_install_and_visibility():
    c = ExpertResidencyCoordinator(3, capacity=2, n_experts=8)
    assert c.resolve(5) is None and c.stats.misses == 1
    t = c.prepare(5)
    assert c.resolve(5) is None and c.in_flight(5)          # not visible before publish
    with pytest.raises(ResidencyError):
        c.prepare(5)
    with pytest.raises(ResidencyError):
        c.publish(t)                                          # must activate first
    c.activate(t)
    c.publish(t)
    assert c.resolve(5) == (t.slot, t.generation) and c.is_current(t.slot, t.generation)
    with pytest.raises(ResidencyError):
        c.prepare(5)


def test_lru_eviction_never_takes_leased_or_reserved_slots():
    c = ExpertResidencyCoordinator(0, capacity=3, n_experts=16)
    for e in (1, 2, 3):
        install(c, e)
    c.resolve(1)                                              # 2 is now least recently used
    s1, g1 = c.lease(2)                                       # ...but leased
    t = c.prepare(4)
    assert t.evicted == 3 and c.resident() == [1, 2]
    t5 = c.prepare(5)                                         # slot of 1 (only unleased READY one)
    assert t5.evicted == 1
    with pytest.raises(ResidencyError):
        c.prepare(6)                                          # 2 leased, two slots reserved
    c.release(s1, g1)
    t6 = c.prepare(6)
    assert t6.evicted == 2
    for tk in (t, t5, t6):
        c.activate(tk); c.publish(tk)
    assert c.resident() == [4, 5, 6] and c.stats.evictions == 3
    assert not c.is_current(s1, g1) and c.stats.stale_resolves == 1      # old generation is stale


def test_cancel_promote_and_evict():
    c = ExpertResidencyCoordinator(0, capacity=1, n_experts=4)
    t = c.prepare(2, required=False)
    assert c.promote(2) and not c.promote(2) and c.stats.promoted == 1
    c.cancel(t)
    assert not c.in_flight(2) and c.resolve(2) is None
    with pytest.raises(ResidencyError):
        c.activate(t)                                         # ticket is dead (generation bumped)
    install(c, 3)
    s, g = c.lease(3)
    assert not c.evict(3)
    c.release(s, g)
    assert c.evict(3) and c.resident() == []
    with pytest.raises(ResidencyError):
        c.release(s, g)


def test_plan_residency_and_controller():
    caps = plan_residency(device_budget_bytes=100 * 21, expert_bytes=21, moe_layers=list(range(3, 13)), n_experts=256,
                          min_per_layer=9, max_fraction=0.5)
    assert set(caps) == set(range(3, 13)) and all(v == 10 for v in caps.values())
    caps = plan_residency(10 ** 12, 21, [1, 2], 256, 9, max_fraction=0.5)
    assert caps == {1: 128, 2: 128}                           # capped at 50 % of the experts
    caps = plan_residency(10, 21, [1], 256, 9)
    assert caps == {1: 9}                                     # never below the working set
    ctl = ExpertResidencyController([1, 2], {1: 4, 2: 4}, 8)
    install(ctl.layer(1), 3)
    assert ctl.stats()[1].installs == 1 and ctl.stats()[2].installs == 0


def test_predictor_learns_frequency_and_transitions():
    p = ExpertPredictor(8)
    tel = ExpertTelemetry()
    for step in range(40):
        used = [0, 1] if step % 2 == 0 else [2, 3]           # strict alternation
        p.observe(0, used)
        tel.record(0, used)
    # after an odd step (2, 3 used) the next is (0, 1)
    assert set(p.predict(0, 2)) == {0, 1}
    p.observe(0, [0, 1])
    assert p.stats.hits == 2 and p.stats.precision == 1.0
    assert set(p.predict(0, 2, exclude=[2])) & {2} == set()
    assert tel.top(0, 2) == [0, 1] and abs(tel.coverage(0, [0, 1]) - 0.5) < 1e-9
