"""Expert placement: balanced renumbering of a layer's experts over ranks, applied to the weights."""
import pytest
import torch

from ferrule_b200.models import config as C
from ferrule_b200.models import deepseek as D
from ferrule_b200.models import weights as W
from ferrule_b200.parallel import placement as P


def test_balanced_order_is_an_even_deterministic_permutation():
    load = [100, 90, 80, 70, 1, 1, 1, 1, 5, 5, 5, 5, 0, 0, 0, 0]
    order = P.balanced_order(load, 4)
    assert sorted(order) == list(range(16))
    assert P.balanced_order(load, 4) == order
    by_id = P.rank_loads(load, list(range(16)), 4)
    by_plan = P.rank_loads(load, order, 4)
    assert by_id == [340.0, 4.0, 20.0, 0.0] and sorted(by_plan) == [85.0, 87.0, 92.0, 100.0]   # one hot expert per rank
    assert P.imbalance(load, order, 4) < 1.2 < P.imbalance(load, list(range(16)), 4)
    for r in range(4):
        chunk = order[r * 4:(r + 1) * 4]
        assert chunk == sorted(chunk), "original id order inside a rank"
    assert P.inverse_order(order)[order[5]] == 5
    with pytest.raises(ValueError):
        P.balanced_order(load[:15], 4)
    # an even load keeps every expert where it was
    assert P.plan_expert_placement([[3] * 8], 4) == {}
    assert P.plan_expert_placement([[], [0] * 8], 4) == {}


def test_group_limited_routers_move_whole_groups():
    # 4 groups of 4: groups 0 and 1 are hot; two ranks must get one hot group each
    load = [9, 9, 9, 9, 8, 8, 8, 8, 1, 1, 1, 1, 0, 0, 0, 0]
    order = P.balanced_order(load, 2, n_groups=4)
    groups = [order[i:i + 4] for i in range(0, 16, 4)]
    assert all(g == list(range(g[0], g[0] + 4)) and g[0] % 4 == 0 for g in groups), "groups stay contiguous"
    loads = P.rank_loads(load, order, 2)
    assert sorted(loads) == [36.0, 36.0]
    with pytest.raises(ValueError):
        P.balanced_order(load, 8, n_groups=4)


def _logits(w, ids):
    cfg = w.cfg
    pool = D.KvPool(cfg, 8, 16, "cpu")
    fwd = D.ReferenceForward(w, pool)
    T = len(ids)
    mk = lambda v, dt: torch.tensor(v, dtype=dt)
    bt = torch.zeros(1, 4, dtype=torch.int32)
    bt[0, :2] = torch.tensor([1, 2])
    b = D.DeviceBatch(mk(ids, torch.int32), mk(list(range(T)), torch.int32), mk([16 + i for i in range(T)], torch.int64),
                      mk([0] * T, torch.int32), mk(list(range(T)), torch.int32), bt, mk([T - 1], torch.int32), T, 1)
    return fwd, fwd.forward(b)[0]


def test_renumbered_experts_compute_the_same_function_and_land_on_the_planned_ranks():
    cfg = C.tiny_fixture()
    E = cfg.n_routed_experts
    moe_layers = [i for i in range(cfg.n_layers) if i >= cfg.n_dense_layers]
    g = torch.Generator().manual_seed(0)
    plan = {i: torch.randperm(E, generator=g).tolist() for i in moe_layers}
    ids = torch.randint(0, cfg.vocab_size, (24,), generator=g).tolist()
    base = W.random_weights(cfg, dtype=torch.float32, seed=3, router_zipf=1.1)
    moved = W.random_weights(cfg, dtype=torch.float32, seed=3, router_zipf=1.1, expert_orders=plan)
    _, want = _logits(base, ids)
    _, got = _logits(moved, ids)
    assert torch.allclose(got, want, atol=1e-4 * float(want.abs().max()))
    li = moe_layers[0]
    assert not torch.equal(moved.layers[li].e_w13, base.layers[li].e_w13)
    for j in range(E):
        assert torch.equal(moved.layers[li].e_w13[j], base.layers[li].e_w13[plan[li][j]])
        assert torch.equal(moved.layers[li].router_w[j], base.layers[li].router_w[plan[li][j]])
    # the in-place form on an unsharded model gives the same weights
    again = W.random_weights(cfg, dtype=torch.float32, seed=3, router_zipf=1.1)
    P.permute_experts_(again, plan)
    assert torch.equal(again.layers[li].e_w2, moved.layers[li].e_w2)
    assert torch.equal(again.layers[li].router_bias, moved.layers[li].router_bias)
    # a rank of a sharded layout draws exactly its planned experts
    world = 2
    for r in range(world):
        shard = W.random_weights(cfg, dtype=torch.float32, seed=3, router_zipf=1.1, tp_rank=r, tp_world=world,
                                 expert_orders=plan)
        lo, hi = shard.e_lo, shard.e_hi
        assert torch.equal(shard.layers[li].e_w13, moved.layers[li].e_w13[lo:hi])
        assert torch.equal(shard.layers[li].router_w, moved.layers[li].router_w)
    with pytest.raises(ValueError):
        P.permute_experts_(shard, plan)
    with pytest.raises(ValueError):
        W.random_weights(cfg, dtype=torch.float32, seed=3, expert_orders={li: [0] * E})


def test_calibrated_plan_evens_out_a_skewed_router():
    """Zipf(1.1) popularity: count routes over a calibration batch, plan for 4 ranks, and measure again on the
    renumbered model - the busiest rank carries what the plan said it would."""
    cfg = C.tiny_fixture()
    E, world = cfg.n_routed_experts, 4
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist()
    base = W.random_weights(cfg, dtype=torch.float32, seed=5, router_zipf=1.1)
    counter = P.RouteCounter(cfg.n_layers, E)
    fwd, _ = _logits(base, ids[:1])
    counter.attach(fwd)
    _, _ = _logits_with(fwd, base, ids)
    P.RouteCounter.detach(fwd)
    counts = counter.telemetry.counts
    moe_layers = [i for i in range(cfg.n_layers) if sum(counts[i])]
    assert moe_layers and all(sum(counts[i]) == 30 * cfg.topk for i in moe_layers)
    plan = counter.plan(world, min_gain=0.0)
    assert plan, "a skewed router leaves something to balance"
    for i, order in plan.items():
        assert P.imbalance(counts[i], order, world) <= P.imbalance(counts[i], list(range(E)), world)
    moved = W.random_weights(cfg, dtype=torch.float32, seed=5, router_zipf=1.1, expert_orders=plan)
    c2 = P.RouteCounter(cfg.n_layers, E)
    fwd2, _ = _logits(moved, ids[:1])
    c2.attach(fwd2)
    _logits_with(fwd2, moved, ids)
    i = next(iter(plan))
    ident = list(range(E))
    # routes measured on the renumbered model, summed per rank == the plan's prediction from the first count
    assert P.rank_loads(c2.telemetry.counts[i], ident, world) == P.rank_loads(counts[i], plan[i], world)


def _logits_with(fwd, w, ids):
    T = len(ids)
    mk = lambda v, dt: torch.tensor(v, dtype=dt)
    bt = torch.zeros(1, 4, dtype=torch.int32)
    bt[0, :2] = torch.tensor([1, 2])
    b = D.DeviceBatch(mk(ids, torch.int32), mk(list(range(T)), torch.int32), mk([16 + i for i in range(T)], torch.int64),
                      mk([0] * T, torch.int32), mk(list(range(T)), torch.int32), bt, mk([T - 1], torch.int32), T, 1)
    return fwd, fwd.forward(b)[0]


def test_cli_plans_a_placement_and_applies_it(tmp_path):
    import contextlib, io, json
    from ferrule_b200.cli.main import main as cli_main
    common = ["--preset", "tiny-fixture", "--device", "cpu", "--router-zipf", "1.1", "--ctx-size", "64", "--page-size", "16"]
    out = tmp_path / "plan.json"
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        assert cli_main(["plan-placement", *common, "--ranks", "4", "--requests", "4", "--prompt-tokens", "24",
                         "--max-tokens", "4", "--max-seqs", "4", "--out", str(out)]) == 0
    rep = json.loads(buf.getvalue().strip().splitlines()[-1])
    assert rep["routes"] > 0 and rep["written"] == str(out)
    for layer in rep["layers"].values():
        assert layer["imbalance_planned"] <= layer["imbalance_by_id"]
    plan = json.loads(out.read_text())["plan"]
    assert plan and all(sorted(o) == list(range(8)) for o in plan.values())
    toks = []
    for extra in ([], ["--expert-plan", str(out)]):
        buf = io.StringIO()
        with contextlib.redirect_stdout(buf):
            assert cli_main(["generate", *common, "--tokens", "5,9,11", "--max-tokens", "6", "--ignore-eos", "--max-seqs", "2",
                             *extra]) == 0
        toks.append(json.loads(buf.getvalue().strip().splitlines()[-1])["tokens"])
    assert toks[0] == toks[1] and len(toks[0]) == 6


@pytest.mark.gpu
def test_route_counter_reads_the_kernel_paths_routes():
    """Every MoE layer reports rows x top-k routes, the observed forward returns what the unobserved one does, and
    a model renumbered by the resulting plan computes the same logits."""
    cfg = C.smoke_gpu()
    dev = "cuda"
    w = W.random_weights(cfg, device=dev, seed=1, std=0.05, router_zipf=1.1)
    g = torch.Generator().manual_seed(0)
    T = 40
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=g).tolist()
    mk = lambda v, dt: torch.tensor(v, dtype=dt, device=dev)
    bt = torch.zeros(1, 8, dtype=torch.int32)
    bt[0, :3] = torch.tensor([1, 2, 3])

    def run(weights, observer=None):
        pool = D.KvPool(cfg, 16, 16, dev)
        fwd = D.CudaForward(weights, pool, max_rows=64, max_logit_rows=4, decode_rows=8, max_seq_len=128, attn_splits=2)
        if observer is not None:
            observer.attach(fwd)
        b = D.DeviceBatch(mk(ids, torch.int32), mk(list(range(T)), torch.int32), mk([16 + i for i in range(T)], torch.int64),
                          mk([0] * T, torch.int32), mk(list(range(T)), torch.int32), bt.to(dev), mk([T - 1], torch.int32), T, 1)
        nid, _, logits = fwd.forward(b, want_logits=True)
        torch.cuda.synchronize()
        return int(nid[0]), logits.float().cpu()

    counter = P.RouteCounter(cfg.n_layers, cfg.n_routed_experts)
    tok_obs, logits_obs = run(w, counter)
    tok, logits = run(w)
    assert tok_obs == tok and torch.equal(logits_obs, logits)
    counts = counter.telemetry.counts
    moe = [i for i in range(cfg.n_layers) if sum(counts[i])]
    assert moe and all(sum(counts[i]) == T * cfg.topk for i in moe)
    plan = counter.plan(4, min_gain=0.0)
    moved = W.random_weights(cfg, device=dev, seed=1, std=0.05, router_zipf=1.1, expert_orders=plan)
    _, logits_moved = run(moved)
    assert float((logits_moved - logits).abs().max()) <= 0.05 * float(logits.abs().max()) + 1e-3
