"""Expert placement for tensor / expert parallel ranks: which experts sit on which rank.

Experts are owned in contiguous id ranges (rank r holds ids [r * E / world, (r + 1) * E / world)), so a layer's
step lasts as long as its busiest rank: the reductions that follow wait for it.  With a skewed router (a few hot
experts) sharding by id piles hot experts onto the same rank.  Placement keeps the contiguous-range kernels and
instead renumbers the experts of a layer: physical id j holds original expert `order[j]`.  The renumbering is
applied to the weights once - router rows, router bias, expert tensors, the values of a hash-routing table - so
the model computes the same function and no kernel sees a remap table.

`plan_expert_placement` balances measured per-expert load (route counts from `ExpertTelemetry`) over the ranks
with the longest-processing-time rule under the equal-count constraint; with group-limited routing (experts in
`n_groups` contiguous groups, a token may only use `topk_groups` of them) whole groups are the unit that moves,
because the router's group scores are taken over contiguous id ranges.

The reference plans placement in its inert parallelism policy only
(crates/ferrule-model/src/support/policies.rs:56-77); its per-expert popularity source is
crates/ferrule-model/src/moe/telemetry.rs:9-60.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch


def rank_loads(load: Sequence[float], order: Sequence[int], world: int) -> List[float]:
    """Load per rank when physical id j holds original expert order[j]."""
    E = len(order)
    per = E // world
    return [float(sum(load[order[j]] for j in range(r * per, (r + 1) * per))) for r in range(world)]


def imbalance(load: Sequence[float], order: Sequence[int], world: int) -> float:
    """Busiest rank over the mean rank (1.0 = perfectly even)."""
    loads = rank_loads(load, order, world)
    mean = sum(loads) / world
    return max(loads) / mean if mean > 0 else 1.0


def balanced_order(load: Sequence[float], world: int, n_groups: int = 1) -> List[int]:
    """Physical order of one layer's experts: longest-processing-time assignment of experts (or, for group-limited
    routers, of whole groups) to ranks, every rank receiving the same number.  Within a rank the original id
    order is kept, experts of equal load keep their relative order (the plan is deterministic)."""
    E = len(load)
    if E % world:
        raise ValueError(f"{E} experts do not divide over {world} ranks")
    if n_groups > 1:
        if E % n_groups or n_groups % world:
            raise ValueError(f"{n_groups} groups of {E} experts do not divide over {world} ranks")
        gs = E // n_groups
        gload = [sum(load[g * gs:(g + 1) * gs]) for g in range(n_groups)]
        gorder = balanced_order(gload, world)
        return [g * gs + i for g in gorder for i in range(gs)]
    per = E // world
    bins: List[List[int]] = [[] for _ in range(world)]
    totals = [0.0] * world
    for e in sorted(range(E), key=lambda i: (-float(load[i]), i)):
        open_ranks = [r for r in range(world) if len(bins[r]) < per]
        r = min(open_ranks, key=lambda i: (totals[i], i))
        bins[r].append(e)
        totals[r] += float(load[e])
    return [e for b in bins for e in sorted(b)]


def plan_expert_placement(counts: Sequence[Sequence[float]], world: int, n_groups: int = 1,
                          min_gain: float = 0.02) -> Dict[int, List[int]]:
    """counts[layer][expert] (zero rows = layer without routed experts) -> {layer: order} for the layers whose
    busiest rank gets at least `min_gain` (relative) lighter; layers that are already even keep their ids."""
    plan: Dict[int, List[int]] = {}
    for layer, row in enumerate(counts):
        if not row or sum(row) <= 0:
            continue
        ident = list(range(len(row)))
        order = balanced_order(row, world, n_groups)
        if imbalance(row, order, world) <= imbalance(row, ident, world) * (1.0 - min_gain):
            plan[layer] = order
    return plan


def inverse_order(order: Sequence[int]) -> List[int]:
    """new physical id of every original expert."""
    inv = [0] * len(order)
    for j, e in enumerate(order):
        inv[e] = j
    return inv


def _take(t, index: torch.Tensor):
    """Rows `index` of an expert-indexed tensor, or of every part of a quantised expert weight."""
    if t is None:
        return None
    if isinstance(t, torch.Tensor):
        return t[index.to(t.device)].contiguous()
    from ..models.expert_arena import _like, _parts
    return _like(t, [p[index.to(p.device)].contiguous() for p in _parts(t)])


def permute_layer_experts_(lw, order: Sequence[int]) -> None:
    """Renumber the routed experts of one (unsharded) layer in place: physical id j <- original expert order[j]."""
    E = lw.router_w.shape[0]
    if sorted(order) != list(range(E)):
        raise ValueError("order is not a permutation of the layer's experts")
    idx = torch.tensor(list(order), dtype=torch.int64)
    lw.router_w = lw.router_w[idx.to(lw.router_w.device)].contiguous()
    if lw.router_bias is not None:
        lw.router_bias = lw.router_bias[idx.to(lw.router_bias.device)].contiguous()
    if getattr(lw, "hash_table", None) is not None:
        inv = torch.tensor(inverse_order(order), dtype=lw.hash_table.dtype, device=lw.hash_table.device)
        lw.hash_table = inv[lw.hash_table.long()]
    lw.e_w13, lw.e_w2 = _take(lw.e_w13, idx), _take(lw.e_w2, idx)


def permute_experts_(weights, plan: Dict[int, Sequence[int]]) -> None:
    """Apply a placement plan to an unsharded model (layer indices as in `weights.layers`; proposal stages follow
    the target layers)."""
    if getattr(weights, "tp_world", 1) != 1:
        raise ValueError("placement is applied before the experts are sharded over ranks")
    layers = list(weights.layers) + [m.layer for m in getattr(weights, "mtp", [])]
    for layer, order in plan.items():
        lw = layers[layer]
        if not getattr(lw, "is_moe", True) or lw.router_w is None:
            raise ValueError(f"layer {layer} has no routed experts")
        permute_layer_experts_(lw, order)


def plan_from_telemetry(telemetry, world: int, n_groups: int = 1, min_gain: float = 0.02,
                        layers: Optional[int] = None) -> Dict[int, List[int]]:
    """`utils.telemetry.ExpertTelemetry` -> placement plan."""
    rows = telemetry.counts if layers is None else telemetry.counts[:layers]
    return plan_expert_placement(rows, world, n_groups, min_gain)


class RouteCounter:
    """Route statistics of whole forwards: attach to a forward (`ReferenceForward` or `CudaForward`), run
    representative batches, read `telemetry.counts[layer][expert]` (global expert ids).  On the device the ids of
    every MoE layer are copied to the host, so calibration steps run eagerly (no graph, no look-ahead)."""

    def __init__(self, n_layers: int, n_experts: int):
        from ..utils.telemetry import ExpertTelemetry
        self.telemetry = ExpertTelemetry(n_layers, n_experts)
        self.n_experts = n_experts

    def __call__(self, layer: int, idx: torch.Tensor, tokens: int) -> None:
        if layer >= self.telemetry.n_layers:
            return
        counts = torch.bincount(idx.reshape(-1).long().clamp(0, self.n_experts - 1), minlength=self.n_experts)
        self.telemetry.record_counts(layer, counts.tolist(), tokens)

    def attach(self, forward) -> "RouteCounter":
        forward.route_observer = self
        return self

    @staticmethod
    def detach(forward) -> None:
        forward.route_observer = None

    def plan(self, world: int, n_groups: int = 1, min_gain: float = 0.02) -> Dict[int, List[int]]:
        return plan_from_telemetry(self.telemetry, world, n_groups, min_gain)
