"""Per-layer expert selection telemetry: how often each routed expert was chosen, for residency planning
and the hot-set predictor.  Counts are accumulated on the host from the route tables a step already
copies back when experts are streamed, or from an explicit `record` call.

Counterpart of crates/ferrule-model/src/moe/telemetry.rs:9-60.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Sequence


class ExpertTelemetry:
    def __init__(self, n_layers: int, n_experts: int):
        self.n_layers, self.n_experts = n_layers, n_experts
        self.counts: List[List[int]] = [[0] * n_experts for _ in range(n_layers)]
        self.tokens: List[int] = [0] * n_layers

    def record(self, layer: int, experts: Iterable[int], tokens: int = 1) -> None:
        row = self.counts[layer]
        for e in experts:
            if 0 <= e < self.n_experts:
                row[e] += 1
        self.tokens[layer] += tokens

    def record_counts(self, layer: int, per_expert: Sequence[int], tokens: int) -> None:
        row = self.counts[layer]
        for e, c in enumerate(per_expert):
            row[e] += int(c)
        self.tokens[layer] += tokens

    def hottest(self, layer: int, k: int) -> List[int]:
        row = self.counts[layer]
        return sorted(range(self.n_experts), key=lambda e: (-row[e], e))[:k]

    def coverage(self, layer: int, resident: Iterable[int]) -> float:
        """Share of this layer's routes that a resident set would have served."""
        row = self.counts[layer]
        total = sum(row)
        return sum(row[e] for e in set(resident)) / total if total else 1.0

    def snapshot(self) -> Dict[str, object]:
        return {"tokens": list(self.tokens), "top": {l: self.hottest(l, 8) for l in range(self.n_layers) if self.tokens[l]}}
