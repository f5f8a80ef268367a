"""Hot-set prediction and selection telemetry for routed experts.

`ExpertTelemetry` counts how often each expert of each layer was selected.  `ExpertPredictor`
scores experts from three signals kept per layer - frequency (exponentially decayed count),
recency (steps since last use) and transition (which experts followed the ones used in the
previous step) - and proposes the next prefetch set.  Counterpart of
crates/ferrule-model/src/moe/prediction.rs:14-110, :251-520 and moe/telemetry.rs:11-170.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass
from typing import Dict, Iterable, List, Set


class ExpertTelemetry:
    def __init__(self):
        self.counts: Dict[int, Dict[int, int]] = defaultdict(lambda: defaultdict(int))
        self.tokens: Dict[int, int] = defaultdict(int)

    def record(self, layer: int, experts: Iterable[int], tokens: int = 1) -> None:
        c = self.counts[layer]
        for e in experts:
            c[e] += 1
        self.tokens[layer] += tokens

    def top(self, layer: int, n: int) -> List[int]:
        c = self.counts.get(layer, {})
        return [e for e, _ in sorted(c.items(), key=lambda kv: (-kv[1], kv[0]))[:n]]

    def coverage(self, layer: int, resident: Iterable[int]) -> float:
        c = self.counts.get(layer, {})
        tot = sum(c.values())
        return (sum(c.get(e, 0) for e in resident) / tot) if tot else 0.0


@dataclass
class PredictorWeights:
    frequency: float = 1.0
    recency: float = 0.5
    transition: float = 1.0
    decay: float = 0.95


@dataclass
class PredictionStats:
    predictions: int = 0
    predicted: int = 0
    hits: int = 0

    @property
    def precision(self) -> float:
        return self.hits / self.predicted if self.predicted else 0.0


class ExpertPredictor:
    def __init__(self, n_experts: int, weights: PredictorWeights = None):
        self.n, self.w = n_experts, weights or PredictorWeights()
        self.freq: Dict[int, List[float]] = {}
        self.last: Dict[int, List[int]] = {}
        self.trans: Dict[int, Dict[int, Dict[int, float]]] = {}
        self.prev: Dict[int, Set[int]] = {}
        self.step: Dict[int, int] = defaultdict(int)
        self._last_pred: Dict[int, Set[int]] = {}
        self.stats = PredictionStats()

    def observe(self, layer: int, experts: Iterable[int]) -> None:
        used = set(experts)
        f = self.freq.setdefault(layer, [0.0] * self.n)
        l = self.last.setdefault(layer, [-10 ** 9] * self.n)
        tr = self.trans.setdefault(layer, {})
        self.step[layer] += 1
        for e in range(self.n):
            f[e] *= self.w.decay
        for e in used:
            f[e] += 1.0
            l[e] = self.step[layer]
        for p in self.prev.get(layer, ()):
            row = tr.setdefault(p, {})
            for e in used:
                row[e] = row.get(e, 0.0) * self.w.decay + 1.0
        pred = self._last_pred.pop(layer, None)
        if pred is not None:
            self.stats.hits += len(pred & used)
        self.prev[layer] = used

    def predict(self, layer: int, n: int, exclude: Iterable[int] = ()) -> List[int]:
        f = self.freq.get(layer)
        if f is None:
            return []
        skip = set(exclude)
        l, tr, now = self.last[layer], self.trans.get(layer, {}), self.step[layer]
        fmax = max(max(f), 1e-9)
        score = []
        for e in range(self.n):
            if e in skip:
                continue
            t = sum(tr.get(p, {}).get(e, 0.0) for p in self.prev.get(layer, ()))
            s = self.w.frequency * f[e] / fmax + self.w.recency / (1.0 + now - l[e]) + self.w.transition * t / (1.0 + t)
            score.append((-s, e))
        out = [e for _, e in sorted(score)[:n]]
        self._last_pred[layer] = set(out)
        self.stats.predictions += 1
        self.stats.predicted += len(out)
        return out
