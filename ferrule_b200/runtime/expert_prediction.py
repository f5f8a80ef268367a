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
    """Per layer: decayed use counts, last-use steps and a decayed transition matrix (rows: experts of the previous
    pass, columns: experts of the pass that followed) as numpy arrays - one observation is a few vector operations,
    cheap enough to run for every streamed layer of every step."""

    def __init__(self, n_experts: int, weights: PredictorWeights = None):
        import numpy as np
        self._np = np
        self.n, self.w = n_experts, weights or PredictorWeights()
        self.freq: Dict[int, "np.ndarray"] = {}
        self.last: Dict[int, "np.ndarray"] = {}
        self.trans: Dict[int, "np.ndarray"] = {}
        self.prev: Dict[int, List[int]] = {}
        self.step: Dict[int, int] = defaultdict(int)
        self._last_pred: Dict[int, Set[int]] = {}
        self.stats = PredictionStats()

    def observe(self, layer: int, experts: Iterable[int]) -> None:
        np = self._np
        used = sorted({int(e) for e in experts if 0 <= int(e) < self.n})
        f = self.freq.get(layer)
        if f is None:
            f = self.freq[layer] = np.zeros(self.n)
            self.last[layer] = np.full(self.n, -10 ** 9, dtype=np.int64)
            self.trans[layer] = np.zeros((self.n, self.n), dtype=np.float32)
        self.step[layer] += 1
        f *= self.w.decay
        if used:
            f[used] += 1.0
            self.last[layer][used] = self.step[layer]
            prev = self.prev.get(layer)
            if prev:
                rows = self.trans[layer][np.ix_(prev, used)]
                self.trans[layer][np.ix_(prev, used)] = rows * self.w.decay + 1.0
        pred = self._last_pred.pop(layer, None)
        if pred is not None:
            self.stats.hits += len(pred & set(used))
        self.prev[layer] = used

    def predict(self, layer: int, n: int, exclude: Iterable[int] = ()) -> List[int]:
        np = self._np
        f = self.freq.get(layer)
        if f is None or n <= 0:
            return []
        now = self.step[layer]
        prev = self.prev.get(layer) or []
        t = self.trans[layer][prev].sum(0) if prev else np.zeros(self.n)
        score = (self.w.frequency * f / max(float(f.max()), 1e-9) + self.w.recency / (1.0 + now - self.last[layer])
                 + self.w.transition * t / (1.0 + t))
        skip = [int(e) for e in exclude if 0 <= int(e) < self.n]
        if skip:
            score = score.copy()
            score[skip] = -np.inf
        order = np.lexsort((np.arange(self.n), -score))            # best score first, lower id on ties
        out = [int(e) for e in order[:n] if score[e] > -np.inf]
        self._last_pred[layer] = set(out)
        self.stats.predictions += 1
        self.stats.predicted += len(out)
        return out
