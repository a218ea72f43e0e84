"""Draft-length policies: how many draft tokens to verify for a sequence this round.

  tau rule   : depth = number of leading draft positions whose confidence >= tau, at least 1
               (reference: engine-rs/src/spec_policy.rs:31-34)
  theta rule : longest prefix whose cumulative confidence product stays >= theta (qwen/graph.rs:127-537)
  rate rule  : maximise expected emitted tokens per millisecond with a step-cost model, acceptance
               probabilities from a calibrated table updated online per request (spec_policy.rs:28-106)
  cost model : DS-style round cost = base + per_seq * seqs + per_row * rows ms, used to split a row budget
               over the sequences of a batch (ds41/serve.rs:165-237: 22 + 0.5 seqs + 2.5 rows)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence


def tau_depth(conf: Sequence[float], tau: float, max_depth: int) -> int:
    d = 0
    for c in conf[:max_depth]:
        if c < tau:
            break
        d += 1
    return max(1, d) if conf else 0


def theta_depth(conf: Sequence[float], theta: float, max_depth: int) -> int:
    p, d = 1.0, 0
    for c in conf[:max_depth]:
        p *= c
        if p < theta:
            break
        d += 1
    return d


@dataclass
class CostModel:
    base_ms: float = 22.0
    per_seq_ms: float = 0.5
    per_row_ms: float = 2.5

    def round_ms(self, seqs: int, rows: int) -> float:
        return self.base_ms + self.per_seq_ms * seqs + self.per_row_ms * rows

    def fit(self, samples: Sequence[tuple]) -> None:
        """Recursive-least-squares style refit from (seqs, rows, measured ms) samples (closed form, 3 unknowns)."""
        import numpy as np
        if len(samples) < 4:
            return
        A = np.array([[1.0, s, r] for s, r, _ in samples])
        y = np.array([m for _, _, m in samples])
        x, *_ = np.linalg.lstsq(A, y, rcond=None)
        self.base_ms, self.per_seq_ms, self.per_row_ms = (max(float(v), 0.0) for v in x)


@dataclass
class AcceptanceTable:
    """P[depth][bucket]: probability that draft position `depth` is accepted given its confidence bucket,
    calibrated online (exponential moving average per cell)."""
    depths: int = 7
    buckets: int = 20
    prior: float = 0.5
    lr: float = 0.05
    p: List[List[float]] = field(default_factory=list)

    def __post_init__(self):
        if not self.p:
            self.p = [[min(0.99, self.prior + 0.5 * b / self.buckets) for b in range(self.buckets)]
                      for _ in range(self.depths)]

    def _cell(self, depth: int, conf: float):
        return min(depth, self.depths - 1), min(int(conf * self.buckets), self.buckets - 1)

    def prob(self, depth: int, conf: float) -> float:
        d, b = self._cell(depth, conf)
        return self.p[d][b]

    def observe(self, depth: int, conf: float, accepted: bool) -> None:
        d, b = self._cell(depth, conf)
        self.p[d][b] += self.lr * ((1.0 if accepted else 0.0) - self.p[d][b])


def rate_depth(conf: Sequence[float], table: AcceptanceTable, cost: CostModel, seqs: int, other_rows: int,
               max_depth: int) -> int:
    """Depth k maximising E[tokens emitted] / round_ms.  E = 1 + sum_i prod_{j<=i} P_j (bonus token always)."""
    best_k, best_rate = 0, 1.0 / cost.round_ms(seqs, other_rows + 1)
    e, p = 1.0, 1.0
    for k, c in enumerate(conf[:max_depth], start=1):
        p *= table.prob(k - 1, c)
        e += p
        rate = e / cost.round_ms(seqs, other_rows + 1 + k)
        if rate > best_rate:
            best_k, best_rate = k, rate
    return best_k


def split_rows(confs: List[Sequence[float]], row_budget: int, table: AcceptanceTable, max_depth: int) -> List[int]:
    """Per-sequence draft counts under a total row budget: greedily give the next row to the sequence whose next
    draft position has the highest marginal acceptance probability (ragged widths, DSpark-style)."""
    n = len(confs)
    depth = [0] * n
    prob = [1.0] * n
    rows = n                                           # one row per sequence is always verified
    while rows < row_budget:
        best, gain = -1, 0.0
        for i in range(n):
            if depth[i] < min(max_depth, len(confs[i])):
                g = prob[i] * table.prob(depth[i], confs[i][depth[i]])
                if g > gain:
                    best, gain = i, g
        if best < 0:
            break
        prob[best] = gain
        depth[best] += 1
        rows += 1
    return depth
