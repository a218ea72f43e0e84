"""Speculative verification core: draft trees, the acceptance walk and stop handling.

A draft is a list of nodes in topological order, `Node(parent, token)`, parent = -1 for children of the committed
tip.  The target scores every node in ONE forward (node j sees the committed context plus its ancestors); the
walk then follows, from the tip, the first child whose token equals the target's prediction at the current node,
until no child matches.  The accepted path plus the target's prediction at its end (the bonus token) are exactly
the tokens greedy decoding would have produced.  Reference: engine-rs/src/speculative.rs:3-38 (Node, accept walk),
qwen/spec.rs:89-96 (chain prefix match).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple


@dataclass(frozen=True)
class Node:
    parent: int
    token: int


def check_topological(nodes: Sequence[Node]) -> None:
    for j, n in enumerate(nodes):
        if not -1 <= n.parent < j:
            raise ValueError(f"node {j}: parent {n.parent} is not an earlier node")


def chain(tokens: Sequence[int]) -> List[Node]:
    return [Node(i - 1, t) for i, t in enumerate(tokens)]


def accept(nodes: Sequence[Node], root_pred: int, node_preds: Sequence[int], budget: Optional[int] = None,
           stop: Sequence[int] = ()) -> Tuple[List[int], List[int], bool]:
    """Walk the tree.  root_pred = target's prediction after the committed tip (the token that must come next);
    node_preds[j] = target's prediction after node j.  Returns (accepted node indices, emitted tokens, stopped):
    emitted = accepted tokens + the bonus prediction, cut at `budget` tokens and after the first stop token."""
    check_topological(nodes)
    path: List[int] = []
    out: List[int] = []
    want, cur = root_pred, -1
    stopped = False
    while True:
        if budget is not None and len(out) >= budget:
            return path, out, stopped
        nxt = next((j for j, n in enumerate(nodes) if n.parent == cur and n.token == want), None)
        if nxt is None:
            out.append(want)                       # bonus token: the target's own prediction
            stopped = want in stop
            return path, out, stopped
        path.append(nxt)
        out.append(want)
        if want in stop:
            return path, out, True
        cur, want = nxt, node_preds[nxt]


def parents_of(nodes: Sequence[Node]) -> List[int]:
    return [n.parent for n in nodes]
