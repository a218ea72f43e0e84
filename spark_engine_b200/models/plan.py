"""Batch plan: which rows (tokens) one forward pass processes.

A forward pass processes `R` rows grouped into segments; a segment is a run of rows of ONE sequence
slot in ascending position order (a prefill chunk, one decode row, or 1+k speculative rows).
The same description drives the torch path (host lists) and the kernels (device int32 arrays), so
graphs captured for a (segments, rows) shape replay with new contents.  The reference batches
<= 8 sequences / <= 64 rows the same way (engine-rs/src/qwen/graph.rs:538-845,
qwen_gdn.cu:636-711 `nseg`, device-side accepted counts `nd[]`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch


@dataclass
class Segment:
    slot: int
    r0: int           # first row of the segment inside the batch
    n: int            # rows
    pos0: int         # position of the first row = committed length of the sequence
    parents: Optional[List[int]] = None   # tree verify: parent row (segment-local, -1 = committed tip)


@dataclass
class Plan:
    ids: torch.Tensor                 # [R] int64 token ids
    pos: torch.Tensor                 # [R] int64 positions (rope / causality)
    segs: List[Segment]
    logit_rows: torch.Tensor          # [L] int64 rows whose logits are wanted
    dev: dict = field(default_factory=dict)   # device-side int32 mirrors for the kernels
    has_media: bool = False                   # some ids are salted media placeholders (outside the vocabulary)
    mm_rows: Optional[list] = None            # multimodal: [(first row, tensor [n, hidden])] written over the embedding
                                              # rows of salted placeholder ids (multimodal/canvas.py)

    @property
    def rows(self) -> int:
        return int(self.ids.shape[0])

    @property
    def is_tree(self) -> bool:
        return any(s.parents is not None for s in self.segs)


def depth_of(parents: List[int]) -> List[int]:
    d = []
    for j, p in enumerate(parents):
        assert p < j, "tree nodes must be in topological order"
        d.append(0 if p < 0 else d[p] + 1)
    return d


def make_plan(items: List[Tuple[int, List[int], int]], device="cpu", all_logits: bool = True,
              parents: Optional[List[Optional[List[int]]]] = None) -> Plan:
    """items: (slot, token ids, pos0) per segment.  `all_logits` False keeps only each segment's
    last row (prefill)."""
    ids, pos, segs, lrows = [], [], [], []
    r = 0
    for i, (slot, toks, pos0) in enumerate(items):
        par = parents[i] if parents is not None else None
        n = len(toks)
        segs.append(Segment(slot, r, n, pos0, par))
        ids += list(toks)
        if par is None:
            pos += list(range(pos0, pos0 + n))
        else:
            pos += [pos0 + d for d in depth_of(par)]
        lrows += list(range(r, r + n)) if all_logits else [r + n - 1]
        r += n
    p = Plan(torch.tensor(ids, dtype=torch.long, device=device),
             torch.tensor(pos, dtype=torch.long, device=device), segs,
             torch.tensor(lrows, dtype=torch.long, device=device))
    if str(device) != "cpu":
        p.dev = plan_device_arrays(p, device)
    return p


def plan_device_arrays(p: Plan, device) -> dict:
    """int32 arrays the kernels read: per-row slot / position / segment-local index / first row."""
    R = p.rows
    row_slot = torch.empty(R, dtype=torch.int32)
    row_j = torch.empty(R, dtype=torch.int32)
    row_r0 = torch.empty(R, dtype=torch.int32)
    row_pos0 = torch.empty(R, dtype=torch.int32)
    for s in p.segs:
        row_slot[s.r0: s.r0 + s.n] = s.slot
        row_j[s.r0: s.r0 + s.n] = torch.arange(s.n, dtype=torch.int32)
        row_r0[s.r0: s.r0 + s.n] = s.r0
        row_pos0[s.r0: s.r0 + s.n] = s.pos0
    seg = torch.tensor([[s.slot, s.r0, s.n, s.pos0] for s in p.segs], dtype=torch.int32)
    return {"row_slot": row_slot.to(device), "row_j": row_j.to(device), "row_r0": row_r0.to(device),
            "row_pos0": row_pos0.to(device), "seg": seg.to(device), "pos32": p.pos.to(torch.int32),
            "ids32": p.ids.to(torch.int32)}
