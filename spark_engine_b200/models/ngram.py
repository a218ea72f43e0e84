"""Hashed n-gram embedding rows for a batch plan (DS-style engram / Qwen-style PLE tables).

The hash of a position needs the two previous token ids of its sequence; the model keeps the id
history per slot.  Rows are gathered from a host table (the real tables are 2^22 x 1024 and larger:
they stay in pinned host memory and are streamed one layer ahead, reference
engine-rs/src/ds41/engram.rs:123-509) or from a device table when it is small.
"""
from __future__ import annotations

import torch

from ..oracle import layers as L


def ngram_rows_for_plan(model, plan) -> torch.Tensor:
    cfg = model.cfg
    table = model.W["ngram_table"]
    head_rows = table.shape[0] // cfg.ngram_heads
    hist = getattr(model, "id_history", None)
    if hist is None:
        hist = model.id_history = {}
    out = []
    ids_cpu = plan.ids.cpu()
    for s in plan.segs:
        past = hist.get(s.slot, torch.empty(0, dtype=torch.long))[: s.pos0]
        seg_ids = ids_cpu[s.r0: s.r0 + s.n]
        if s.parents is None:
            full = torch.cat((past, seg_ids))
            rows = L.ngram_ids(full, cfg.ngram_heads, head_rows)[s.pos0:]
            hist[s.slot] = full
        else:   # tree rows: each node sees its own ancestor chain
            rows = []
            for j in range(s.n):
                chain, i = [], j
                while i >= 0:
                    chain.append(int(seg_ids[i]))
                    i = s.parents[i]
                full = torch.cat((past, torch.tensor(chain[::-1], dtype=torch.long)))
                rows.append(L.ngram_ids(full, cfg.ngram_heads, head_rows)[-1])
            rows = torch.stack(rows)
        out.append(table[rows.to(table.device)].flatten(1).float())
    return torch.cat(out, 0).to(plan.ids.device)
