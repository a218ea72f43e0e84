"""Hashed n-gram embedding rows for a batch plan (DS-style engram / Qwen-style PLE tables).

The hash of a position needs the two previous token ids of its sequence; the model keeps the id
history per slot.  Rows are gathered from a host table (the real tables are 2^22 x 1024 and larger:
they stay in pinned host memory and are streamed one layer ahead, reference
engine-rs/src/ds41/engram.rs:123-509) or from a device table when it is small.
"""
from __future__ import annotations

import torch

from ..oracle import layers as L


def chain_row_ids(model, slot: int, pos0: int, new_ids) -> list:
    """Table rows of `new_ids` appended to the history of `slot` at `pos0`, in plain integer arithmetic (a decode
    round hashes one or a few positions per sequence: no tensor ops on the host).  Updates the history.  Equals
    `oracle.layers.ngram_ids` on the whole sequence, restricted to the new positions."""
    cfg = model.cfg
    heads = cfg.ngram_heads
    head_rows = model.W["ngram_table"].shape[0] // heads
    hist = getattr(model, "id_history", None)
    if hist is None:
        hist = model.id_history = {}
    past = hist.get(slot, torch.empty(0, dtype=torch.long))[:pos0]
    tail = [-1, -1] + past[-2:].tolist()
    m0, m1, m2 = (L._wrap64(v) for v in L.NGRAM_MULT)
    half = heads // 2
    out = []
    for t in new_ids:
        t = int(t)
        bi = L._wrap64(t * m0) ^ L._wrap64(tail[-1] * m1)
        tri = bi ^ L._wrap64(tail[-2] * m2)
        rb, rt = bi % head_rows, tri % head_rows
        out.append([(rb if h < half else rt) + h * head_rows for h in range(heads)])
        tail.append(t)
    hist[slot] = torch.cat((past, torch.tensor([int(t) for t in new_ids], dtype=torch.long)))
    return out


def row_ids_for_plan(model, plan) -> torch.Tensor:
    """Table row ids [R, heads] (int64, on the host) of every row of the plan; updates the per-slot id history."""
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
        seg_ids = ids_cpu[s.r0: s.r0 + s.n].long()
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
        out.append(rows)
    return torch.cat(out, 0)


def prefetch_for_plan(model, plan):
    """Start the host gather + upload of this forward's table rows (a host-resident table behind an `EngramTable`), so
    that they travel while the layers before the first n-gram layer compute.  No-op for device tables and for
    captured rounds (their rows are staged with the plan)."""
    eng = getattr(model, "engram", None)
    d = plan.dev
    if eng is None or d.get("ngram_emb") is not None or d.get("ngram_rows") is not None or "ngram_fut" in d:
        return
    d["ngram_fut"] = eng.prefetch(row_ids_for_plan(model, plan))


def ngram_rows_for_plan(model, plan) -> torch.Tensor:
    """fp32 [R, heads * dim] concatenated table rows of the plan's positions; computed once per forward (all n-gram
    layers read the same rows through their own projections)."""
    cfg = model.cfg
    table = model.W["ngram_table"]
    d = plan.dev
    if d.get("ngram_emb") is not None:     # captured round, host-resident table: the rows themselves were staged
        return d["ngram_emb"].flatten(1).float()
    staged = d.get("ngram_rows")
    if staged is not None:                 # captured round, device table: the row ids were staged, gather on the device
        return table[staged].flatten(1).float()
    if d.get("ngram_cache") is not None:
        return d["ngram_cache"]
    eng = getattr(model, "engram", None)
    if eng is not None:
        from ..cache.engram import EngramTable
        if "ngram_fut" not in d:
            prefetch_for_plan(model, plan)
        emb = EngramTable.take(d.pop("ngram_fut")).view(plan.rows, -1).float()
    else:
        rows = row_ids_for_plan(model, plan)
        emb = table[rows.to(table.device)].flatten(1).float().to(plan.ids.device)
    d["ngram_cache"] = emb
    return emb
