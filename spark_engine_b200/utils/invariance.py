"""Row-invariance probe: localise the first layer whose output for a row depends on the other rows of the batch.

Decode must be batch-invariant (a sequence decoded next to three others gets the bits it gets alone; captured graphs,
speculative verification and prefix reuse all rely on it).  When an end-to-end check fails, this probe runs the same row
alone and inside a batch on two fresh models with every layer's residual stream tapped (`Model.tap_layers`) and reports
the first layer where the row differs and by how much, i.e. the kernel to look at.
Reference: engine-rs/src/forward.rs:546-556 and spec_probe.rs:2821+ (`probe_begin` / `probe_take` row-invariance taps).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch

from ..models.plan import make_plan


def layer_rows(model, items, device=None) -> List[torch.Tensor]:
    """Residual stream after every layer for the rows of one forward over `items` ([(slot, token ids, first position)])."""
    model.tap_layers = set(range(len(model.layers)))
    model.forward(make_plan(items, device=device or model.device), commit=False)
    taps = [model.taps[i].float().cpu() for i in range(len(model.layers))]
    model.tap_layers = None
    return taps


def first_divergent_layer(make_model: Callable[[], object], prompts: Sequence[Sequence[int]], probe: int = 0,
                          rows: int = 1, atol: float = 0.0) -> Optional[Tuple[int, float]]:
    """Prefill `prompts` on two fresh models, then run `rows` more tokens of sequence `probe` alone on one and together with
    one row of every other sequence on the other.  Returns (layer, max abs difference) of the first layer whose rows for
    the probed sequence differ by more than `atol`, or None when every layer agrees."""
    alone, batch = make_model(), make_model()
    for m in (alone, batch):
        for s, p in enumerate(prompts):
            m.forward(make_plan([(s, list(p[:-rows]) if s == probe else list(p[:-1]), 0)], device=m.device, all_logits=False))
    tail = list(prompts[probe][-rows:])
    pos = len(prompts[probe]) - rows
    a = layer_rows(alone, [(probe, tail, pos)])
    items, r0, at = [], 0, 0
    for s, p in enumerate(prompts):
        toks = tail if s == probe else [p[-1]]
        if s == probe:
            at = r0
        items.append((s, toks, pos if s == probe else len(p) - 1))
        r0 += len(toks)
    b = layer_rows(batch, items)
    for li, (x, y) in enumerate(zip(a, b)):
        d = (x - y[at: at + rows]).abs().max().item()
        if d > atol:
            return li, d
    return None
