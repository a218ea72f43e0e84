"""LLMEngine: the public inference API (prefill / batched decode rounds / generate).

One engine per GPU rank.  Decode rounds run from captured CUDA graphs: a graph is keyed by the row
layout (rows per sequence x sequences) and the attention split bucket, its inputs (token ids,
positions, segment table, KV bases) live in fixed device buffers refreshed by ONE pinned host->device
copy per round, and the sampled token ids come back with one device->host read.  The reference does
the same per round (engine-rs/src/spec_probe.rs:314-331 `replay_checked`: upload token ids,
graph.replay(); qwen/graph.rs:538-845 batched graphs keyed by the store set and widths).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..config import EngineConfig, ModelConfig
from ..models.model import Model
from ..models.plan import make_plan
from .graphs import GraphCache, RoundGraph, ctx_bucket, runtime_signature


@dataclass
class GenStats:
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    rounds: int = 0
    tokens: int = 0
    drafted_tokens: int = 0
    accepted_drafts: int = 0


class LLMEngine:
    def __init__(self, cfg: ModelConfig, W: dict, ecfg: Optional[EngineConfig] = None, device="cuda",
                 max_seqs: int = 4, kv_tokens_per_seq: int = 4096, tp=None):
        self.cfg, self.ecfg = cfg, ecfg or EngineConfig()
        dtype = torch.float32 if str(device) == "cpu" else torch.bfloat16
        self.model = Model(cfg, W, device=device, dtype=dtype, n_slots=max_seqs,
                           kv_tokens=max_seqs * kv_tokens_per_seq, slot_tokens=kv_tokens_per_seq, tp=tp)
        self.device = self.model.device
        self.graphs = GraphCache(runtime_signature(self.ecfg) if self.device.type == "cuda" else "")
        # every family captures: hashed n-gram layers get their table rows staged with the plan (row ids for a device
        # table, the gathered rows themselves for a host-resident one)
        self.use_graphs = self.ecfg.cuda_graphs and self.device.type == "cuda"
        self.stats = GenStats()
        self._rounds_since_check = 0

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, slot: int, ids: Sequence[int], chunk: Optional[int] = None) -> torch.Tensor:
        """Chunked prefill of a fresh sequence; returns the logits of the last prompt token."""
        chunk = chunk or self.ecfg.prefill_chunk
        m = self.model
        vocab = self.cfg.vocab
        for t in ids:                       # client-supplied ids never index the embedding table unchecked
            if not 0 <= t < vocab and not (1 << 20) <= t < (1 << 24):
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab} entries")
        m.reset_slot(slot)
        last = None
        for c0 in range(0, len(ids), chunk):
            toks = list(ids[c0: c0 + chunk])
            plan = make_plan([(slot, toks, c0)], device=self.device, all_logits=False)
            last = m.forward(plan)
        return last[0]

    @torch.no_grad()
    def prefill_many(self, slots: Sequence[int], ids_list: Sequence[Sequence[int]], chunk: Optional[int] = None) -> torch.Tensor:
        """Prefill of several fresh sequences in shared forwards: every forward takes up to `chunk` rows in total, one
        segment per sequence that still has prompt tokens left, so the weights of a layer (and the trellis decode of
        the experts) are paid once for all of them.  Returns the last-token logits [len(slots), vocab]."""
        chunk = chunk or self.ecfg.prefill_chunk
        m = self.model
        vocab = self.cfg.vocab
        for ids in ids_list:
            for t in ids:
                if not 0 <= t < vocab and not (1 << 20) <= t < (1 << 24):
                    raise ValueError(f"token id {t} is outside the vocabulary of {vocab} entries")
        for s in slots:
            m.reset_slot(s)
        done = [0] * len(slots)
        last: List[Optional[torch.Tensor]] = [None] * len(slots)
        while any(d < len(ids) for d, ids in zip(done, ids_list)):
            live = [i for i, ids in enumerate(ids_list) if done[i] < len(ids)]
            share = max(1, chunk // len(live))
            items = [(slots[i], list(ids_list[i][done[i]: done[i] + share]), done[i]) for i in live]
            out = m.forward(make_plan(items, device=self.device, all_logits=False))
            for row, (i, it) in enumerate(zip(live, items)):
                done[i] += len(it[1])
                if done[i] >= len(ids_list[i]):
                    last[i] = out[row]
        return torch.stack(last)

    # ------------------------------------------------------------------ decode
    def _ctx_bucket(self, max_ctx: int) -> int:
        return ctx_bucket(max_ctx)

    @torch.no_grad()
    def decode_round(self, slots: Sequence[int], ids: Sequence[int]) -> List[int]:
        """One greedy token for each listed sequence (rows batched in one forward)."""
        m = self.model
        pos0 = [m.seqs[s].length for s in slots]
        self._check_capacity(slots, pos0, 1)
        if not self.use_graphs:
            plan = make_plan([(s, [t], p) for s, t, p in zip(slots, ids, pos0)], device=self.device)
            logits = m.forward(plan)
            return m.greedy(logits).tolist()
        key = (tuple(slots), 1, self._ctx_bucket(max(pos0) + 1))
        g = self.graphs.get(key, lambda: RoundGraph(self.model, slots, 1, key[2], pool=self.graphs.pool))
        g.stage([[t] for t in ids], pos0)
        g.run(commit=True)
        torch.cuda.current_stream().synchronize()
        for s, p in zip(slots, pos0):
            m.seqs[s].length = p + 1
        self._rounds_since_check += 1
        if self._rounds_since_check >= 64:
            self.check_device_status()
        return g.out_host.tolist()

    def _check_capacity(self, slots: Sequence[int], pos0: Sequence[int], rows_per_seq: int):
        """Host-side guard of the KV regions: a round that would write a row past a slot's region is refused before
        anything is staged or replayed (a captured round carries fixed KV bases, so the kernels cannot check it)."""
        m = self.model
        for s, p in zip(slots, pos0):
            cap = m.seqs[s].kv_cap
            if p + rows_per_seq > cap:
                raise RuntimeError(f"sequence in slot {s} is at {p} tokens: {rows_per_seq} more row(s) exceed its "
                                   f"KV region of {cap} tokens")

    @torch.no_grad()
    def decode_steps(self, slots: Sequence[int], ids: Sequence[int], steps: int) -> List[List[int]]:
        """`steps` greedy tokens for each listed sequence with the sampled ids fed back on the device: one staging
        copy, `steps` graph replays, one read-back per step queued behind them (no host round trip between steps).
        Returns [steps][len(slots)] token ids.  Falls back to `decode_round` per step where rounds are not captured."""
        m = self.model
        pos0 = [m.seqs[s].length for s in slots]
        self._check_capacity(slots, pos0, steps)
        if not self.use_graphs or self.cfg.ngram_layers:
            out, cur = [], list(ids)
            for _ in range(steps):
                cur = self.decode_round(slots, cur)
                out.append(cur)
            return out
        key = (tuple(slots), 1, self._ctx_bucket(max(pos0) + steps))
        g = self.graphs.get(key, lambda: RoundGraph(self.model, slots, 1, key[2], pool=self.graphs.pool))
        g.stage([[t] for t in ids], pos0)
        ring = torch.empty(steps, len(slots), dtype=torch.int32).pin_memory()
        first = 0
        if g.graph is None:                      # first use of this layout: capture with one ordinary round
            g.run(commit=True)
            ring[0].copy_(g.out_ids, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            g.stage([[int(t)] for t in ring[0].tolist()], [p + 1 for p in pos0])
            first = 1
        for i in range(first, steps):
            g.replay_fed()
            ring[i].copy_(g.fed_out_ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        for s, p in zip(slots, pos0):
            m.seqs[s].length = p + steps
        self._rounds_since_check += steps
        if self._rounds_since_check >= 64:
            self.check_device_status()
        return ring.tolist()

    def check_device_status(self):
        """Fail-stop on a device-side error: a bounded wait that ran out (a peer that never arrived, a stalled
        pipeline) leaves its code in the status word instead of hanging the GPU; the host raises here."""
        self._rounds_since_check = 0
        if self.device.type != "cuda":
            return
        from ..ops import cuda as cu
        st = cu.read_status(self.device)
        if st[0] != 0:
            raise RuntimeError(f"device status {st}: a kernel gave up waiting (code {st[0]}, detail {st[1:]})")

    @torch.no_grad()
    def generate(self, prompts: List[Sequence[int]], max_new: int, stop_ids: Sequence[int] = ()) -> List[List[int]]:
        """Greedy generation for up to `max_seqs` prompts at once (public API used by the bench)."""
        n = len(prompts)
        assert n <= self.model.n_slots
        outs: List[List[int]] = [[] for _ in range(n)]
        t0 = time.perf_counter()
        cur = []
        for s, p in enumerate(prompts):
            cur.append(int(self.model.greedy(self.prefill(s, p).unsqueeze(0))[0]))
            outs[s].append(cur[-1])
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        t1 = time.perf_counter()
        live = list(range(n))
        for _ in range(max_new - 1):
            nxt = self.decode_round(live, [cur[s] for s in live])
            for s, t in zip(live, nxt):
                cur[s] = t
                outs[s].append(t)
            self.stats.rounds += 1
            live = [s for s in live if cur[s] not in stop_ids]
            if not live:
                break
        if self.device.type == "cuda":
            torch.cuda.synchronize()
        t2 = time.perf_counter()
        self.stats.prefill_ms += (t1 - t0) * 1e3
        self.stats.decode_ms += (t2 - t1) * 1e3
        self.stats.tokens += sum(len(o) for o in outs)
        return outs
