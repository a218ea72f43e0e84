"""Captured CUDA graphs of the serving rounds: target rounds (plain decode, speculative verify, commit of the accepted
rows) and the MTP drafter's chain.

A graph is keyed by its row layout (which slots, rows per sequence) and the attention split bucket.  Everything a
replay reads -- token ids, positions, segment table, sampling parameters, accepted-row counts -- lives in ONE packed
device buffer refreshed by ONE pinned host->device copy; the sampled ids (and the drafter's confidences) come back
with one device->host read.  Rows of a sequence that has fewer drafts than the layout are padded by repeating its last
token at the following positions: a padded row only reads rows written by the same launch, its own KV rows are
overwritten by the next round, and the accept walk never looks at it.
Reference: engine-rs/src/spec_probe.rs:314-331 (`replay_checked`), qwen/graph.rs:538-845 (verify graphs keyed by the
store set and widths, commit graph with device-side accepted counts `nd[]`), spec_probe.rs:1793-1840 (serve_round).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..models.plan import Plan, Segment


class GraphCache:
    """Captured graphs of one engine: least-recently-used eviction, keys prefixed by the flag signature (a changed switch
    can never replay a graph captured under the old setting), one memory pool shared by every capture (graphs of one
    engine replay one at a time on one stream, so they can share their intermediate buffers; what a graph hands out --
    logits, hidden rows, sampled ids -- stays allocated for as long as the graph object lives).
    Reference: engine-rs/src/spec_probe.rs:316-327 (flag signature), qwen/graph.rs:538-845 (graph sets per store set)."""

    def __init__(self, signature: str = "", max_entries: int = 64):
        from collections import OrderedDict
        self.signature, self.max_entries = signature, max_entries
        self.d = OrderedDict()
        self._pool = None
        self.evicted = 0

    @property
    def pool(self):
        if self._pool is None and torch.cuda.is_available():
            self._pool = torch.cuda.graph_pool_handle()
        return self._pool

    def get(self, key: tuple, make):
        full = (self.signature,) + tuple(key)
        g = self.d.get(full)
        if g is not None:
            self.d.move_to_end(full)
            return g
        g = make()
        self.d[full] = g
        while len(self.d) > self.max_entries:
            self.d.popitem(last=False)
            self.evicted += 1
        return g

    def __len__(self):
        return len(self.d)

    def values(self):
        return self.d.values()

    def __bool__(self):
        return len(self.d) > 0


def runtime_signature(ecfg=None) -> str:
    """What a captured graph depends on besides its layout: the engine's flag signature and the kernel-level switches."""
    from ..ops import cuda as cu
    parts = [ecfg.signature() if ecfg is not None else ""]
    for name in ("FUSED_DECODE", "SHARED_AS_PAIR", "FUSED_COMBINE", "SIDE_STREAMS"):
        parts.append(f"{name}={getattr(cu, name, None)}")
    return ";".join(parts)


def ctx_bucket(max_ctx: int) -> int:
    b = 256
    while b < max_ctx:
        b *= 2
    return b


def _layout_arrays(slots, k, dev):
    n = len(slots)
    return {"row_slot": torch.tensor([s for s in slots for _ in range(k)], dtype=torch.int32, device=dev),
            "row_j": torch.tensor(list(range(k)) * n, dtype=torch.int32, device=dev),
            "row_r0": torch.tensor([i * k for i in range(n) for _ in range(k)], dtype=torch.int32, device=dev)}


class RoundGraph:
    """Captured target forward over a fixed row layout (rows_per_seq rows for each listed slot)."""

    def __init__(self, model, slots: Sequence[int], rows_per_seq: int, bucket: int, sample: bool = False, pool=None):
        self.m, self.slots, self.k, self.sample = model, list(slots), rows_per_seq, sample
        self.pool = pool
        m = model
        dev = m.device
        n = len(self.slots)
        R = n * rows_per_seq
        self.R, self.n = R, n
        # packed staging, int32 units: seeds i64[R] | noise positions i64[R] | ids[R] pos[R] row_pos0[R] seg[n*4] |
        # temperatures f32[R] | accepted rows[n]
        self.o_int = 4 * R
        total = 4 * R + 3 * R + 4 * n + R + n
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)
        o = self.o_int
        self.h_seed, self.h_spos = self.host[:2 * R].view(torch.int64), self.host[2 * R:4 * R].view(torch.int64)
        self.h_temp = self.host[o + 3 * R + 4 * n: o + 4 * R + 4 * n].view(torch.float32)
        self.h_acc = self.host[o + 4 * R + 4 * n:]
        self.d_seed, self.d_spos = self.dev[:2 * R].view(torch.int64), self.dev[2 * R:4 * R].view(torch.int64)
        self.d_temp = self.dev[o + 3 * R + 4 * n: o + 4 * R + 4 * n].view(torch.float32)
        self.d_acc = self.dev[o + 4 * R + 4 * n:]
        self.plan_ints = self.dev[o:]                   # [ids | pos | row_pos0 | seg]: what the advance kernel walks
        self.row_kv = torch.zeros(R, dtype=torch.int64, device=dev)
        self.out_host = torch.zeros(R, dtype=torch.int32).pin_memory()
        segs = [Segment(s, i * rows_per_seq, rows_per_seq, 0) for i, s in enumerate(self.slots)]
        self.plan = Plan(ids=torch.zeros(R, dtype=torch.long, device=dev), pos=torch.zeros(R, dtype=torch.long, device=dev),
                         segs=segs, logit_rows=torch.arange(R, device=dev))
        d = {"ids32": self.dev[o: o + R], "pos32": self.dev[o + R: o + 2 * R], "row_pos0": self.dev[o + 2 * R: o + 3 * R],
             "seg": self.dev[o + 3 * R: o + 3 * R + 4 * n].view(n, 4), "row_kv": self.row_kv, "max_ctx": bucket}
        d.update(_layout_arrays(self.slots, rows_per_seq, dev))
        # hashed n-gram layers: the row ids of each position come from the token history, which lives on the host
        self.ng_host = None
        if m.cfg.ngram_layers:
            self.ng_host = torch.zeros(R, m.cfg.ngram_heads, dtype=torch.int64).pin_memory()
            table = m.W["ngram_table"]
            if table.device.type == "cuda":
                d["ngram_rows"] = torch.zeros(R, m.cfg.ngram_heads, dtype=torch.int64, device=dev)
            else:      # host-resident table: the rows themselves are gathered on the host and staged like the ids
                d["ngram_emb"] = torch.zeros(R, m.cfg.ngram_heads, table.shape[1], dtype=table.dtype, device=dev)
        self.plan.dev = d
        self.graph = None
        self.graph_fed = None          # the same round followed by the device-side feedback of the sampled ids
        self.graph_commit = None
        self.pendings = []             # (mixer, pending inputs) of the linear-attention layers of a non-committing round
        self.out_ids = None
        self.logits = None
        self.hidden = None
        self.launches = 0
        self.commit_launches = 0

    # ---------------------------------------------------------------------------------------- staging
    def stage(self, ids: List[List[int]], pos0: List[int], temps: Optional[Sequence[float]] = None,
              seeds: Optional[Sequence[int]] = None):
        R, n, k, o = self.R, self.n, self.k, self.o_int
        h = self.host
        m = self.m
        ids_l, pos_l, p0_l, seg_l = [], [], [], []
        for i, s in enumerate(self.slots):
            p = pos0[i]
            ids_l += list(ids[i]) + [ids[i][-1]] * (k - len(ids[i]))
            pos_l += range(p, p + k)
            p0_l += [p] * k
            seg_l += [s, i * k, k, p]
            self.plan.segs[i].pos0 = p
        h[o: o + 3 * R + 4 * n] = torch.tensor(ids_l + pos_l + p0_l + seg_l, dtype=torch.int32)
        if self.sample:
            self.h_temp.copy_(torch.tensor([(temps[i] if temps is not None else 0.0) for i in range(n) for _ in range(k)],
                                           dtype=torch.float32))
            self.h_seed.copy_(torch.tensor([(seeds[i] if seeds is not None else 0) for i in range(n) for _ in range(k)],
                                           dtype=torch.int64))
            self.h_spos.copy_(torch.tensor([q + 1 for q in pos_l], dtype=torch.int64))
        self.dev.copy_(h, non_blocking=True)
        if self.ng_host is not None:
            from ..models.ngram import chain_row_ids
            for i, s in enumerate(self.slots):
                row = list(ids[i]) + [ids[i][-1]] * (k - len(ids[i]))
                self.ng_host[i * k:(i + 1) * k] = torch.tensor(chain_row_ids(m, s, pos0[i], row), dtype=torch.int64)
            if "ngram_rows" in self.plan.dev:
                self.plan.dev["ngram_rows"].copy_(self.ng_host, non_blocking=True)
            else:
                from ..cache.engram import EngramTable
                emb = EngramTable.take(m.engram.prefetch(self.ng_host))
                self.plan.dev["ngram_emb"].copy_(emb.view_as(self.plan.dev["ngram_emb"]))

    def set_kv(self):
        m = self.m
        kv = torch.tensor([m.seqs[s].kv_base for s in self.slots for _ in range(self.k)], dtype=torch.int64)
        self.row_kv.copy_(kv)

    # ---------------------------------------------------------------------------------------- the round
    def _body(self, commit: bool):
        from ..ops import cuda as cu
        m = self.m
        self.plan.ids = self.plan.dev["ids32"]
        logits = m.forward(self.plan, commit=commit, graph_mode=True)
        self.hidden = m.hidden_out
        if self.sample:
            off = m.tp.rank * logits.shape[1] if m.tp is not None else 0
            logits = cu.gumbel_perturb(logits.contiguous(), self.d_temp, self.d_seed, self.d_spos, off)
        self.logits = logits
        self.out_ids = m.greedy(logits)

    def run(self, commit: bool):
        m = self.m
        from ..ops import cuda as cu
        if self.graph is None:
            self.set_kv()
            # eager warm-up sizes every persistent scratch buffer, then capture
            # (warm-up runs without commit: linear-attention state is written exactly once, by the replay)
            n0 = cu.launch_count()
            self._body(False)
            self.launches = cu.launch_count() - n0
            m._pending_plan = None
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.pool):
                self._body(commit)
            cu.add_launches(-self.launches)       # the capture pass launched nothing
            m._pending_plan = None
            self.graph = g
            if not commit:
                self.pendings = [(mix, mix.pending) for _, mix, _ in m.layers if getattr(mix, "pending", None) is not None]
        self.replay()
        self.out_host.copy_(self.out_ids, non_blocking=True)

    def replay(self):
        from ..ops import cuda as cu
        self.graph.replay()
        cu.add_launches(self.launches)

    def replay_fed(self):
        """Replay the round and feed its sampled ids back on the device: ids <- sampled, every position + 1.  The next
        replay is then the next decode step without any host work in between (one row per sequence, no hashed
        n-gram layers: their row ids come from the host)."""
        from ..ops import cuda as cu
        assert self.k == 1 and self.ng_host is None
        if self.graph_fed is None:
            if self.graph is None:
                raise RuntimeError("run() the round once before device-fed replays")
            torch.cuda.synchronize()
            keep = (self.logits, self.hidden, self.out_ids)      # the plain round's outputs stay its own
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.pool):
                self._body(True)
                cu.check(cu.lib().spark_decode_advance(cu.P(self.plan_ints), cu.P(self.out_ids), self.n, cu.stream()),
                         "spark_decode_advance")
            cu.add_launches(-(self.launches + 1))
            self.graph_fed = g
            self.fed_out_ids = self.out_ids
            self.logits, self.hidden, self.out_ids = keep
        self.graph_fed.replay()
        cu.add_launches(self.launches + 1)

    # ---------------------------------------------------------------------------------------- commit
    def commit_rows(self, counts: Sequence[int]):
        """After a non-committing replay: advance every linear-attention state by the first counts[i] rows of segment
        i.  The counts travel in the packed buffer's tail; the captured launches read them on the device.  KV rows need
        no commit: the accepted prefix already sits in place."""
        from ..ops import cuda as cu
        if not self.pendings:
            return
        for i, c in enumerate(counts):
            self.h_acc[i] = c
        self.d_acc.copy_(self.h_acc, non_blocking=True)
        if self.graph_commit is None:
            n0 = cu.launch_count()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.pool):
                self._commit_body()
            self.commit_launches = cu.launch_count() - n0
            cu.add_launches(-self.commit_launches)
            self.graph_commit = g
        self.graph_commit.replay()
        cu.add_launches(self.commit_launches)

    def _commit_body(self):
        from ..ops import cuda as cu
        for mix, pend in self.pendings:
            if hasattr(mix.c, "gate_rank"):
                cu.kda_mixer(mix, pend[0], pend[1], self.plan, True, n_rows=self.d_acc)
            else:
                cu.gdn_mixer(mix, pend[0], pend[1], self.plan, True, n_rows=self.d_acc)


class MtpGraph:
    """Captured MTP drafter round for a fixed set of slots: catch-up over up to k (hidden, next token) pairs per
    sequence, then `depth` chained draft steps with the sampled draft fed back on the device.  Returns the drafts and
    the drafter's confidence in each (softmax probability of the drafted token) with one read."""

    def __init__(self, model, slots: Sequence[int], k: int, depth: int, bucket: int, pool=None):
        self.m, self.slots, self.k, self.depth = model, list(slots), k, depth
        self.pool = pool
        m, dev = model, model.device
        n = len(self.slots)
        R = n * k
        self.n, self.R = n, R
        H = m.cfg.hidden
        # int32 units: seeds i64[n] | noise positions i64[depth*n] | last rows i64[n] |
        #              A = ids[R] pos[R] row_pos0[R] seg[4n] | B = ids[n] pos[n] row_pos0[n] seg[4n] | temperatures f32[n]
        o64 = 2 * n + 2 * depth * n + 2 * n
        self.oA, self.oB = o64, o64 + 3 * R + 4 * n
        total = self.oB + 3 * n + 4 * n + n
        self.host = torch.zeros(total, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros(total, dtype=torch.int32, device=dev)

        def views(t):
            return (t[:2 * n].view(torch.int64), t[2 * n: 2 * n + 2 * depth * n].view(torch.int64).view(depth, n),
                    t[2 * n + 2 * depth * n: o64].view(torch.int64), t[self.oB + 7 * n:].view(torch.float32))
        self.h_seed, self.h_spos, self.h_last, self.h_temp = views(self.host)
        self.d_seed, self.d_spos, self.d_last, self.d_temp = views(self.dev)
        self.hid_in = torch.zeros(R, H, dtype=torch.float32, device=dev)
        self.kvA = torch.zeros(R, dtype=torch.int64, device=dev)
        self.kvB = torch.zeros(n, dtype=torch.int64, device=dev)
        oA, oB = self.oA, self.oB
        segsA = [Segment(s, i * k, k, 0) for i, s in enumerate(self.slots)]
        self.planA = Plan(ids=torch.zeros(R, dtype=torch.long, device=dev), pos=torch.zeros(R, dtype=torch.long, device=dev),
                          segs=segsA, logit_rows=self.d_last)
        self.planA.gather_logit_rows = True
        dA = {"ids32": self.dev[oA: oA + R], "pos32": self.dev[oA + R: oA + 2 * R], "row_pos0": self.dev[oA + 2 * R: oA + 3 * R],
              "seg": self.dev[oA + 3 * R: oA + 3 * R + 4 * n].view(n, 4), "row_kv": self.kvA, "max_ctx": bucket}
        dA.update(_layout_arrays(self.slots, k, dev))
        self.planA.dev = dA
        segsB = [Segment(s, i, 1, 0) for i, s in enumerate(self.slots)]
        self.planB = Plan(ids=torch.zeros(n, dtype=torch.long, device=dev), pos=torch.zeros(n, dtype=torch.long, device=dev),
                          segs=segsB, logit_rows=torch.arange(n, device=dev))
        dB = {"ids32": self.dev[oB: oB + n], "pos32": self.dev[oB + n: oB + 2 * n], "row_pos0": self.dev[oB + 2 * n: oB + 3 * n],
              "seg": self.dev[oB + 3 * n: oB + 7 * n].view(n, 4), "row_kv": self.kvB, "max_ctx": bucket}
        dB.update(_layout_arrays(self.slots, 1, dev))
        self.planB.dev = dB
        self.plan_ints_B = self.dev[oB:]
        self.out = torch.zeros(2, depth, n, dtype=torch.int32, device=dev)     # [0] drafts, [1] confidences (fp32 bits)
        self.out_host = torch.zeros(2, depth, n, dtype=torch.int32).pin_memory()
        self.graph = None
        self.launches = 0

    def stage(self, pend_tokens: List[List[int]], pend_hidden: List[List[torch.Tensor]], lengths: List[int],
              temps: Sequence[float], seeds: Sequence[int]):
        """pend_tokens[i] / pend_hidden[i]: the (hidden, next token) pairs sequence i's drafter has not seen (1..k of
        them, the last one ends at the committed length lengths[i])."""
        n, k, R, oA, oB, depth = self.n, self.k, self.R, self.oA, self.oB, self.depth
        h = self.host
        rows = []
        for i, s in enumerate(self.slots):
            c = len(pend_tokens[i])
            assert 1 <= c <= k
            toks = list(pend_tokens[i]) + [pend_tokens[i][-1]] * (k - c)
            hid = list(pend_hidden[i]) + [pend_hidden[i][-1]] * (k - c)
            rows += hid
            p0 = lengths[i] - c
            for j in range(k):
                r = i * k + j
                h[oA + r] = toks[j]
                h[oA + R + r] = p0 + j
                h[oA + 2 * R + r] = p0
            h[oA + 3 * R + 4 * i: oA + 3 * R + 4 * i + 4] = torch.tensor([s, i * k, k, p0], dtype=torch.int32)
            self.planA.segs[i].pos0 = p0
            # chain rows: the advance kernel runs before every chain step, so they start one position early
            h[oB + i] = 0
            h[oB + n + i] = lengths[i] - 1
            h[oB + 2 * n + i] = lengths[i] - 1
            h[oB + 3 * n + 4 * i: oB + 3 * n + 4 * i + 4] = torch.tensor([s, i, 1, lengths[i] - 1], dtype=torch.int32)
            self.h_last[i] = i * k + c - 1
            self.h_seed[i] = seeds[i]
            self.h_temp[i] = temps[i]
            for d in range(depth):
                self.h_spos[d, i] = lengths[i] + 1 + d
        self.dev.copy_(h, non_blocking=True)
        self.hid_in.copy_(torch.stack(rows))

    def _body(self):
        from ..ops import cuda as cu
        m = self.m
        off = None
        self.planA.ids = self.planA.dev["ids32"]
        self.planB.ids = self.planB.dev["ids32"]
        lg = m.mtp_forward(self.planA, self.hid_in)
        h = m.mtp_hidden.index_select(0, self.d_last)
        for i in range(self.depth):
            if off is None:
                off = m.tp.rank * lg.shape[1] if m.tp is not None else 0
            x = cu.gumbel_perturb(lg.clone(), self.d_temp, self.d_seed, self.d_spos[i], off)
            tok = m.greedy(x)
            self.out[0, i].copy_(tok)
            self.out[1, i].view(torch.float32).copy_(cu.token_prob(lg, self.out[0, i], m.tp))
            if i + 1 < self.depth:
                cu.check(cu.lib().spark_decode_advance(cu.P(self.plan_ints_B), cu.P(self.out[0, i]), self.n, cu.stream()),
                         "spark_decode_advance")
                lg = m.mtp_forward(self.planB, h)
                h = m.mtp_hidden

    def run(self):
        from ..ops import cuda as cu
        m = self.m
        if self.graph is None:
            self.kvA.copy_(torch.tensor([m.seqs[s].kv_base for s in self.slots for _ in range(self.k)], dtype=torch.int64))
            self.kvB.copy_(torch.tensor([m.seqs[s].kv_base for s in self.slots], dtype=torch.int64))
            keep = self.dev.clone()
            n0 = cu.launch_count()
            self._body()                          # eager warm-up sizes the scratch buffers
            self.launches = cu.launch_count() - n0
            self.dev.copy_(keep)                  # the warm-up advanced the chain rows: restore the staged plan
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, pool=self.pool):
                self._body()
            cu.add_launches(-self.launches)
            self.graph = g
        self.graph.replay()
        cu.add_launches(self.launches)
        self.out_host.copy_(self.out, non_blocking=True)

    def result(self):
        """(drafts [n][depth], confidences [n][depth]) after the stream has been synchronised."""
        d = self.out_host[0].t().tolist()
        c = self.out_host[1].view(torch.float32).t().tolist()
        return d, c


class SpecGraphs:
    """The captured rounds a speculative decoder replays, keyed by layout (LRU, shared pool: `GraphCache`)."""

    def __init__(self, model, signature: str = "", max_entries: int = 64):
        self.m = model
        self.rounds = GraphCache(signature, max_entries)
        self.mtp = GraphCache(signature, max_entries)
        self.mtp._pool = None

    def round_graph(self, slots, k: int, max_ctx: int) -> RoundGraph:
        key = (tuple(slots), k, ctx_bucket(max_ctx))
        return self.rounds.get(key, lambda: RoundGraph(self.m, slots, k, key[2], sample=True, pool=self.rounds.pool))

    def mtp_graph(self, slots, k: int, depth: int, max_ctx: int) -> MtpGraph:
        key = (tuple(slots), k, depth, ctx_bucket(max_ctx))
        return self.mtp.get(key, lambda: MtpGraph(self.m, slots, k, depth, key[3], pool=self.rounds.pool))
