"""Speculative decoding rounds on top of the model runner: propose -> verify (ONE batched target forward over all
draft rows of all sequences) -> accept -> commit the accepted rows in place -> drafter catch-up.

Drafters: the MTP head chain (`MtpDrafter`: fc(embed(next token), target hidden) -> one layer -> shared lm_head,
chained `depth` times), prompt-lookup drafts, or any callable returning draft chains / trees.  Verification never
writes linear-attention state: the model keeps the rows' inputs pending and `commit` replays the accepted prefix
(reference: qwen/graph.rs:538-845 verify with commit=false + commit graph, spec_probe.rs:1793-1840 serve_round).
Greedy output is token-for-token the output of plain greedy decoding; sampled output uses position-keyed Gumbel
noise shared by drafter and target, so it is a function of (prompt, seed) only.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..models.plan import make_plan
from . import policy as P
from .lookup import LookupIndex
from .tree import Node, accept, chain, parents_of


@dataclass
class SeqSpec:
    """Per-sequence speculative state."""
    slot: int
    last_token: int                       # sampled, not yet in the KV cache / linear state
    hidden: Optional[torch.Tensor] = None  # target hidden of the row that produced last_token  [H]
    pending_mtp: List[tuple] = field(default_factory=list)   # (hidden, token) pairs the MTP cache has not seen yet
    lookup: Optional[LookupIndex] = None
    temperature: float = 0.0
    seed: int = 0
    generated: List[int] = field(default_factory=list)
    drafted: int = 0
    accepted: int = 0
    table: P.AcceptanceTable = field(default_factory=P.AcceptanceTable)


class MtpDrafter:
    """Chain drafts from the MTP head (its own KV cache lives in model.mtp_layers, positions = target positions)."""

    def __init__(self, model):
        self.m = model

    def propose(self, seq: SeqSpec, depth: int):
        """Returns (tokens, confidences).  First feeds the (hidden, token) pairs accepted since the last round
        (catch-up), whose last row yields the first draft; then chains on the head's own hidden state."""
        m = self.m
        dev = m.device
        L = m.seqs[seq.slot].length                      # committed target length; last_token sits at position L
        pend = seq.pending_mtp
        if not pend or depth <= 0:
            return [], []
        n = len(pend)
        pos0 = L - n                                     # MTP row p consumes (hidden_p, token_{p+1})
        toks = [t for _, t in pend]
        hid = torch.stack([h for h, _ in pend]).to(dev)
        plan = make_plan([(seq.slot, toks, pos0)], device=dev, all_logits=False)
        lg = m.mtp_forward(plan, hid)[0]
        seq.pending_mtp = []
        drafts, confs = [], []
        h = m.mtp_hidden[-1]
        for i in range(depth):
            tok = m.sample(lg, seq.temperature, seq.seed, L + 1 + i)
            drafts.append(tok)
            confs.append(m.token_prob(lg, tok))
            if i + 1 == depth:
                break
            plan = make_plan([(seq.slot, [tok], L + i)], device=dev)
            lg = m.mtp_forward(plan, h.unsqueeze(0))[0]
            h = m.mtp_hidden[-1]
        return drafts, confs


class SpecDecoder:
    def __init__(self, model, drafter="mtp", depth: int = 3, policy: str = "all", theta: float = 0.3, tau: float = 0.3,
                 cost: Optional[P.CostModel] = None, max_rows: int = 64, lookup_n: int = 3, graphs: bool = False):
        """`graphs`: replay captured CUDA graphs for the drafter chain, the verify forward and the commit (chain
        rounds on the device); tree rounds and host-side drafters' proposals stay eager."""
        self.m = model
        self.graphs = None
        if graphs and model.device.type == "cuda":
            from ..serving.graphs import SpecGraphs
            self.graphs = SpecGraphs(model)
        self.depth, self.policy, self.theta, self.tau = depth, policy, theta, tau
        self.cost = cost or P.CostModel()
        self.max_rows = max_rows
        self.lookup_n = lookup_n
        self.drafter = MtpDrafter(model) if drafter == "mtp" and model.mtp_layers else drafter
        self.rounds = 0

    # ---------------------------------------------------------------------------------------------
    def start(self, slot: int, prompt: Sequence[int], temperature: float = 0.0, seed: int = 0, chunk: int = 4096) -> SeqSpec:
        """Prefill a fresh sequence and sample its first token."""
        m = self.m
        m.reset_slot(slot)
        pend, last, hid = [], None, None
        for c0 in range(0, len(prompt), chunk):
            toks = list(prompt[c0: c0 + chunk])
            plan = make_plan([(slot, toks, c0)], device=m.device, all_logits=False)
            last = m.forward(plan)[0]
            hid = m.hidden_out
            if m.mtp_layers:
                nxt = list(prompt[c0 + 1: c0 + len(toks) + 1])
                # MTP row p needs token p+1: all but the chunk's last row are known now
                mp = make_plan([(slot, nxt, c0)], device=m.device, all_logits=False) if nxt else None
                if mp is not None:
                    m.mtp_forward(mp, hid[: len(nxt)])
        first = m.sample(last, temperature, seed, len(prompt))
        seq = SeqSpec(slot, first, hid[-1].clone(), temperature=temperature, seed=seed)
        seq.pending_mtp = [(hid[-1].clone(), first)]
        seq.lookup = LookupIndex(self.lookup_n)
        seq.lookup.extend(list(prompt) + [first])
        seq.generated = [first]
        return seq

    def _draft(self, seq: SeqSpec, depth: int):
        if depth <= 0:
            return [], []
        copy = seq.lookup.propose(depth) if seq.lookup is not None else []
        if isinstance(self.drafter, MtpDrafter):
            d, c = self.drafter.propose(seq, depth)
            if len(copy) > len(d):                       # a long verbatim continuation beats the head
                return copy, [0.9] * len(copy)
            return d, c
        if callable(self.drafter):
            return self.drafter(seq, depth)
        return copy, [0.9] * len(copy)

    def _choose(self, seq: SeqSpec, confs, n_seqs: int, other_rows: int) -> int:
        if self.policy == "tau":
            return P.tau_depth(confs, self.tau, self.depth)
        if self.policy == "theta":
            return P.theta_depth(confs, self.theta, self.depth)
        if self.policy == "rate":
            return P.rate_depth(confs, seq.table, self.cost, n_seqs, other_rows, self.depth)
        return min(len(confs), self.depth)

    # ---------------------------------------------------------------------------------------------
    def _propose_graph(self, seqs: List[SeqSpec], L: List[int]):
        """All sequences' MTP chains in one captured replay; same proposals as `_draft` one by one."""
        m, k = self.m, 1 + self.depth
        g = self.graphs.mtp_graph([s.slot for s in seqs], k, self.depth, max(L) + self.depth + 1)
        g.stage([[t for _, t in s.pending_mtp] for s in seqs], [[h for h, _ in s.pending_mtp] for s in seqs], L,
                [s.temperature for s in seqs], [s.seed for s in seqs])
        g.run()
        torch.cuda.current_stream().synchronize()
        drafts, confs = g.result()
        out = []
        for s, d, c in zip(seqs, drafts, confs):
            s.pending_mtp = []
            copy = s.lookup.propose(self.depth) if s.lookup is not None else []
            out.append((copy, [0.9] * len(copy)) if len(copy) > len(d) else (d, c))
        return out

    @torch.no_grad()
    def round(self, seqs: List[SeqSpec], budgets: Optional[List[int]] = None, stop: Sequence[int] = (),
              proposals: Optional[List[tuple]] = None) -> List[List[int]]:
        """One speculative round over all given sequences.  Returns the tokens emitted per sequence.  `proposals`:
        (draft tokens, confidences) per sequence from the caller instead of the drafter."""
        m = self.m
        L = [m.seqs[s.slot].length for s in seqs]
        k_graph = 1 + self.depth
        use_g = (self.graphs is not None and len(seqs) * k_graph <= 16
                 and all(l + k_graph + 1 <= m.seqs[s.slot].kv_cap for s, l in zip(seqs, L)))
        given = proposals is not None
        if given:
            pass
        elif use_g and self.depth > 0 and isinstance(self.drafter, MtpDrafter) and \
                all(1 <= len(s.pending_mtp) <= k_graph for s in seqs):
            proposals = self._propose_graph(seqs, L)
        else:
            proposals = [self._draft(s, self.depth) for s in seqs]
        drafts, draft_confs = [], []
        for s, (d, c) in zip(seqs, proposals):
            k = len(d) if given else self._choose(s, c, len(seqs), sum(1 + len(x) for x in drafts))
            drafts.append(list(d[:k]))
            draft_confs.append(list(c[:k]))
        toks = [[s.last_token] + d for s, d in zip(seqs, drafts)]
        temps, seeds = [s.temperature for s in seqs], [s.seed for s in seqs]
        if use_g and max(len(t) for t in toks) <= k_graph:
            # captured verify: every sequence padded to the layout's rows; the commit replays device-side counts
            k = k_graph if any(drafts) else 1
            vg = self.graphs.round_graph([s.slot for s in seqs], k, max(L) + k)
            vg.stage(toks, L, temps, seeds)
            vg.run(commit=(k == 1))
            torch.cuda.current_stream().synchronize()
            flat = vg.out_host.tolist()
            all_preds = [flat[i * k: i * k + len(t)] for i, t in enumerate(toks)]
            hidden = vg.hidden.clone()                   # the next replay overwrites the graph's buffer
            row0 = [i * k for i in range(len(seqs))]
            plan = None
        else:
            vg = None
            plan = make_plan([(s.slot, t, l) for s, t, l in zip(seqs, toks, L)], device=m.device)
            logits = m.forward(plan, commit=False)
            hidden = m.hidden_out
            rows_of = [(s, seg.pos0 + 1 + j) for s, seg in zip(seqs, plan.segs) for j in range(seg.n)]
            flat = m.sample_rows(logits, [s.temperature for s, _ in rows_of], [s.seed for s, _ in rows_of],
                                 [p for _, p in rows_of])
            all_preds = [flat[seg.r0: seg.r0 + seg.n] for seg in plan.segs]
            row0 = [seg.r0 for seg in plan.segs]
        emitted, accepted_rows = [], []
        for i, (s, d) in enumerate(zip(seqs, drafts)):
            preds = all_preds[i]
            budget = budgets[i] if budgets is not None else None
            path, out, stopped = accept(chain(d), preds[0], preds[1:], budget=budget, stop=stop)
            n = len(path)
            rows = list(range(n + 1)) if len(out) == n + 1 else list(range(len(out)))
            # rows committed: the last sampled token plus the accepted drafts that are actually emitted
            if len(out) <= n:                              # budget or stop cut inside the accepted prefix
                rows = list(range(len(out)))
            accepted_rows.append(rows)
            # online calibration of the cells the rate policy reads: (depth, the drafter's own confidence)
            cj = draft_confs[i]
            for j, tok in enumerate(d):
                s.table.observe(j, cj[j] if j < len(cj) else 0.5, j < n)
            s.drafted += len(d)
            s.accepted += n
            emitted.append(out)
        if vg is None:
            m.commit(accepted_rows)
        else:
            if vg.k > 1:
                vg.commit_rows([len(r) for r in accepted_rows])
            for s, l, rows in zip(seqs, L, accepted_rows):
                m.seqs[s.slot].length = l + len(rows)
        for i, (s, out) in enumerate(zip(seqs, emitted)):
            r0, rows = row0[i], accepted_rows[i]
            # MTP catch-up inputs: (hidden of committed row j, the token that follows it)
            new_pairs = []
            for j in rows:
                nxt = out[j] if j < len(out) else None
                if nxt is not None:
                    new_pairs.append((hidden[r0 + j] if vg is not None else hidden[r0 + j].clone(), nxt))
            s.pending_mtp = new_pairs
            s.last_token = out[-1]
            s.hidden = hidden[r0 + rows[-1]] if vg is not None else hidden[r0 + rows[-1]].clone()
            s.generated.extend(out)
            if s.lookup is not None:
                s.lookup.extend(out)
        self.rounds += 1
        return emitted

    @torch.no_grad()
    def round_tree(self, seqs: List[SeqSpec], trees: List[List[Node]], budgets: Optional[List[int]] = None,
                   stop: Sequence[int] = ()) -> List[List[int]]:
        """One speculative round with a verification TREE per sequence (nodes in topological order, parent -1 = the
        last sampled token): every node is one extra row that sees the committed context plus its own ancestors; the
        accept walk follows the target's samples through the tree and the accepted root-to-leaf path is committed
        (linear-attention states replayed along the path, KV rows compacted).  Tree rows read the committed context
        densely, which equals sequential decoding only while the sparse-attention layers still select everything; past
        that context the tree's first-child spine is verified as a chain (whose rows go through the selection like
        decode rows), so the round stays lossless.  Reference: engine-rs/src/speculative.rs,
        spec_probe.rs:254-460 (tree topologies), mla_latent.rs:472-773."""
        m = self.m
        limit = m.sparse_ctx_limit()
        if limit is not None and any(m.seqs[s.slot].length + 1 + len(nodes) > limit for s, nodes in zip(seqs, trees)):
            props = []
            for nodes in trees:
                spine, cur = [], -1
                while True:
                    nxt = next((i for i, nd in enumerate(nodes) if nd.parent == cur), None)
                    if nxt is None:
                        break
                    spine.append(nodes[nxt].token)
                    cur = nxt
                props.append((spine, [0.5] * len(spine)))
            return self.round(seqs, budgets, stop, proposals=props)
        items, parents = [], []
        for s, nodes in zip(seqs, trees):
            L = m.seqs[s.slot].length
            items.append((s.slot, [s.last_token] + [n.token for n in nodes], L))
            parents.append([-1] + [n.parent + 1 for n in nodes])
        plan = make_plan(items, device=m.device, parents=parents)
        logits = m.forward(plan, commit=False)
        hidden = m.hidden_out
        emitted, accepted_rows = [], []
        temps, seeds, poss = [], [], []
        for s, seg in zip(seqs, plan.segs):
            depth = [0] * seg.n
            for j in range(1, seg.n):
                depth[j] = depth[seg.parents[j]] + 1
            temps += [s.temperature] * seg.n
            seeds += [s.seed] * seg.n
            poss += [seg.pos0 + 1 + d for d in depth]
        all_preds = m.sample_rows(logits, temps, seeds, poss)
        for i, (s, nodes) in enumerate(zip(seqs, trees)):
            seg = plan.segs[i]
            preds = all_preds[seg.r0: seg.r0 + seg.n]
            budget = budgets[i] if budgets is not None else None
            path, out, _ = accept(nodes, preds[0], preds[1:], budget=budget, stop=stop)
            rows = [0] + [n + 1 for n in path]
            rows = rows[: len(out)] if len(out) <= len(path) else rows
            accepted_rows.append(rows)
            s.drafted += len(nodes)
            s.accepted += len(path)
            emitted.append(out)
        m.commit(accepted_rows)
        for i, (s, out) in enumerate(zip(seqs, emitted)):
            seg, rows = plan.segs[i], accepted_rows[i]
            s.pending_mtp = [(hidden[seg.r0 + r].clone(), out[j]) for j, r in enumerate(rows) if j < len(out)]
            s.last_token = out[-1]
            s.hidden = hidden[seg.r0 + rows[-1]].clone()
            s.generated.extend(out)
            if s.lookup is not None:
                s.lookup.extend(out)
        self.rounds += 1
        return emitted

    def generate(self, prompts: List[Sequence[int]], max_new: int, stop: Sequence[int] = (), temperature: float = 0.0,
                 seed: int = 0) -> List[List[int]]:
        seqs = [self.start(i, p, temperature, seed) for i, p in enumerate(prompts)]
        live = [s for s in seqs if len(s.generated) < max_new and s.generated[-1] not in stop]
        while live:
            budgets = [max_new - len(s.generated) for s in live]
            self.round(live, budgets, stop)
            live = [s for s in live if len(s.generated) < max_new and s.generated[-1] not in stop]
        return [s.generated[:max_new] for s in seqs]
