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
                 cost: Optional[P.CostModel] = None, max_rows: int = 64, lookup_n: int = 3):
        self.m = model
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
    @torch.no_grad()
    def round(self, seqs: List[SeqSpec], budgets: Optional[List[int]] = None, stop: Sequence[int] = ()) -> List[List[int]]:
        """One speculative round over all given sequences.  Returns the tokens emitted per sequence."""
        m = self.m
        drafts, draft_confs = [], []
        for s in seqs:
            d, c = self._draft(s, self.depth)
            k = self._choose(s, c, len(seqs), sum(1 + len(x) for x in drafts))
            drafts.append(d[:k])
            draft_confs.append(list(c[:k]))
        items = []
        for s, d in zip(seqs, drafts):
            L = m.seqs[s.slot].length
            items.append((s.slot, [s.last_token] + d, L))
        plan = make_plan(items, device=m.device)
        logits = m.forward(plan, commit=False)
        hidden = m.hidden_out
        emitted, accepted_rows = [], []
        rows_of = [(s, seg.pos0 + 1 + j) for s, seg in zip(seqs, plan.segs) for j in range(seg.n)]
        all_preds = m.sample_rows(logits, [s.temperature for s, _ in rows_of], [s.seed for s, _ in rows_of],
                                  [p for _, p in rows_of])
        for i, (s, d) in enumerate(zip(seqs, drafts)):
            seg = plan.segs[i]
            L = seg.pos0
            preds = all_preds[seg.r0: seg.r0 + seg.n]
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
        m.commit(accepted_rows)
        for i, (s, out) in enumerate(zip(seqs, emitted)):
            seg, rows = plan.segs[i], accepted_rows[i]
            toks_in = [s.last_token] + drafts[i]
            # MTP catch-up inputs: (hidden of committed row j, the token that follows it)
            new_pairs = []
            for j in rows:
                nxt = out[j] if j < len(out) else None
                if nxt is not None:
                    new_pairs.append((hidden[seg.r0 + j].clone(), nxt))
            s.pending_mtp = new_pairs
            s.last_token = out[-1]
            s.hidden = hidden[seg.r0 + rows[-1]].clone()
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
        (linear-attention states replayed along the path, KV rows compacted).  Reference: engine-rs/src/speculative.rs,
        spec_probe.rs:254-460 (tree topologies), mla_latent.rs:472-773."""
        m = self.m
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
