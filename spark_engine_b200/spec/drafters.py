"""Model-conditioned drafters besides the MTP chain.

`FeatureDrafter` (DFlash2 style): a small bf16/fp32 model conditioned on feature taps of the target (residual stream
after a few layers, concatenated), with grouped causal-conv blocks, windowed GQA over its own slab of past states and
an MLP; for each of `depth` future positions a selector emits the top-K candidate tokens of a sub-vocabulary head
with unary scores, plus pairwise edge scores between consecutive positions; the draft is the greedy path through
(unary + edge), alternatives become siblings of a verification tree.
`StageDrafter` (DSpark style): a stack of draft stages (small top-k MoE blocks) that emit a block of drafts per
round; a Markov head couples each draft to the previous draft token, a confidence head gives the probability that
the draft is accepted, and the draft length is chosen per sequence from the cumulative confidence.
Both are callables `(seq, depth) -> (tokens, confidences)` for `SpecDecoder(drafter=...)`.
Reference: engine-rs/src/dflash.rs:178-262,876-1016 (Candidates{ids,unary,edges,path,conf}), shim/draft_*.cu;
engine-rs/src/ds41/spec.rs:1-24,117-131, ds41/serve.rs:165-237.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from .tree import Node


# ------------------------------------------------------------------------------------------------ candidates
@dataclass
class Candidates:
    ids: torch.Tensor       # [depth, K] candidate token ids per future position
    unary: torch.Tensor     # [depth, K] scores
    edges: torch.Tensor     # [depth-1, K, K] score of (candidate a at j) -> (candidate b at j+1)
    path: List[int]         # chosen candidate index per position
    conf: List[float]       # confidence of the chosen candidate per position


def greedy_path(unary: torch.Tensor, edges: torch.Tensor) -> List[int]:
    """Position 0: best unary; position j+1: best unary + edge from the chosen candidate (ties -> lowest index)."""
    path = [int(torch.argmax(unary[0]))]
    for j in range(unary.shape[0] - 1):
        path.append(int(torch.argmax(unary[j + 1] + edges[j, path[-1]])))
    return path


def to_tree(c: Candidates, widths: Sequence[int]) -> List[Node]:
    """Verification tree: the greedy path is the spine; at depth j the `widths[j] - 1` best other candidates (by
    unary + edge from the spine's previous node) hang off the same parent as leaves.  Parents precede children."""
    nodes: List[Node] = []
    parent = -1
    for j, w in enumerate(widths[: c.ids.shape[0]]):
        score = c.unary[j] if j == 0 else c.unary[j] + c.edges[j - 1, c.path[j - 1]]
        order = torch.sort(score, descending=True, stable=True).indices.tolist()
        spine = len(nodes)
        nodes.append(Node(parent, int(c.ids[j, c.path[j]])))
        for a in [a for a in order if a != c.path[j]][: max(0, w - 1)]:
            nodes.append(Node(parent, int(c.ids[j, a])))
        parent = spine
    return nodes


# ------------------------------------------------------------------------------------------------ DFlash2 style
@dataclass
class FeatureDrafterConfig:
    target_hidden: int = 256
    taps: Sequence[int] = (0, 1)         # target layers whose residual stream conditions the drafter
    d_model: int = 128
    n_layers: int = 2
    n_q: int = 4
    n_kv: int = 2
    head_dim: int = 32
    window: int = 64                     # past drafter states kept per sequence
    conv_k: int = 4
    conv_groups: int = 4
    depth: int = 4                       # future positions per step
    cand_k: int = 16
    sub_vocab: int = 512                 # head scores only the first `sub_vocab` (most frequent) tokens
    edge_rank: int = 32
    vocab: int = 1024


def init_feature_drafter(c: FeatureDrafterConfig, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    m = lambda *s: torch.randn(*s, generator=g) * 0.05
    W = {"fc": m(c.d_model, len(c.taps) * c.target_hidden), "embed": m(c.vocab, c.d_model), "norm": torch.ones(c.d_model),
         "pos_q": m(c.depth, c.d_model, c.d_model), "head": m(c.sub_vocab, c.d_model),
         "edge_u": m(c.edge_rank, c.d_model), "edge_v": m(c.edge_rank, c.d_model), "layers": []}
    for _ in range(c.n_layers):
        W["layers"].append({"n1": torch.ones(c.d_model), "conv": m(c.d_model, c.d_model // c.conv_groups, c.conv_k),
                            "qkv": m((c.n_q + 2 * c.n_kv) * c.head_dim, c.d_model), "o": m(c.d_model, c.n_q * c.head_dim),
                            "n2": torch.ones(c.d_model), "fc1": m(4 * c.d_model, c.d_model), "fc2": m(c.d_model, 4 * c.d_model)})
    return W


def _rms(x, w, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _to(W, device):
    if isinstance(W, dict):
        return {k: _to(v, device) for k, v in W.items()}
    if isinstance(W, list):
        return [_to(v, device) for v in W]
    return W.to(device)


def select_candidates(logits: torch.Tensor, embed: torch.Tensor, edge_u: torch.Tensor, edge_v: torch.Tensor, K: int):
    """logits [depth, sub_vocab] -> (ids, unary, edges, path, conf): sorted top-K log-probabilities per position,
    low-rank pairwise scores and the greedy path.  On the device: two kernels (`draft.cu`) around two small matmuls."""
    if logits.is_cuda:
        from ..ops import cuda as cu
        ids, unary = cu.draft_topk(logits.float().contiguous(), K)
        e = embed[ids.long()]
        edges, path, _, conf = cu.draft_path(unary, ids, (e @ edge_u.t()).float().contiguous(),
                                             (e @ edge_v.t()).float().contiguous())
        return ids.long(), unary, edges, path.tolist(), conf.tolist()
    logp = torch.log_softmax(logits, -1)
    unary, ids = torch.sort(logp, dim=-1, descending=True, stable=True)
    unary, ids = unary[:, :K], ids[:, :K]
    e = embed[ids]                                                                    # [depth, K, d_model]
    edges = torch.einsum("jar,jbr->jab", e[:-1] @ edge_u.t(), e[1:] @ edge_v.t())
    path = greedy_path(unary, edges)
    return ids, unary, edges, path, [float(torch.exp(unary[j, a])) for j, a in enumerate(path)]


class FeatureDrafter:
    def __init__(self, model, cfg: FeatureDrafterConfig, W: Optional[dict] = None, seed: int = 0, device="cpu"):
        """`device`: where the drafter's weights and windows live; on a GPU the candidate selection runs on kernels."""
        self.m, self.c = model, cfg
        self.device = torch.device(device)
        self.W = _to(W or init_feature_drafter(cfg, seed), self.device)
        model.tap_layers = set(cfg.taps)
        self.slabs = {}                   # slot -> [n_layers] list of (k, v, conv history) windows
        self.last: Optional[Candidates] = None

    def _features(self, seq) -> torch.Tensor:
        """Concatenated taps of the row that produced seq.last_token (the target ran it in the previous round)."""
        taps = getattr(self.m, "taps", {})
        rows = [taps[i][-1].float().flatten().to(self.device) for i in self.c.taps]
        return torch.cat(rows)

    def _step(self, slot: int, x: torch.Tensor) -> torch.Tensor:
        """One drafter position: x [d_model] -> hidden [d_model]; appends to the slot's windows."""
        c, W = self.c, self.W
        st = self.slabs.setdefault(slot, [{"k": [], "v": [], "h": []} for _ in range(c.n_layers)])
        for lw, s in zip(W["layers"], st):
            h = _rms(x, lw["n1"])
            s["h"] = (s["h"] + [h])[-c.conv_k:]
            hist = torch.stack([torch.zeros_like(h)] * (c.conv_k - len(s["h"])) + s["h"], 1)      # [d_model, conv_k]
            gsz = c.d_model // c.conv_groups                  # grouped causal conv: output o reads its group's channels
            conv = torch.einsum("goik,gik->go", lw["conv"].view(c.conv_groups, gsz, gsz, c.conv_k),
                                hist.view(c.conv_groups, gsz, c.conv_k)).reshape(c.d_model)
            h = F.silu(conv)
            qkv = lw["qkv"] @ h
            q = qkv[: c.n_q * c.head_dim].view(c.n_q, c.head_dim)
            k = qkv[c.n_q * c.head_dim: (c.n_q + c.n_kv) * c.head_dim].view(c.n_kv, c.head_dim)
            v = qkv[(c.n_q + c.n_kv) * c.head_dim:].view(c.n_kv, c.head_dim)
            s["k"] = (s["k"] + [k])[-c.window:]
            s["v"] = (s["v"] + [v])[-c.window:]
            K, V = torch.stack(s["k"], 1), torch.stack(s["v"], 1)                    # [n_kv, T, D]
            rep = c.n_q // c.n_kv
            att = torch.softmax(torch.einsum("hd,htd->ht", q, K.repeat_interleave(rep, 0)) / c.head_dim ** 0.5, -1)
            x = x + lw["o"] @ torch.einsum("ht,htd->hd", att, V.repeat_interleave(rep, 0)).flatten()
            x = x + lw["fc2"] @ F.gelu(lw["fc1"] @ _rms(x, lw["n2"]))
        return x

    def candidates(self, seq) -> Candidates:
        c, W = self.c, self.W
        x = W["fc"] @ self._features(seq) + W["embed"][seq.last_token]
        h = _rms(self._step(seq.slot, x), W["norm"])
        q = torch.einsum("jde,e->jd", W["pos_q"], h)                                  # one query per future position
        logits = q @ W["head"].t()                                                    # [depth, sub_vocab]
        ids, unary, edges, path, conf = select_candidates(logits, W["embed"], W["edge_u"], W["edge_v"], c.cand_k)
        self.last = Candidates(ids, unary, edges, path, conf)
        return self.last

    def __call__(self, seq, depth: int):
        cand = self.candidates(seq)
        n = min(depth, len(cand.path))
        return [int(cand.ids[j, cand.path[j]]) for j in range(n)], cand.conf[:n]


# ------------------------------------------------------------------------------------------------ DSpark style
@dataclass
class StageDrafterConfig:
    hidden: int = 256
    stages: int = 3
    block: int = 5                       # drafts per round
    n_experts: int = 8
    top_k: int = 3
    ffn: int = 64
    markov_rank: int = 16
    vocab: int = 1024
    threshold: float = 0.5               # stop drafting when the cumulative confidence falls below


def init_stage_drafter(c: StageDrafterConfig, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    m = lambda *s: torch.randn(*s, generator=g) * 0.05
    return {"embed": m(c.vocab, c.hidden), "head": m(c.vocab, c.hidden), "mk_a": m(c.vocab, c.markov_rank),
            "mk_b": m(c.vocab, c.markov_rank), "conf": m(c.hidden), "norm": torch.ones(c.hidden),
            "stages": [{"mix": m(c.hidden, 2 * c.hidden), "gate": m(c.n_experts, c.hidden),
                        "w_gu": m(c.n_experts, 2 * c.ffn, c.hidden), "w_down": m(c.n_experts, c.hidden, c.ffn)}
                       for _ in range(c.stages)]}


class StageDrafter:
    def __init__(self, cfg: StageDrafterConfig, W: Optional[dict] = None, seed: int = 0):
        self.c, self.W = cfg, W or init_stage_drafter(cfg, seed)

    def _stage(self, sw, h, e):
        c = self.c
        x = sw["mix"] @ torch.cat((h, e))
        p = torch.softmax(sw["gate"] @ x, -1)
        idx = torch.sort(p, descending=True, stable=True).indices[: c.top_k]
        w = p[idx] / p[idx].sum()
        out = torch.zeros_like(x)
        for wi, ei in zip(w.tolist(), idx.tolist()):                                   # slot order, like the target's MoE
            gu = sw["w_gu"][ei] @ x
            out = out + wi * (sw["w_down"][ei] @ (F.silu(gu[: c.ffn]) * gu[c.ffn:]))
        return h + out

    def propose_block(self, hidden: torch.Tensor, last_token: int):
        """Up to `block` drafts with their confidences; every draft conditions the next through the Markov head
        (low-rank bigram term) and the stages' recurrent hidden."""
        c, W = self.c, self.W
        h, tok = hidden.float().flatten().cpu(), last_token
        toks, confs = [], []
        for _ in range(c.block):
            e = W["embed"][tok]
            for sw in W["stages"]:
                h = self._stage(sw, h, e)
            hn = _rms(h, W["norm"])
            logits = W["head"] @ hn + W["mk_b"] @ W["mk_a"][tok]                       # Markov head: bigram coupling
            tok = int(torch.argmax(logits))
            toks.append(tok)
            confs.append(float(torch.sigmoid(W["conf"] @ hn + torch.log_softmax(logits, -1)[tok])))
        return toks, confs

    def draft_length(self, confs: Sequence[float], cap: int) -> int:
        """Per-sequence length: the longest prefix whose cumulative confidence stays >= threshold."""
        acc, n = 1.0, 0
        for cf in confs[:cap]:
            acc *= cf
            if acc < self.c.threshold:
                break
            n += 1
        return n

    def __call__(self, seq, depth: int):
        toks, confs = self.propose_block(seq.hidden, seq.last_token)
        n = self.draft_length(confs, min(depth, self.c.block))
        return toks[:n], confs[:n]
