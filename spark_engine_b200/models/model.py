"""Incremental model runner: fixed-address sequence state, chunked prefill, batched decode rows,
speculative verify without commit, in-place commit of the accepted rows.

Every layer type has one implementation written against `spark_engine_b200.ops`; the ops run the
hand-written sm_100a kernels on a B200 and plain PyTorch on CPU (fp32 plumbing tests).  State per
sequence slot: linear-attention matrices + conv tails (gated-DeltaNet / KDA), KV rows in a pool
(GQA: K,V + indexer keys; MLA: latent rows + indexer pools).  Verify rows never write linear
state: their inputs are kept pending and `commit()` replays the accepted prefix, as the reference
does for Qwen (`GdnPending`, engine-rs/src/qwen/model.rs:1556-1700) and GLM (correction records,
kda_correction.rs:64-222); KV rows are written in place past the committed length.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F

from ..config import ModelConfig
from ..oracle import layers as L
from .. import ops
from .plan import Plan, Segment, depth_of


class SeqInfo:
    """Committed length and KV region of a slot."""
    __slots__ = ("length", "kv_base", "kv_cap")

    def __init__(self, kv_base: int, kv_cap: int):
        self.length, self.kv_base, self.kv_cap = 0, kv_base, kv_cap


def _anc_mask(seg: Segment) -> torch.Tensor:
    """[n, n] bool: row j may attend to segment row i (ancestors and itself)."""
    n = seg.n
    m = torch.zeros(n, n, dtype=torch.bool)
    for j in range(n):
        if seg.parents is None:
            m[j, : j + 1] = True
        else:
            i = j
            while i >= 0:
                m[j, i] = True
                i = seg.parents[i]
    return m


# ============================================================================= mixers
class GdnMixer:
    def __init__(self, cfg: ModelConfig, w: dict, n_slots: int, device, dtype):
        c = cfg.gdn
        self.cfg, self.c, self.w = cfg, c, w
        self.nq = c.n_k_heads * c.head_dim
        self.nv = c.n_v_heads * c.head_dim
        self.C = 2 * self.nq + self.nv
        self.S = torch.zeros(n_slots, c.n_v_heads, c.head_dim, c.head_dim, device=device, dtype=torch.float32)
        # kernels keep conv tails per value head ([slot, 3, Hv, 3D]) so no two CTAs share an entry
        self.kernel_layout = ops.use_kernels(self.S)
        if self.kernel_layout:
            self.tail = torch.zeros(n_slots, c.conv_k - 1, c.n_v_heads, 3 * c.head_dim, device=device, dtype=torch.float32)
        else:
            self.tail = torch.zeros(n_slots, c.conv_k - 1, self.C, device=device, dtype=torch.float32)
        self.pending = None

    def reset(self, slot: int):
        self.S[slot].zero_()
        self.tail[slot].zero_()

    # The kernels keep the conv history per value head ([3, Hv, 3D]: that head's q, k, v channels); the generic path
    # wants one row of all channels ([3, 2*nq + nv]).  Tree-verify rows run the generic path on the device too.
    def _tail_get(self, slot: int) -> torch.Tensor:
        t = self.tail[slot]
        if not self.kernel_layout:
            return t
        c, D = self.c, self.c.head_dim
        rep = c.n_v_heads // c.n_k_heads
        qk = t[:, ::rep, : 2 * D]                                    # one value head per key head carries q and k
        return torch.cat((qk[..., :D].reshape(3, -1), qk[..., D:].reshape(3, -1), t[..., 2 * D:].reshape(3, -1)), 1)

    def _tail_set(self, slot: int, g: torch.Tensor):
        if not self.kernel_layout:
            self.tail[slot] = g
            return
        c, D = self.c, self.c.head_dim
        rep = c.n_v_heads // c.n_k_heads
        q = g[:, : self.nq].view(3, c.n_k_heads, D).repeat_interleave(rep, 1)
        k = g[:, self.nq: 2 * self.nq].view(3, c.n_k_heads, D).repeat_interleave(rep, 1)
        v = g[:, 2 * self.nq:].view(3, c.n_v_heads, D)
        self.tail[slot] = torch.cat((q, k, v), -1)

    def _seg(self, proj, ab, S0, tail0, parents=None):
        """Sequential oracle math for one segment.  Returns (o_gated, S_end, tail_end) and, for
        trees, per-node states are materialised (torch path only)."""
        c = self.c
        T = proj.shape[0]
        pre = proj[:, : self.C].float()
        z = proj[:, self.C:].float().view(T, c.n_v_heads, c.head_dim)
        b, a = ab[:, : c.n_v_heads].float(), ab[:, c.n_v_heads:].float()
        g = -torch.exp(self.w["A_log"].float()) * F.softplus(a + self.w["dt_bias"].float())
        beta = torch.sigmoid(b)
        rep = c.n_v_heads // c.n_k_heads
        if parents is None:
            y = F.silu(L.causal_conv(pre, self.w["conv"].float(), tail=tail0))
            q, k, v = self._qkv(y)
            o, S = L.gdn_recurrence(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v, g, beta, S0)
            tail = torch.cat((tail0, pre), 0)[-(c.conv_k - 1):]
        else:
            states: Dict[int, tuple] = {-1: (S0, tail0)}
            o = pre.new_empty(T, c.n_v_heads, c.head_dim)
            for j in range(T):
                Sp, tp = states[parents[j]]
                y = F.silu(L.causal_conv(pre[j: j + 1], self.w["conv"].float(), tail=tp))
                q, k, v = self._qkv(y)
                oj, Sj = L.gdn_recurrence(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v,
                                          g[j: j + 1], beta[j: j + 1], Sp)
                o[j] = oj[0]
                states[j] = (Sj, torch.cat((tp, pre[j: j + 1]), 0)[-(c.conv_k - 1):])
            S, tail = states[T - 1]
        o = L.rms(o, self.w["norm"].float(), self.cfg.norm_eps) * torch.sigmoid(z)
        return o.reshape(T, self.nv), S, tail

    def _qkv(self, y):
        c, T = self.c, y.shape[0]
        q = y[:, : self.nq].view(T, c.n_k_heads, c.head_dim)
        k = y[:, self.nq: 2 * self.nq].view(T, c.n_k_heads, c.head_dim)
        v = y[:, 2 * self.nq:].view(T, c.n_v_heads, c.head_dim)
        q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + self.cfg.norm_eps) * c.head_dim ** -0.5
        k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + self.cfg.norm_eps)
        return q, k, v

    def forward(self, h, plan: Plan, seqs, commit: bool):
        proj, ab = ops.linear_pair(h, self.w["in"], self.w["ab"])
        fast = ops.gdn_mixer(self, proj, ab, plan, commit)
        if fast is not None:
            o = fast
        else:
            outs = []
            for s in plan.segs:
                o, S, tail = self._seg(proj[s.r0: s.r0 + s.n], ab[s.r0: s.r0 + s.n], self.S[s.slot],
                                       self._tail_get(s.slot), s.parents)
                if commit:
                    self.S[s.slot] = S
                    self._tail_set(s.slot, tail)
                outs.append(o)
            o = torch.cat(outs, 0).to(h.dtype)
        self.pending = None if commit else (proj, ab, plan)
        return ops.row_parallel(o, self.w["o"], getattr(self, "tp", None))

    def commit(self, accepted: List[List[int]]):
        """Replay the accepted rows (segment-local row indices, a root-to-leaf path) into the state."""
        if self.pending is None:
            return
        proj, ab, plan = self.pending
        if ops.gdn_commit(self, proj, ab, plan, accepted):
            self.pending = None
            return
        for s, rows in zip(plan.segs, accepted):
            if not rows:
                continue
            idx = torch.tensor([s.r0 + j for j in rows], device=proj.device)
            _, S, tail = self._seg(proj[idx], ab[idx], self.S[s.slot], self._tail_get(s.slot))
            self.S[s.slot] = S
            self._tail_set(s.slot, tail)
        self.pending = None

    def state_tensors(self):
        return {"S": self.S, "tail": self.tail}


class KdaMixer:
    def __init__(self, cfg: ModelConfig, w: dict, n_slots: int, device, dtype):
        c = cfg.kda
        self.cfg, self.c, self.w = cfg, c, w
        self.n = c.n_heads * c.head_dim
        self.S = torch.zeros(n_slots, c.n_heads, c.head_dim, c.head_dim, device=device, dtype=torch.float32)
        self.tail = torch.zeros(n_slots, c.conv_k - 1, 3 * self.n, device=device, dtype=torch.float32)
        self.pending = None

    def reset(self, slot: int):
        self.S[slot].zero_()
        self.tail[slot].zero_()

    def _seg(self, pre, lr, S0, tail0, parents=None):
        c, n = self.c, self.n
        T = pre.shape[0]
        r = c.gate_rank
        pre = pre.float()
        lr = lr.float()
        beta = torch.sigmoid(lr[:, 2 * r:])
        g1 = (lr[:, :r] @ self.w["f_b"].float().t()).view(T, c.n_heads, c.head_dim)
        lam = -5.0 / (1.0 + torch.exp(-torch.exp(self.w["A_log"].float()).view(1, -1, 1)
                                      * (g1 + self.w["dt_bias"].float().view(1, c.n_heads, c.head_dim))))
        g2 = (lr[:, r:2 * r] @ self.w["g_b"].float().t()).view(T, c.n_heads, c.head_dim)

        def qkv(y):
            t = y.shape[0]
            q = y[:, :n].view(t, c.n_heads, c.head_dim)
            k = y[:, n:2 * n].view(t, c.n_heads, c.head_dim)
            v = y[:, 2 * n:].view(t, c.n_heads, c.head_dim)
            q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * c.head_dim ** -0.5
            k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
            return q, k, v

        if parents is None:
            y = F.silu(L.causal_conv(pre, self.w["conv"].float(), tail=tail0))
            q, k, v = qkv(y)
            o, S = L.kda_recurrence(q, k, v, lam, beta, S0)
            tail = torch.cat((tail0, pre), 0)[-(c.conv_k - 1):]
        else:
            states = {-1: (S0, tail0)}
            o = pre.new_empty(T, c.n_heads, c.head_dim)
            for j in range(T):
                Sp, tp = states[parents[j]]
                y = F.silu(L.causal_conv(pre[j: j + 1], self.w["conv"].float(), tail=tp))
                q, k, v = qkv(y)
                oj, Sj = L.kda_recurrence(q, k, v, lam[j: j + 1], beta[j: j + 1], Sp)
                o[j] = oj[0]
                states[j] = (Sj, torch.cat((tp, pre[j: j + 1]), 0)[-(c.conv_k - 1):])
            S, tail = states[T - 1]
        o = self.w["o_norm"].float() * (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5)) * torch.sigmoid(g2)
        return o.reshape(T, n), S, tail

    def forward(self, h, plan: Plan, seqs, commit: bool):
        pre, lr = ops.linear_pair(h, self.w["in"], self.w["lr_a"])
        fast = ops.kda_mixer(self, pre, lr, plan, commit)
        if fast is not None:
            o = fast
        else:
            outs = []
            for s in plan.segs:
                o, S, tail = self._seg(pre[s.r0: s.r0 + s.n], lr[s.r0: s.r0 + s.n], self.S[s.slot],
                                       self.tail[s.slot], s.parents)
                if commit:
                    self.S[s.slot], self.tail[s.slot] = S, tail
                outs.append(o)
            o = torch.cat(outs, 0).to(h.dtype)
        self.pending = None if commit else (pre, lr, plan)
        return ops.row_parallel(o, self.w["o"], getattr(self, "tp", None))

    def commit(self, accepted):
        if self.pending is None:
            return
        pre, lr, plan = self.pending
        if ops.kda_commit(self, pre, lr, plan, accepted):
            self.pending = None
            return
        for s, rows in zip(plan.segs, accepted):
            if not rows:
                continue
            idx = torch.tensor([s.r0 + j for j in rows], device=pre.device)
            _, S, tail = self._seg(pre[idx], lr[idx], self.S[s.slot], self.tail[s.slot])
            self.S[s.slot], self.tail[s.slot] = S, tail
        self.pending = None

    def state_tensors(self):
        return {"S": self.S, "tail": self.tail}


class AttnMixer:
    """Softmax GQA with optional q/k norm, output gate and block-sparse selection."""

    def __init__(self, cfg: ModelConfig, w: dict, kv_tokens: int, device, dtype, alloc=None):
        """`alloc(rows, row_shape, dtype, rows_of)`: allocator of the per-token tensors (growable backing), default dense."""
        c = cfg.attn
        self.cfg, self.c, self.w = cfg, c, w
        self.nq = c.n_q_heads * c.head_dim * (2 if c.gated else 1)
        self.nkv = c.n_kv_heads * c.head_dim
        self.fp8 = cfg.kv_dtype == "fp8" and str(device) != "cpu"
        kvd = torch.float8_e4m3fn if self.fp8 else dtype
        alloc = alloc or (lambda rows, shape, dt, rows_of=None: torch.zeros(rows, *shape, device=device, dtype=dt))
        self.k = alloc(kv_tokens, (c.n_kv_heads, c.head_dim), kvd, lambda t: t)
        self.v = alloc(kv_tokens, (c.n_kv_heads, c.head_dim), kvd, lambda t: t)
        if self.fp8:   # per-(token, head) fp32 scale (reference: qwen_qsa.cu:69-177)
            self.ks = alloc(kv_tokens, (c.n_kv_heads,), torch.float32, lambda t: t)
            self.vs = alloc(kv_tokens, (c.n_kv_heads,), torch.float32, lambda t: t)
        if c.sparse_topk_blocks:
            self.ik_raw = alloc(kv_tokens, (c.idx_dim,), torch.float32, lambda t: t)
            self.ik_pool = alloc((kv_tokens + c.block - 1) // c.block + 1, (c.idx_dim,), torch.float32,
                                 lambda t, b=c.block: (t + b - 1) // b + 1)
        self.inv = L.yarn_inv_freq(c.rope_dim, c.rope_theta, c.yarn_factor, c.yarn_orig_len).to(device)
        self.pending = None

    def reset(self, slot: int):
        pass

    # -- KV access (dequantising when FP8) ------------------------------------------------
    def _store(self, base, k, v):
        n = k.shape[0]
        if self.fp8:
            for src, dst, sc in ((k, self.k, self.ks), (v, self.v, self.vs)):
                amax = src.float().abs().amax(-1).clamp_min(1e-8)
                s = amax / 448.0
                dst[base: base + n] = (src.float() / s.unsqueeze(-1)).to(torch.float8_e4m3fn)
                sc[base: base + n] = s
        else:
            self.k[base: base + n] = k.to(self.k.dtype)
            self.v[base: base + n] = v.to(self.v.dtype)

    def _load(self, base, n):
        if self.fp8:
            return (self.k[base: base + n].float() * self.ks[base: base + n].unsqueeze(-1),
                    self.v[base: base + n].float() * self.vs[base: base + n].unsqueeze(-1))
        return self.k[base: base + n].float(), self.v[base: base + n].float()

    def forward(self, h, plan: Plan, seqs, commit: bool):
        c = self.c
        qkv = ops.linear(h, self.w["qkv"])
        fast = ops.attn_mixer(self, qkv, plan, seqs)
        if fast is not None:
            return ops.row_parallel(fast, self.w["o"], getattr(self, "tp", None))
        R = h.shape[0]
        D = c.head_dim
        qg = qkv[:, : self.nq].float().view(R, c.n_q_heads, -1)
        q = qg[..., :D]
        k = qkv[:, self.nq: self.nq + self.nkv].float().view(R, c.n_kv_heads, D)
        v = qkv[:, self.nq + self.nkv: self.nq + 2 * self.nkv].float().view(R, c.n_kv_heads, D)
        if c.qk_norm:
            q = L.rms(q, self.w["q_norm"].float(), self.cfg.norm_eps, True)
            k = L.rms(k, self.w["k_norm"].float(), self.cfg.norm_eps, True)
        q = L.rope_neox(q, plan.pos, c.rope_dim, c.rope_theta, self.inv)
        k = L.rope_neox(k, plan.pos, c.rope_dim, c.rope_theta, self.inv)
        if c.sparse_topk_blocks:
            o0 = self.nq + 2 * self.nkv
            qi = qkv[:, o0: o0 + c.idx_heads * c.idx_dim].float().view(R, c.idx_heads, c.idx_dim)
            qi = L.rope_neox(L.rms(qi, self.w["iq_norm"].float(), self.cfg.norm_eps, True), plan.pos,
                             min(c.rope_dim, c.idx_dim), c.rope_theta, self.inv)
            kr = qkv[:, o0 + c.idx_heads * c.idx_dim:].float()
        rep = c.n_q_heads // c.n_kv_heads
        out = q.new_empty(R, c.n_q_heads, D)
        for s in plan.segs:
            si = seqs[s.slot]
            base, L0 = si.kv_base, s.pos0
            assert L0 + s.n <= si.kv_cap, "sequence capacity exceeded"   # fail before writing state
            sl = slice(s.r0, s.r0 + s.n)
            self._store(base + L0, k[sl], v[sl])
            kk, vv = self._load(base, L0 + s.n)
            mask = torch.zeros(s.n, L0 + s.n, dtype=torch.bool, device=h.device)
            if c.sparse_topk_blocks and s.parents is None:
                self._append_index(base, L0, kr[sl], plan.pos[sl])
                mask = self._sparse_mask(base, L0, s.n, qi[sl]).to(h.device)
            else:
                mask[:, :L0] = True
                mask[:, L0:] = _anc_mask(s).to(h.device)
            sc = torch.einsum("thd,shd->hts", q[sl], kk.repeat_interleave(rep, 1)) / math.sqrt(D)
            sc = sc.masked_fill(~mask.unsqueeze(0), float("-inf"))
            out[sl] = torch.einsum("hts,shd->thd", torch.softmax(sc, -1), vv.repeat_interleave(rep, 1))
        if c.gated:
            out = out * torch.sigmoid(qg[..., D:])
        return ops.linear(out.reshape(R, c.n_q_heads * D).to(h.dtype), self.w["o"])

    def _append_index(self, base, L0, kr, pos):
        """Store raw indexer keys; finish every 4-token block completed by these rows:
        mean-pool BEFORE norm+rope at the block's first position."""
        c = self.c
        n = kr.shape[0]
        self.ik_raw[base + L0: base + L0 + n] = kr
        b0, b1 = L0 // c.block, (L0 + n) // c.block
        if b1 > b0:
            raw = self.ik_raw[base + b0 * c.block: base + b1 * c.block].view(b1 - b0, c.block, c.idx_dim).mean(1)
            p = torch.arange(b0, b1, device=kr.device) * c.block
            kc = L.rope_neox(L.rms(raw, self.w["ik_norm"].float(), self.cfg.norm_eps, True), p,
                             min(c.rope_dim, c.idx_dim), c.rope_theta, self.inv)
            pb = base // c.block
            self.ik_pool[pb + b0: pb + b1] = kc

    def _sparse_mask(self, base, L0, n, qi):
        c = self.c
        pb = base // c.block
        nb = (L0 + n) // c.block
        score = None
        if nb:
            kc = self.ik_pool[pb: pb + nb]
            score = F.relu(torch.einsum("thd,nd->thn", qi, kc)).sum(1) / math.sqrt(c.idx_dim)
        mask = torch.zeros(n, L0 + n, dtype=torch.bool)
        for j in range(n):
            p = L0 + j
            vis = (p + 1) // c.block
            if vis:
                if vis <= c.sparse_topk_blocks:
                    blocks = torch.arange(vis)
                else:
                    blocks = L.stable_topk(score[j, :vis].cpu(), c.sparse_topk_blocks)
                tok = (blocks.unsqueeze(1) * c.block + torch.arange(c.block)).flatten()
                mask[j, tok] = True
            mask[j, vis * c.block: p + 1] = True
        return mask

    def commit(self, accepted):
        """Chains keep their rows in place; a tree path is compacted so accepted node i lands at
        position length+i."""
        pass

    def compact(self, seqs, seg: Segment, rows: List[int]):
        c = self.c
        base = seqs[seg.slot].kv_base + seg.pos0
        tensors = (self.k, self.v) + ((self.ks, self.vs) if self.fp8 else ())
        if c.sparse_topk_blocks:
            tensors = tensors + (self.ik_raw,)
        for i, j in enumerate(rows):
            if i != j:
                for t in tensors:
                    t[base + i] = t[base + j]
        if c.sparse_topk_blocks and ops.use_kernels(self.k):
            # tree rows left their raw indexer keys at their in-flight slots without pooling: finish the blocks that the
            # accepted path completes (mean of the raw keys, then norm + rope at the block's first position)
            kvb, L0, n = seqs[seg.slot].kv_base, seg.pos0, len(rows)
            b0, b1 = L0 // c.block, (L0 + n) // c.block
            if b1 > b0:
                raw = self.ik_raw[kvb + b0 * c.block: kvb + b1 * c.block].view(b1 - b0, c.block, c.idx_dim).mean(1)
                p = torch.arange(b0, b1, device=raw.device) * c.block
                kc = L.rope_neox(L.rms(raw, self.w["ik_norm"].float(), self.cfg.norm_eps, True), p,
                                 min(c.rope_dim, c.idx_dim), c.rope_theta, self.inv)
                self.ik_pool[kvb // c.block + b0: kvb // c.block + b1] = kc

    def state_tensors(self):
        d = {"k": self.k, "v": self.v}
        if self.fp8:
            d.update(ks=self.ks, vs=self.vs)
        if self.c.sparse_topk_blocks:
            d.update(ik_raw=self.ik_raw, ik_pool=self.ik_pool)
        return d


def _latent_tiles(kv_lora: int):
    nt = kv_lora // 128 if kv_lora >= 128 else 1
    return nt, kv_lora // nt


def pack_latent_fp8(rows: torch.Tensor, kv_lora: int) -> torch.Tensor:
    """[n, kv_lora + rope] fp32 -> packed uint8 rows [n, kv_lora + 16 + 2 rope]: e4m3 codes with one fp32 scale per
    tile (amax / 448), four scale slots, the rope dims in bf16."""
    n = rows.shape[0]
    nt, tw = _latent_tiles(kv_lora)
    tiles = rows[:, :kv_lora].reshape(n, nt, tw)
    amax = tiles.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    codes = (tiles / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8).reshape(n, kv_lora)
    sc = torch.zeros(n, 4, dtype=torch.float32, device=rows.device)
    sc[:, :nt] = scale[..., 0]
    rope = rows[:, kv_lora:].to(torch.bfloat16).contiguous().view(torch.uint8).reshape(n, -1)
    return torch.cat((codes, sc.view(torch.uint8).reshape(n, 16), rope), 1)


def unpack_latent_fp8(packed: torch.Tensor, kv_lora: int) -> torch.Tensor:
    n = packed.shape[0]
    nt, tw = _latent_tiles(kv_lora)
    codes = packed[:, :kv_lora].contiguous().view(torch.float8_e4m3fn).float().reshape(n, nt, tw)
    sc = packed[:, kv_lora: kv_lora + 16].contiguous().view(torch.float32)[:, :nt]
    # through bf16, as the kernels expand the codes into bf16 tiles
    lat = (codes * sc.unsqueeze(-1)).reshape(n, kv_lora).to(torch.bfloat16).float()
    rope = packed[:, kv_lora + 16:].contiguous().view(torch.bfloat16).float()
    return torch.cat((lat, rope), 1)


class MlaMixer:
    """Multi-head latent attention in the absorbed form over a latent KV cache (kv_lora + rope dims
    per token), with the DSA indexer (softmax-gated 4-token pools, top-k pools + tail), optional
    sliding window and attention sink.  Reference: engine-rs/src/mla_latent.rs:196-248,406-470;
    dsa.rs:127-230; shim/ds41_attn.cu:90-424."""

    def __init__(self, cfg: ModelConfig, w: dict, kv_tokens: int, device, dtype, alloc=None):
        c = cfg.mla
        self.cfg, self.c, self.w = cfg, c, w
        self.fp8 = cfg.kv_dtype == "fp8" and (str(device) != "cpu" or cfg.kv_quant_on_cpu)
        alloc = alloc or (lambda rows, shape, dt, rows_of=None: torch.zeros(rows, *shape, device=device, dtype=dt))
        if self.fp8:
            # packed rows: kv_lora e4m3 codes | 4 fp32 tile scales | rope dims in bf16 (656 bytes for 512 + 64 against
            # 1152 in bf16; reference: shim/latent.cu:25-47, 528-byte rows without a separate rope part)
            self.lat = alloc(kv_tokens, (c.kv_lora + 16 + 2 * c.rope_dim,), torch.uint8, lambda t: t)
        else:
            self.lat = alloc(kv_tokens, (c.kv_lora + c.rope_dim,), torch.float32 if str(device) == "cpu" else dtype, lambda t: t)
        self.ik = alloc(kv_tokens, (c.idx_dim,), torch.float32, lambda t: t)       # LayerNorm'ed keys
        self.ig = alloc(kv_tokens, (c.idx_dim,), torch.float32, lambda t: t)       # pool gates
        self.pool = alloc(kv_tokens // c.pool + 2, (c.idx_dim,), torch.float32, lambda t, b=c.pool: t // b + 2)
        # absorbed projections: q_nope . W_uk  and  o_lat . W_uv
        kvb = w["kv_b"].float().view(c.n_heads, 2 * c.head_dim, c.kv_lora)
        self.w_uk = kvb[:, : c.head_dim].contiguous()       # [H, D, kv_lora]
        self.w_uv = kvb[:, c.head_dim:].contiguous()        # [H, D, kv_lora]
        self.pending = None

    def reset(self, slot: int):
        pass

    def forward(self, h, plan: Plan, seqs, commit: bool):
        c = self.c
        R = h.shape[0]
        fast = ops.mla_mixer(self, h, plan, seqs)
        if fast is not None:
            return ops.row_parallel(fast, self.w["o"], getattr(self, "tp", None))
        a = ops.linear(h, self.w["a"]).float()
        o0 = c.q_lora
        o1 = o0 + c.kv_lora + c.rope_dim
        cq = L.rms(a[:, :o0], self.w["q_a_norm"].float(), self.cfg.norm_eps)
        ckv = L.rms(a[:, o0: o0 + c.kv_lora], self.w["kv_a_norm"].float(), self.cfg.norm_eps)
        qb = ops.linear(cq.to(h.dtype), self.w["q_b"]).float()
        nq = c.n_heads * (c.head_dim + c.rope_dim)
        q = qb[:, :nq].view(R, c.n_heads, c.head_dim + c.rope_dim)
        qi = qb[:, nq:].view(R, c.idx_heads, c.idx_dim)
        q_lat = torch.einsum("thd,hdl->thl", q[..., : c.head_dim], self.w_uk)          # absorb W_uk
        if c.rope_dim:
            qr = L.rope_neox(q[..., c.head_dim:], plan.pos, c.rope_dim, c.rope_theta)
            kr = L.rope_neox(a[:, o0 + c.kv_lora: o1].view(R, 1, c.rope_dim), plan.pos, c.rope_dim, c.rope_theta)[:, 0]
            row = torch.cat((ckv, kr), -1)
            q_full = torch.cat((q_lat, qr), -1)
        else:
            row, q_full = ckv, q_lat
        ik = L.layer_norm(a[:, o1: o1 + c.idx_dim], self.w["k_ln_w"].float(), self.w["k_ln_b"].float())
        ig = a[:, o1 + c.idx_dim: o1 + 2 * c.idx_dim]
        hw = a[:, o1 + 2 * c.idx_dim:] * c.idx_heads ** -0.5
        scale = 1.0 / math.sqrt(c.head_dim + c.rope_dim)
        out = q_lat.new_empty(R, c.n_heads, c.kv_lora)
        for s in plan.segs:
            si = seqs[s.slot]
            base, L0 = si.kv_base, s.pos0
            assert L0 + s.n <= si.kv_cap, "sequence capacity exceeded"
            sl = slice(s.r0, s.r0 + s.n)
            self._lat_store(base + L0, row[sl])
            if s.parents is None:
                self._append_index(base, L0, ik[sl], ig[sl])
                mask = self._mask(base, L0, s.n, qi[sl], hw[sl]).to(h.device)
            else:
                # tree rows keep their raw indexer keys and gates at their in-flight slots; pools are finished when
                # the accepted path is compacted
                self.ik[base + L0: base + L0 + s.n] = ik[sl]
                self.ig[base + L0: base + L0 + s.n] = ig[sl]
                mask = torch.zeros(s.n, L0 + s.n, dtype=torch.bool, device=h.device)
                mask[:, :L0] = True
                mask[:, L0:] = _anc_mask(s).to(h.device)
            lat = self._lat_load(base, base + L0 + s.n)
            sc = torch.einsum("thl,sl->hts", q_full[sl], lat) * scale
            sc = sc.masked_fill(~mask.unsqueeze(0), float("-inf"))
            if c.sink:
                snk = self.w["sink"].float().view(-1, 1, 1)
                m = torch.maximum(sc.max(-1, keepdim=True).values, snk)
                e = torch.exp(sc - m)
                p = e / (e.sum(-1, keepdim=True) + torch.exp(snk - m))
            else:
                p = torch.softmax(sc, -1)
            out[sl] = torch.einsum("hts,sl->thl", p, lat[:, : c.kv_lora])
        o = torch.einsum("thl,hdl->thd", out, self.w_uv)                                 # expand W_uv
        return ops.linear(o.reshape(R, c.n_heads * c.head_dim).to(h.dtype), self.w["o"])

    def _lat_store(self, lo: int, rows):
        if not self.fp8:
            self.lat[lo: lo + rows.shape[0]] = rows.to(self.lat.dtype)
            return
        self.lat[lo: lo + rows.shape[0]] = pack_latent_fp8(rows.float(), self.c.kv_lora)

    def _lat_load(self, lo: int, hi: int):
        if not self.fp8:
            return self.lat[lo:hi].float()
        return unpack_latent_fp8(self.lat[lo:hi], self.c.kv_lora)

    def _append_index(self, base, L0, ik, ig):
        c = self.c
        n = ik.shape[0]
        self.ik[base + L0: base + L0 + n] = ik
        self.ig[base + L0: base + L0 + n] = ig
        b0, b1 = L0 // c.pool, (L0 + n) // c.pool
        if b1 > b0:
            kb = self.ik[base + b0 * c.pool: base + b1 * c.pool].view(b1 - b0, c.pool, c.idx_dim)
            gb = self.ig[base + b0 * c.pool: base + b1 * c.pool].view(b1 - b0, c.pool, c.idx_dim) \
                + self.w["ape"].float().view(1, c.pool, c.idx_dim)
            pb = base // c.pool
            self.pool[pb + b0: pb + b1] = (torch.softmax(gb, 1) * kb).sum(1)

    def _mask(self, base, L0, n, qi, hw):
        """Visibility [n, L0+n] of each row: its top-k pools (all of them while there are <= top-k), the tokens after
        the last complete pool, and the sliding window.  Vectorised on the device of the cache."""
        c = self.c
        dev = qi.device
        pb = base // c.pool
        tot = L0 + n
        nb = tot // c.pool
        p = L0 + torch.arange(n, device=dev)
        vis = (p + 1) // c.pool
        tok = torch.arange(tot, device=dev).unsqueeze(0)
        mask = (tok >= (vis * c.pool).unsqueeze(1)) & (tok <= p.unsqueeze(1))
        if c.window:
            mask |= (tok >= (p + 1 - c.window).clamp_min(0).unsqueeze(1)) & (tok <= p.unsqueeze(1))
        if nb:
            visible = torch.arange(nb, device=dev).unsqueeze(0) < vis.unsqueeze(1)
            if nb <= c.topk_pools:
                chosen = visible
            else:
                pk = self.pool[pb: pb + nb]
                sc = F.relu(torch.einsum("thd,nd->thn", qi, pk) * c.idx_dim ** -0.5)
                score = torch.einsum("th,thn->tn", hw, sc).masked_fill(~visible, float("-inf"))
                order = torch.sort(score, dim=1, descending=True, stable=True).indices[:, : c.topk_pools]
                chosen = torch.zeros(n, nb, dtype=torch.bool, device=dev).scatter_(1, order, True) & visible
            mask[:, : nb * c.pool] |= chosen.repeat_interleave(c.pool, 1)
        return mask

    def commit(self, accepted):
        pass

    def compact(self, seqs, seg: Segment, rows: List[int]):
        c = self.c
        kvb, L0, n = seqs[seg.slot].kv_base, seg.pos0, len(rows)
        base = kvb + L0
        for i, j in enumerate(rows):
            if i != j:
                for t in (self.lat, self.ik, self.ig):
                    t[base + i] = t[base + j]
        # the pools that the accepted path completes (tree rows never pool at verification time)
        b0, b1 = L0 // c.pool, (L0 + n) // c.pool
        if b1 > b0:
            kb = self.ik[kvb + b0 * c.pool: kvb + b1 * c.pool].view(b1 - b0, c.pool, c.idx_dim)
            gb = self.ig[kvb + b0 * c.pool: kvb + b1 * c.pool].view(b1 - b0, c.pool, c.idx_dim) \
                + self.w["ape"].float().view(1, c.pool, c.idx_dim).to(kb.device)
            self.pool[kvb // c.pool + b0: kvb // c.pool + b1] = (torch.softmax(gb, 1) * kb).sum(1)

    def state_tensors(self):
        return {"lat": self.lat, "ik": self.ik, "ig": self.ig, "pool": self.pool}


# ============================================================================= MLP / MoE
class MoeBlock:
    def __init__(self, cfg: ModelConfig, w: dict):
        self.cfg, self.c, self.w = cfg, cfg.moe, w
        self.dense = "dense_gu" in w

    def forward(self, h, defer: bool = False):
        c = self.c
        if self.dense:
            gu = ops.linear(h, self.w["dense_gu"])
            return ops.linear(ops.swiglu(gu, c.swiglu_limit), self.w["dense_down"])
        return ops.moe(h, self.w, c, defer)


# ============================================================================= the model
class Model:
    def __init__(self, cfg: ModelConfig, W: dict, device="cpu", dtype=torch.float32, n_slots: int = 4,
                 kv_tokens: int = 4096, slot_tokens: Optional[int] = None, tp=None, kv_backing=None):
        """`tp`: tensor/expert-parallel context (spark_engine_b200.parallel.tp); `W` then holds this rank's shard.
        `kv_backing`: a `cache.kv.KvBacking`; the per-token cache tensors then reserve address space for `kv_tokens`
        and are backed on demand (a `KvManager` backs a region before it leases it)."""
        self.cfg, self.W, self.device, self.dtype = cfg, W, torch.device(device), dtype
        self.tp = tp
        self.kv_backing = kv_backing
        self.lcfg = tp.local_config(cfg) if tp is not None else cfg      # per-rank head counts
        self.n_slots, self.kv_tokens = n_slots, kv_tokens
        per = slot_tokens or kv_tokens // n_slots
        # with a growable backing no region exists until a KvManager leases (and backs) one
        self.seqs = [SeqInfo(i * per, per) if kv_backing is None else SeqInfo(0, 0) for i in range(n_slots)]
        self.layers = self._build_layers(W["layers"])
        self.mtp_layers = self._build_layers(W["mtp"]["layers"]) if "mtp" in W else []
        self.hidden_out = None
        # a hashed n-gram table that stays on the host is read through asynchronous gathers into a pinned ring
        self.engram = None
        if cfg.ngram_layers and self.device.type == "cuda" and W["ngram_table"].device.type == "cpu":
            from ..cache.engram import EngramTable
            self.engram = EngramTable(W["ngram_table"], device=self.device, ring_slots=3,
                                      max_rows=4096 * cfg.ngram_heads)
        if tp is not None and hasattr(tp, "sp_min_rows") and (cfg.ngram_layers or cfg.hc_kind != "none"):
            tp.sp_min_rows = 0           # these blocks read the whole residual between updates: keep it replicated

    def _build_layers(self, lws):
        out = []
        for lw in lws:
            kind = lw["type"]
            if kind == "gdn":
                mix = GdnMixer(self.lcfg, lw["mix"], self.n_slots, self.device, self.dtype)
            elif kind == "kda":
                mix = KdaMixer(self.lcfg, lw["mix"], self.n_slots, self.device, self.dtype)
            elif kind == "attn":
                mix = AttnMixer(self.lcfg, lw["mix"], self.kv_tokens, self.device, self.dtype,
                                self.kv_backing.alloc if self.kv_backing is not None else None)
            elif kind == "mla":
                mix = MlaMixer(self.lcfg, lw["mix"], self.kv_tokens, self.device, self.dtype,
                               self.kv_backing.alloc if self.kv_backing is not None else None)
            else:
                raise ValueError(kind)
            mix.tp = self.tp
            out.append((lw, mix, MoeBlock(self.cfg, lw["mlp"])))
        return out

    # -- sequence bookkeeping ---------------------------------------------------------------
    def reset_slot(self, slot: int):
        self.seqs[slot].length = 0
        for _, mix, _ in self.layers + self.mtp_layers:
            mix.reset(slot)

    def set_kv_region(self, slot: int, base: int, cap: int):
        self.seqs[slot].kv_base, self.seqs[slot].kv_cap = base, cap

    # -- forward ----------------------------------------------------------------------------
    def _block(self, lw, mix, mlp, X, pend, plan, commit):
        """One decoder block.  `pend` is the previous block's MLP output, still to be added to the residual
        (under tensor parallelism it is this rank's partial sum): the add, the all-reduce and this block's
        first RMSNorm happen in one fused op.  Returns (X, new pending output)."""
        cfg, tp = self.cfg, self.tp
        if cfg.hc_kind == "none":
            # decode rounds on the device: the MoE combine is deferred into the next residual update (one launch for
            # combine + add + norm; under tensor parallelism the combine happens inside the all-reduce push)
            deferred = plan.rows <= 16 and X.is_cuda and (tp is None or hasattr(tp, "argmax"))
            if "ngram" in lw:
                if pend is not None:
                    _, X = ops.add_rmsnorm(pend, X, lw["in_norm"], cfg.norm_eps, tp)
                    pend = None
                X = ops.ngram_embed(self, X, plan, lw["ngram"])
            h, X = ops.add_rmsnorm(pend, X, lw["in_norm"], cfg.norm_eps, tp)
            a = mix.forward(h, plan, self.seqs, commit)
            h, X = ops.add_rmsnorm(a, X, lw["post_norm"], cfg.norm_eps, tp)
            return X, mlp.forward(h, defer=deferred)
        # hyper-connections: `pend` carries the previous block's output with its write-back coefficients; every site
        # applies it and forms its own mixed row in one pass over the streams
        if cfg.hc_kind == "gated":
            X, h, _, post = ops.hc_gated_site(X, pend, lw["hc_mix"], cfg.norm_eps, tp)
            a = mix.forward(h, plan, self.seqs, commit)
            X, h, _, post2 = ops.hc_gated_site(X, (a, post), lw["hc_mlp"], cfg.norm_eps, tp)
            return X, (mlp.forward(h), post2)
        X, h, post, comb = ops.mhc_site(X, pend, lw["hc_mix"], cfg.sinkhorn_iters, cfg.norm_eps, tp)
        a = mix.forward(h, plan, self.seqs, commit)
        X, h, post2, comb2 = ops.mhc_site(X, (a, post, comb), lw["hc_mlp"], cfg.sinkhorn_iters, cfg.norm_eps, tp)
        return X, (mlp.forward(h), post2, comb2)

    @torch.no_grad()
    def forward(self, plan: Plan, commit: bool = True, want_hidden: bool = False, graph_mode: bool = False):
        """Run all layers over the plan's rows.  Returns logits [len(plan.logit_rows), vocab].
        With commit=False no linear-attention state nor sequence length changes: call
        `commit(accepted)` afterwards."""
        cfg, W = self.cfg, self.W
        if not graph_mode:                   # a captured round carries fixed KV bases: the engine checks before it stages
            for sg in plan.segs:
                if sg.pos0 + sg.n > self.seqs[sg.slot].kv_cap:
                    raise RuntimeError(f"slot {sg.slot}: rows up to position {sg.pos0 + sg.n} exceed its KV region of "
                                       f"{self.seqs[sg.slot].kv_cap} tokens")
        if plan.mm_rows:
            # salted placeholder ids are outside the vocabulary: look up row 0 for them, then write the encoded media
            # rows over those positions (engine-rs/src/weights.rs:536-569)
            from ..multimodal.canvas import MM_BASE, inject_rows
            salted = plan.ids >= MM_BASE
            X = ops.embed(W["embed"], torch.where(salted, torch.zeros_like(plan.ids), plan.ids), self.dtype)
            X[salted.to(X.device)] = 0
            X = inject_rows(X, plan.ids, plan.mm_rows)
        else:
            X = ops.embed(W["embed"], plan.ids, self.dtype)
        if cfg.hc_kind != "none":
            X = X.unsqueeze(1).repeat(1, cfg.hc_streams, 1).contiguous()
        self._ids_for_ngram = plan
        if cfg.ngram_layers and self.engram is not None:
            from .ngram import prefetch_for_plan
            prefetch_for_plan(self, plan)        # the gather and the upload overlap the layers before the first n-gram layer
        pend = None
        taps = getattr(self, "tap_layers", None)
        if taps:
            self.taps = {}
        for li, (lw, mix, mlp) in enumerate(self.layers):
            X, pend = self._block(lw, mix, mlp, X, pend, plan, commit)
            if taps and li in taps:          # residual stream after layer li (feature taps of a drafter)
                self.taps[li] = X if (pend is None or cfg.hc_kind != "none") else ops.residual_add(X.clone(), pend)
        if cfg.hc_kind == "gated":
            _, hn, hf, _ = ops.hc_gated_site(X, pend, W["hc_final"], cfg.norm_eps, self.tp)
            X = hf if hf is not None else hn
        elif cfg.hc_kind == "mhc":
            X, hn = ops.mhc_final(X, pend, W["final_norm"], cfg.norm_eps, self.tp)
        else:
            hn, X = ops.add_rmsnorm(pend, X, W["final_norm"], cfg.norm_eps, self.tp)
        if self.tp is not None and getattr(self.tp, "rows_sharded", False):
            X = self.tp.gather_rows(X)       # sequence-parallel prefill kept the residual row-sharded until here
        self.hidden_out = X
        self._pending_plan = None if commit else plan
        if commit and not graph_mode:       # under a captured graph the engine tracks lengths itself
            for s in plan.segs:
                self.seqs[s.slot].length = s.pos0 + s.n
        if plan.logit_rows.shape[0] != hn.shape[0]:
            hn = hn[plan.logit_rows]
        return ops.lm_head(hn, W["lm_head"])

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        """Greedy token ids (int32) from the logits `forward` returned (vocabulary-parallel under TP)."""
        if self.tp is not None:
            return self.tp.greedy(logits, logits.shape[1])
        return ops.argmax(logits)

    def sample_rows(self, logits: torch.Tensor, temps, seeds, positions) -> List[int]:
        """One token per logits row: Gumbel-max with noise keyed by (seed, position, global vocabulary id) where the
        row's temperature is > 0, greedy otherwise.  Correct under vocabulary parallelism (every rank returns the
        same global ids) and one device-to-host read for all rows.
        Reference: engine-rs/src/sampling.rs:20-170, head_select.rs:1-101."""
        if logits.dim() == 1:
            logits = logits.unsqueeze(0)
        off = self.tp.rank * logits.shape[1] if self.tp is not None else 0
        x = ops.gumbel_perturb(logits, temps, seeds, positions, off, self.cfg.vocab)
        return [int(t) for t in self.greedy(x).tolist()]

    def sample(self, logits: torch.Tensor, temperature: float, seed: int, position: int) -> int:
        return self.sample_rows(logits, [temperature], [seed], [position])[0]

    def token_prob(self, logits_row: torch.Tensor, token: int) -> float:
        """softmax(logits)[token] for one row; under vocabulary parallelism the maximum and the exponent sum are
        combined over ranks, so every rank returns the same number."""
        x = logits_row.float().reshape(-1)
        if self.tp is None:
            return float(torch.softmax(x, -1)[token])
        tp, Vl = self.tp, x.shape[0]
        pk = torch.full((1, tp.world), 0.0, dtype=torch.float32, device=x.device)
        pk[0, tp.rank] = x.max()
        mx = tp.allreduce(pk).max()                      # column r has one contributor (rank r): the sum gathers the maxima
        own = tp.rank * Vl <= token < (tp.rank + 1) * Vl
        pk2 = torch.zeros(1, 2, dtype=torch.float32, device=x.device)
        pk2[0, 0] = torch.exp(x - mx).sum()
        if own:
            pk2[0, 1] = torch.exp(x[token - tp.rank * Vl] - mx)
        out = tp.allreduce(pk2)
        return float(out[0, 1] / out[0, 0])

    def commit(self, accepted: List[List[int]]):
        """accepted[i]: segment-local rows of segment i that become part of the sequence, a path
        from the segment's first row (always accepted: it is the last sampled token)."""
        plan = self._pending_plan
        assert plan is not None, "commit() without a pending verify"
        for _, mix, _ in self.layers:
            mix.commit(accepted)
            if plan.is_tree and hasattr(mix, "compact"):
                for s, rows in zip(plan.segs, accepted):
                    mix.compact(self.seqs, s, rows)
        for s, rows in zip(plan.segs, accepted):
            self.seqs[s.slot].length = s.pos0 + len(rows)
        self._pending_plan = None

    # -- MTP drafter ------------------------------------------------------------------------
    @torch.no_grad()
    def sparse_ctx_limit(self) -> Optional[int]:
        """Context length up to which every sparse-attention layer still selects all of it (block-sparse GQA: top-k blocks x
        block; latent attention: top-k pools x pool), or None when no layer selects.  Up to here dense visibility of the
        committed context (what tree-verification rows use) equals what a decode row sees."""
        lim = None
        for _, mix, _ in self.layers:
            c = getattr(mix, "c", None)
            if isinstance(mix, AttnMixer) and c.sparse_topk_blocks:
                v = c.sparse_topk_blocks * c.block
            elif isinstance(mix, MlaMixer):
                v = c.topk_pools * c.pool
            else:
                continue
            lim = v if lim is None else min(lim, v)
        return lim

    def mtp_forward(self, plan: Plan, hidden: torch.Tensor):
        """Draft logits: row i combines embed(plan.ids[i]) (the NEXT token) with `hidden[i]` (target
        hidden of the previous position).  plan positions index the drafter's own KV cache.  Blocks run like the
        target's: the residual stream stays fp32 on the device and every residual update is one fused
        (all-reduce +) add + RMSNorm."""
        cfg, M, tp = self.cfg, self.W["mtp"], self.tp
        ids = plan.ids
        if plan.has_media:                       # salted media placeholders of a prompt: the drafter sees token 0 there
            ids = torch.where(ids >= cfg.vocab, torch.zeros_like(ids), ids)
        e = ops.rmsnorm(ops.embed(self.W["embed"], ids, self.dtype), M["norm_e"], cfg.norm_eps)
        hh = ops.rmsnorm(hidden if hidden.is_cuda else hidden.to(self.dtype), M["norm_h"], cfg.norm_eps)
        X = ops.linear(torch.cat((e, hh), -1), M["fc"])
        if X.is_cuda:
            X = X.float()
        deferred = plan.rows <= 16 and X.is_cuda and (tp is None or hasattr(tp, "argmax"))
        pend = None
        for lw, mix, mlp in self.mtp_layers:
            h, X = ops.add_rmsnorm(pend, X, lw["in_norm"], cfg.norm_eps, tp)
            a = mix.forward(h, plan, self.mtp_seqs(), True)
            h, X = ops.add_rmsnorm(a, X, lw["post_norm"], cfg.norm_eps, tp)
            pend = mlp.forward(h, defer=deferred)
        hn, X = ops.add_rmsnorm(pend, X, M["final_norm"], cfg.norm_eps, tp)
        if tp is not None and getattr(tp, "rows_sharded", False):
            X = tp.gather_rows(X)
        self.mtp_hidden = X
        if plan.logit_rows.shape[0] != hn.shape[0] or getattr(plan, "gather_logit_rows", False):
            hn = hn[plan.logit_rows]
        return ops.lm_head(hn, self.W["lm_head"])

    def mtp_seqs(self):
        return self.seqs

    # -- state snapshot (prefix checkpoints) ----------------------------------------------
    def snapshot(self, slot: int) -> dict:
        """Copy of everything that defines the sequence in `slot` up to its committed length
        (reference: spec_probe.rs:1420-1444 ckpt_save/restore/clone)."""
        si = self.seqs[slot]
        snap = {"length": si.length, "layers": []}
        for _, mix, _ in self.layers + self.mtp_layers:
            d = {}
            for name, t in mix.state_tensors().items():
                if name in ("S", "tail"):
                    d[name] = t[slot].clone()
                elif name in ("ik_pool", "pool"):
                    blk = self.cfg.attn.block if name == "ik_pool" else self.cfg.mla.pool
                    d[name] = t[si.kv_base // blk: si.kv_base // blk + si.length // blk + 1].clone()
                else:
                    d[name] = t[si.kv_base: si.kv_base + si.length].clone()
            snap["layers"].append(d)
        return snap

    def restore(self, slot: int, snap: dict):
        si = self.seqs[slot]
        n = snap["length"]
        assert n <= si.kv_cap, "sequence capacity exceeded"
        for (_, mix, _), d in zip(self.layers + self.mtp_layers, snap["layers"]):
            for name, t in mix.state_tensors().items():
                if name in ("S", "tail"):
                    t[slot] = d[name]
                elif name in ("ik_pool", "pool"):
                    blk = self.cfg.attn.block if name == "ik_pool" else self.cfg.mla.pool
                    t[si.kv_base // blk: si.kv_base // blk + d[name].shape[0]] = d[name]
                else:
                    t[si.kv_base: si.kv_base + n] = d[name]
        si.length = n
