"""Tensor / expert parallelism of the model across the GPUs of one box.

Shard rules (reference: engine-rs/src/weights.rs:119-153,831-864, docs/features.md:59-66):
  * linear-attention and softmax-attention mixers are split by heads (q/k/v/z projections column-parallel,
    the output projection row-parallel); KV heads are replicated when there are fewer of them than ranks;
  * routed experts are split by expert id (each rank owns E/world experts; activations are replicated, so no
    dispatch is needed on this path: a rank computes the pairs of its own experts and the partial outputs
    are summed by the same all-reduce as a row-parallel layer); the shared expert lives on rank 0;
  * lm_head is vocabulary-parallel: each rank scores V/world rows and only (value, index) packets travel
    (reference: head_select.rs:42-67); embeddings, norms, routers, conv taps and gates are replicated.
Two all-reduces per layer remain (after the mixer's output projection and after the MoE); on the device each
is fused with the residual add and the following RMSNorm, and for EXL3 decode rows also with the GEMV.
"""
from __future__ import annotations

import os

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from ..config import ModelConfig
from .. import ops


def local_config(cfg: ModelConfig, world: int) -> ModelConfig:
    c = dataclasses.replace(cfg)
    g = cfg.gdn
    assert g.n_k_heads % world == 0 and g.n_v_heads % world == 0 or "gdn" not in cfg.layer_types
    c.gdn = dataclasses.replace(g, n_k_heads=max(1, g.n_k_heads // world), n_v_heads=max(1, g.n_v_heads // world))
    a = cfg.attn
    assert a.n_q_heads % world == 0 or "attn" not in cfg.layer_types
    c.attn = dataclasses.replace(a, n_q_heads=max(1, a.n_q_heads // world), n_kv_heads=max(1, a.n_kv_heads // world))
    k = cfg.kda
    c.kda = dataclasses.replace(k, n_heads=max(1, k.n_heads // world))
    m = cfg.mla
    c.mla = dataclasses.replace(m, n_heads=max(1, m.n_heads // world))
    return c


def shard_weights(W: dict, cfg: ModelConfig, rank: int, world: int) -> dict:
    """This rank's shard of a full weight dict (dense tensors or packed EXL3 / MXFP4 / MXFP8 / FP8-block weights, cut
    without decoding: quant/formats.py `take_out` / `take_in` / `take_experts`).  A shared expert that lives in the
    expert stacks stays on every rank (decode serves row r's shared pair on rank r % world); a separate shared expert
    stays on rank 0.  Reference: engine-rs/src/weights.rs:119-153,831-864, ds41/cfg.rs:86-113."""
    from ..quant.formats import Exl3Weight, take_experts, take_in, take_out
    ar = torch.arange
    out = {k: v for k, v in W.items() if k not in ("lm_head", "layers", "mtp")}      # replicated tensors and tables
    V = cfg.vocab
    assert V % world == 0
    out["lm_head"] = take_out(W["lm_head"], ar(rank * V // world, (rank + 1) * V // world))

    def layer(lw):
        kind, w = lw["type"], lw["mix"]
        nl = {"type": kind, "in_norm": lw["in_norm"], "post_norm": lw["post_norm"]}
        if kind == "gdn":
            c = cfg.gdn
            D, hk, hv = c.head_dim, c.n_k_heads // world, c.n_v_heads // world
            nq, nv = c.n_k_heads * D, c.n_v_heads * D
            q0, v0 = rank * hk * D, rank * hv * D
            sel = torch.cat((ar(q0, q0 + hk * D), nq + ar(q0, q0 + hk * D), 2 * nq + ar(v0, v0 + hv * D)))
            zsel = 2 * nq + nv + ar(v0, v0 + hv * D)
            hsel = ar(rank * hv, (rank + 1) * hv)
            nl["mix"] = {"in": take_out(w["in"], torch.cat((sel, zsel))),
                         "ab": w["ab"][torch.cat((hsel, c.n_v_heads + hsel)).to(w["ab"].device)].contiguous(),
                         "conv": w["conv"][sel.to(w["conv"].device)].contiguous(),
                         "A_log": w["A_log"][hsel.to(w["A_log"].device)].contiguous(),
                         "dt_bias": w["dt_bias"][hsel.to(w["dt_bias"].device)].contiguous(), "norm": w["norm"],
                         "o": take_in(w["o"], v0, v0 + hv * D)}
        elif kind == "attn":
            c = cfg.attn
            D = c.head_dim
            qw = D * (2 if c.gated else 1)
            hq = c.n_q_heads // world
            nq, nkv = c.n_q_heads * qw, c.n_kv_heads * D
            if c.n_kv_heads >= world:
                hkv = c.n_kv_heads // world
                kv0 = rank * hkv
            else:
                hkv, kv0 = 1, rank * c.n_kv_heads // world
            sel = torch.cat((ar(rank * hq * qw, (rank + 1) * hq * qw), nq + ar(kv0 * D, (kv0 + hkv) * D),
                             nq + nkv + ar(kv0 * D, (kv0 + hkv) * D), ar(nq + 2 * nkv, w["qkv"].shape[0])))
            nl["mix"] = dict(w)
            nl["mix"]["qkv"] = take_out(w["qkv"], sel)
            nl["mix"]["o"] = take_in(w["o"], rank * hq * D, (rank + 1) * hq * D)
        elif kind == "kda":
            c = cfg.kda
            D, hh = c.head_dim, c.n_heads // world
            n, r = c.n_heads * D, c.gate_rank
            ch = ar(rank * hh * D, (rank + 1) * hh * D)                  # this rank's channels inside q, k or v
            sel = torch.cat((ch, n + ch, 2 * n + ch))
            hsel = ar(rank * hh, (rank + 1) * hh)
            dv = w["conv"].device
            nl["mix"] = {"in": take_out(w["in"], sel), "conv": w["conv"][sel.to(dv)].contiguous(),
                         "lr_a": torch.cat((w["lr_a"][: 2 * r], w["lr_a"][(2 * r + hsel).to(w["lr_a"].device)])).contiguous(),
                         "f_b": w["f_b"][ch.to(dv)].contiguous(), "g_b": w["g_b"][ch.to(dv)].contiguous(),
                         "A_log": w["A_log"][hsel.to(dv)].contiguous(), "dt_bias": w["dt_bias"][ch.to(dv)].contiguous(),
                         "o_norm": w["o_norm"], "o": take_in(w["o"], int(ch[0]), int(ch[-1]) + 1)}
        elif kind == "mla":
            c = cfg.mla
            hh = c.n_heads // world
            qw = c.head_dim + c.rope_dim
            nq = c.n_heads * qw
            nl["mix"] = dict(w)                                              # low-rank projections, norms, indexer: replicated
            nl["mix"]["q_b"] = torch.cat((w["q_b"][rank * hh * qw: (rank + 1) * hh * qw], w["q_b"][nq:])).contiguous()
            nl["mix"]["kv_b"] = w["kv_b"][rank * hh * 2 * c.head_dim: (rank + 1) * hh * 2 * c.head_dim].contiguous()
            nl["mix"]["o"] = take_in(w["o"], rank * hh * c.head_dim, (rank + 1) * hh * c.head_dim)
            if "sink" in w:
                nl["mix"]["sink"] = w["sink"][rank * hh: (rank + 1) * hh].contiguous()
        else:
            raise NotImplementedError(f"tensor-parallel shard rule for layer type {kind}")
        for extra in lw:                                                     # n-gram gates etc.: replicated
            if extra not in ("type", "in_norm", "post_norm", "mix", "mlp"):
                nl[extra] = lw[extra]
        m = lw["mlp"]
        if "dense_gu" in m:
            F = cfg.moe.dense_ffn
            f0, f1 = rank * F // world, (rank + 1) * F // world
            nl["mlp"] = {"dense_gu": take_out(m["dense_gu"], torch.cat((ar(f0, f1), F + ar(f0, f1)))),
                         "dense_down": take_in(m["dense_down"], f0, f1)}
        else:
            E = cfg.moe.n_experts
            e0, e1 = rank * E // world, (rank + 1) * E // world
            nm = {"gate": m["gate"], "ep": (e0, e1), "tp_rank": (rank, world)}
            if m.get("shared_in_stack"):
                # stack = E routed experts + the shared expert at index E: keep [e0, e1) and the shared one
                def cut(w):
                    a, b = take_experts(w, e0, e1), take_experts(w, E, E + 1)
                    return Exl3Weight(torch.cat((a.trellis, b.trellis)), torch.cat((a.suh, b.suh)), torch.cat((a.svh, b.svh)),
                                      a.bits, a.kind)
                nm["w_gu"], nm["w_down"] = cut(m["w_gu"]), cut(m["w_down"])
                nm["shared_in_stack"] = True
                e_loc = e1 - e0
                for name, st in (("s_gu", nm["w_gu"]), ("s_down", nm["w_down"])):
                    nm[name] = Exl3Weight(st.trellis[e_loc], st.suh[e_loc], st.svh[e_loc], st.bits, st.kind)
            else:
                nm["w_gu"], nm["w_down"] = take_experts(m["w_gu"], e0, e1), take_experts(m["w_down"], e0, e1)
                if "s_gu" in m and rank == 0:
                    nm["s_gu"], nm["s_down"] = m["s_gu"], m["s_down"]
            if "bias" in m:
                nm["bias"] = m["bias"]
            nl["mlp"] = nm
        return nl

    out["layers"] = [layer(lw) for lw in W["layers"]]
    if "mtp" in W:
        out["mtp"] = dict(W["mtp"])
        out["mtp"]["layers"] = [layer(lw) for lw in W["mtp"]["layers"]]
    return out


shard_dense_weights = shard_weights      # older name: the same rules served dense tensors only


class TPBase:
    def __init__(self, rank: int, world: int):
        self.rank, self.world = rank, world

    def local_config(self, cfg: ModelConfig) -> ModelConfig:
        return local_config(cfg, self.world)

    def can_fuse_gemv(self, x, w) -> bool:
        return False

    def reduce(self, delta) -> torch.Tensor:
        """All-reduced rows of a block output that is still this rank's partial sum (tensor, deferred product or
        uncombined expert outputs)."""
        return self.allreduce(ops.to_tensor(delta).float())

    def greedy(self, logits_local: torch.Tensor, vocab_local: int) -> torch.Tensor:
        """Global arg-max from vocabulary-parallel logits: (value, index) packets, ties -> lowest id."""
        val, idx = logits_local.max(-1)
        pk = torch.zeros(logits_local.shape[0], 2 * self.world, dtype=torch.float32, device=logits_local.device)
        pk[:, 2 * self.rank] = val.float()
        pk[:, 2 * self.rank + 1] = (idx + self.rank * vocab_local).float()
        pk = self.allreduce(pk)
        vals, ids = pk[:, 0::2], pk[:, 1::2]
        best = vals.max(-1, keepdim=True).values
        cand = torch.where(vals == best, ids, torch.full_like(ids, float("inf")))
        return cand.min(-1).values.to(torch.int32)


class CpuTP(TPBase):
    """gloo ranks on CPU: the host-side logic of the sharded model without a GPU."""

    def __init__(self, group=None):
        super().__init__(dist.get_rank(group), dist.get_world_size(group))
        self.group = group

    def allreduce(self, x):
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        acc = torch.zeros_like(x, dtype=torch.float32)
        for p in parts:                      # rank order, like the device kernels
            acc = acc + p.float()
        return acc.to(x.dtype)

    def add_rmsnorm(self, delta, res, w, eps):
        if isinstance(delta, ops.Partial):
            delta = ops.linear(delta.x, delta.w)
        res = res + self.allreduce(delta.float()).to(res.dtype)
        from ..oracle import layers as L
        return L.rms(res.float(), w.float(), eps).to(res.dtype), res


class NcclTP(TPBase):
    """Library baseline on the device: NCCL all-reduce through torch.distributed + ATen ops for the residual add
    and the norm (what a plain PyTorch tensor-parallel implementation does); used by `bench.py --impl aten`."""

    def __init__(self, group=None):
        super().__init__(dist.get_rank(group), dist.get_world_size(group))
        self.group = group

    def allreduce(self, x):
        y = x.float().contiguous()
        dist.all_reduce(y, group=self.group)
        return y.to(x.dtype)

    def add_rmsnorm(self, delta, res, w, eps):
        if isinstance(delta, ops.Partial):
            delta = ops.linear(delta.x, delta.w)
        res = res + self.allreduce(ops.to_tensor(delta).float()).to(res.dtype)
        from ..oracle import layers as L
        return L.rms(res.float(), w.float(), eps).to(torch.bfloat16), res


class DeviceTP(TPBase):
    """Peer-memory tensor parallelism on the GPUs of one box (fused all-reduce kernels)."""

    def __init__(self, arena, hidden: int, rows_cap: int = 1024, name: str = "tp"):
        super().__init__(arena.rank, arena.world)
        from . import symm
        self.arena = arena
        self.rows_cap = rows_cap
        self.ar = symm.FusedAllReduce(arena, name + ".ar", rows_cap, hidden)
        self.pk = symm.FusedAllReduce(arena, name + ".packets", 64, 2 * 8)
        self.argmax = symm.PacketArgmax(arena, name + ".argmax", 64)
        # sequence-parallel prefill: the residual stream of a large chunk lives row-sharded (each rank owns a block of
        # rows); a block output is reduce-scattered to the owners, who add it to their rows, normalise them and
        # all-gather the bf16 result.  Against the all-reduce of full rows this moves (W - 1) / W of one fp32 copy plus
        # one bf16 copy instead of (W - 1) fp32 copies per rank, and the norm runs once per row instead of W times.
        # Reference: engine-rs/src/forward.rs:578-871 (sequence-parallel prefill), shim/mhc.cu:128-181.
        self.sp_min_rows = int(os.environ.get("SPARK_SP_MIN_ROWS", "128"))
        self.rp = symm.RowParallelGemm(arena, name + ".sp", rows_cap, hidden) if hidden <= 4096 and hidden % 4 == 0 else None
        self.rows_sharded = False            # True while the residual of the forward in flight is valid on owned rows only

    def greedy(self, logits_local: torch.Tensor, vocab_local: int) -> torch.Tensor:
        if logits_local.shape[0] <= 64:
            return self.argmax(logits_local.float(), self.rank * vocab_local)
        return super().greedy(logits_local, vocab_local)

    def can_fuse_gemv(self, x, w) -> bool:
        from ..quant.formats import Exl3Weight
        return isinstance(w, Exl3Weight) and not w.experts and w.bits == 4 and x.shape[0] <= 16 and x.is_cuda

    def reduce(self, delta) -> torch.Tensor:
        if isinstance(delta, ops.Partial):
            if self.can_fuse_gemv(delta.x, delta.w):
                return self.ar.gemv_fused(delta.x.contiguous(), delta.w, out_dtype=torch.float32)
            delta = ops.linear(delta.x, delta.w)
        if isinstance(delta, torch.Tensor) and delta.shape[0] > self.rows_cap:
            return torch.cat([self.ar(delta[r0: r0 + self.rows_cap], out_dtype=torch.float32)
                              for r0 in range(0, delta.shape[0], self.rows_cap)])
        return self.ar(delta, out_dtype=torch.float32)

    def allreduce(self, x):
        assert x.shape[0] <= 64 and x.shape[1] <= 16
        pad = torch.zeros(x.shape[0], 16, dtype=torch.float32, device=x.device)
        pad[:, : x.shape[1]] = x
        return self.pk(pad, out_dtype=torch.float32)[:, : x.shape[1]]

    def _sp(self, R: int) -> bool:
        return (self.rp is not None and self.sp_min_rows <= R <= self.rows_cap and R % self.world == 0
                and self.sp_min_rows > 0)

    def _sp_rows(self, part, res, w, eps):
        rpr = part.shape[0] // self.world
        self.rows_sharded = True
        return self.rp.rows(part, res[self.rank * rpr: (self.rank + 1) * rpr], w, eps)

    def gather_rows(self, X: torch.Tensor) -> torch.Tensor:
        """Make a row-sharded residual whole again (every rank contributes its owned block)."""
        if not self.rows_sharded:
            return X
        self.rows_sharded = False
        rpr = X.shape[0] // self.world
        out = torch.empty_like(X)
        dist.all_gather_into_tensor(out, X[self.rank * rpr: (self.rank + 1) * rpr].contiguous())
        return out

    def add_rmsnorm(self, delta, res, w, eps):
        if isinstance(delta, ops.Partial):
            if self._sp(delta.x.shape[0]):
                return self._sp_rows(ops.linear(delta.x, delta.w), res, w, eps), res
            h = self.ar.gemv_fused(delta.x.contiguous(), delta.w, res=res, norm_w=w, eps=eps)
            return h, res
        if not isinstance(delta, torch.Tensor):          # uncombined MoE of a decode round: combined inside the push
            return self.ar(delta, res=res, norm_w=w, eps=eps), res
        R = delta.shape[0]
        if self._sp(R):
            return self._sp_rows(delta, res, w, eps), res
        if R <= self.rows_cap:
            return self.ar(delta, res=res, norm_w=w, eps=eps), res
        outs = []
        for r0 in range(0, R, self.rows_cap):
            outs.append(self.ar(delta[r0: r0 + self.rows_cap], res=res[r0: r0 + self.rows_cap], norm_w=w, eps=eps))
        return torch.cat(outs), res
