"""Random-init models generated directly on the device in the serving weight formats.

Large configs (tens of billions of parameters) are never materialised in fp32: EXL3 tensors are
random trellis words + sign/scale vectors, MXFP4 random nibbles + E8M0 scales, FP8 random e4m3 +
block scales, everything else bf16 N(0, 0.02).  The formats follow the checkpoints the reference
serves (EXL3: engine-rs/src/exl3.rs, qwen/load.rs:106-217; MXFP4/FP8: ds41/load.rs:116-160,331-342).
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..quant import formats as Q


class _DevInit:
    def __init__(self, device, seed: int, fmt: str, bits: int, std: float = 0.02, rank: int = 0):
        self.device, self.fmt, self.bits, self.std, self.rank = device, fmt, bits, std, rank
        self.g = torch.Generator(device=device)          # sharded tensors: a different stream per rank
        self.g.manual_seed(seed + 7919 * rank)
        self.gc = torch.Generator(device=device)         # replicated tensors: the same on every rank
        self.gc.manual_seed(seed + 1)
        self.n = 0

    def _seed(self):
        self.n += 1
        return 1000003 * self.n + 17 + 7919 * self.rank

    def common_seeded(self) -> "_DevInit":
        """An initialiser for a replicated tensor: its seeds depend on the call count only, not on the rank."""
        c = _DevInit(self.device, 0, self.fmt, self.bits, self.std, rank=0)
        c.n = 500000 + self.n
        return c

    def mat_common(self, *shape):
        return (torch.randn(*shape, device=self.device, generator=self.gc) * self.std).to(torch.bfloat16)

    def big(self, n, k, experts=0, kind="dense"):
        """A large projection [n, k] (or experts x [n, k]) in the model's weight format."""
        fmt = self.fmt
        if fmt == "exl3" and n % 128 == 0 and k % 128 == 0:
            return Q.random_exl3(n, k, self.bits, experts, self.std, self._seed(), self.device)
        if fmt == "mx" and k % 128 == 0 and n % 128 == 0:
            if kind == "expert":
                return Q.random_mxfp4(n, k, experts, self.std, self._seed(), self.device)
            if experts == 0:        # dense projections: MXFP8 (E8M0 per 32), the block-scaled tensor-core operand format
                return Q.random_mxfp8(n, k, self.std, self._seed(), self.device)
            return Q.random_fp8_block(n, k, experts, self.std, self._seed(), self.device)
        return self.mat(*(((experts,) if experts else ()) + (n, k)))

    def mat(self, *shape):
        return (torch.randn(*shape, device=self.device, generator=self.g) * self.std).to(torch.bfloat16)

    def f32(self, *shape, lo=None, hi=None, val=None):
        if val is not None:
            return torch.full(shape, val, device=self.device, dtype=torch.float32)
        if lo is not None:
            return torch.rand(*shape, device=self.device, generator=self.g) * (hi - lo) + lo
        return torch.randn(*shape, device=self.device, generator=self.g) * self.std


def _mix(cfg: ModelConfig, it: _DevInit, kind: str) -> dict:
    H = cfg.hidden
    if kind == "gdn":
        c = cfg.gdn
        nq, nv = c.n_k_heads * c.head_dim, c.n_v_heads * c.head_dim
        return {"in": it.big(2 * nq + 2 * nv, H), "ab": it.mat(2 * c.n_v_heads, H),
                "conv": it.f32(2 * nq + nv, c.conv_k, lo=-0.5, hi=0.5),
                "A_log": torch.log(it.f32(c.n_v_heads, lo=1.0, hi=8.0)), "dt_bias": it.f32(c.n_v_heads, lo=-1.0, hi=1.0),
                "norm": it.f32(c.head_dim, val=1.0), "o": it.big(H, nv)}
    if kind == "attn":
        c = cfg.attn
        nq = c.n_q_heads * c.head_dim * (2 if c.gated else 1)
        nkv = c.n_kv_heads * c.head_dim
        nidx = (c.idx_heads + 1) * c.idx_dim if c.sparse_topk_blocks else 0
        w = {"qkv": it.big(nq + 2 * nkv + nidx, H), "o": it.big(H, c.n_q_heads * c.head_dim)}
        if c.qk_norm:
            w["q_norm"], w["k_norm"] = it.f32(c.head_dim), it.f32(c.head_dim)
        if c.sparse_topk_blocks:
            w["iq_norm"], w["ik_norm"] = it.f32(c.idx_dim), it.f32(c.idx_dim)
        return w
    if kind == "kda":
        c = cfg.kda
        n, r = c.n_heads * c.head_dim, c.gate_rank
        return {"in": it.big(3 * n, H), "conv": it.f32(3 * n, c.conv_k, lo=-0.5, hi=0.5),
                "lr_a": it.mat(2 * r + c.n_heads, H), "f_b": it.f32(n, r) * 10, "g_b": it.f32(n, r) * 10,
                "A_log": torch.log(it.f32(c.n_heads, lo=1.0, hi=4.0)), "dt_bias": it.f32(n, lo=-1.0, hi=1.0),
                "o_norm": it.f32(c.head_dim, val=1.0), "o": it.big(H, n)}
    if kind == "mla":
        c = cfg.mla
        idx_rows = 2 * c.idx_dim + c.idx_heads
        w = {"a": it.mat(c.q_lora + c.kv_lora + c.rope_dim + idx_rows, H),
             "q_a_norm": it.f32(c.q_lora, val=1.0), "kv_a_norm": it.f32(c.kv_lora, val=1.0),
             "q_b": it.mat(c.n_heads * (c.head_dim + c.rope_dim) + c.idx_heads * c.idx_dim, c.q_lora),
             "kv_b": it.mat(c.n_heads * 2 * c.head_dim, c.kv_lora),
             "k_ln_w": it.f32(c.idx_dim, val=1.0), "k_ln_b": it.f32(c.idx_dim, val=0.0),
             "ape": it.f32(c.pool, c.idx_dim), "o": it.big(H, c.n_heads * c.head_dim)}
        if c.sink:
            w["sink"] = it.f32(c.n_heads) * 10
        return w
    raise ValueError(kind)


def _mlp(cfg: ModelConfig, it: _DevInit, dense: bool, tp=(0, 1)) -> dict:
    c, H = cfg.moe, cfg.hidden
    rank, world = tp
    if dense:
        Fd = c.dense_ffn // world            # dense MLPs are split by the intermediate dimension
        return {"dense_gu": it.big(2 * Fd, H), "dense_down": it.big(H, Fd)}
    Fs = c.shared_ffn or c.ffn * c.n_shared
    assert c.n_experts % world == 0
    e_loc = c.n_experts // world
    # EXL3 models keep a shared expert of the routed experts' width as one more matrix of the expert stacks (index
    # e_loc): decode treats it as one more (row, expert) pair of the grouped GEMVs, and under tensor parallelism every
    # rank holds it and serves the rows r with r % world == rank.
    stack_shared = bool(c.n_shared) and Fs == c.ffn and it.fmt == "exl3" and H % 128 == 0 and c.ffn % 128 == 0
    n_stack = e_loc + (1 if stack_shared else 0)
    w = {"gate": it.mat_common(c.n_experts + (1 if c.shared_gate else 0), H), "tp_rank": (rank, world)}
    if stack_shared:
        it_s = it.common_seeded()            # the shared expert is replicated: same bits on every rank
        gu_r, dn_r = it.big(2 * c.ffn, H, e_loc, kind="expert"), it.big(H, c.ffn, e_loc, kind="expert")
        gu_s, dn_s = it_s.big(2 * c.ffn, H, 1, kind="expert"), it_s.big(H, c.ffn, 1, kind="expert")
        w["w_gu"] = Q.Exl3Weight(torch.cat((gu_r.trellis, gu_s.trellis)), torch.cat((gu_r.suh, gu_s.suh)),
                                 torch.cat((gu_r.svh, gu_s.svh)), gu_r.bits, gu_r.kind)
        w["w_down"] = Q.Exl3Weight(torch.cat((dn_r.trellis, dn_s.trellis)), torch.cat((dn_r.suh, dn_s.suh)),
                                   torch.cat((dn_r.svh, dn_s.svh)), dn_r.bits, dn_r.kind)
        w["shared_in_stack"] = True
        for name, st in (("s_gu", w["w_gu"]), ("s_down", w["w_down"])):      # views for prefill-size batches
            w[name] = Q.Exl3Weight(st.trellis[e_loc], st.suh[e_loc], st.svh[e_loc], st.bits, st.kind)
    else:
        w["w_gu"] = it.big(2 * c.ffn, H, e_loc, kind="expert")
        w["w_down"] = it.big(H, c.ffn, e_loc, kind="expert")
    if world > 1:
        w["ep"] = (rank * e_loc, (rank + 1) * e_loc)
    if c.router != "softmax":
        w["bias"] = torch.zeros(c.n_experts, device=it.device)
    if c.n_shared and not stack_shared and rank == 0:
        w["s_gu"], w["s_down"] = it.big(2 * Fs, H), it.big(H, Fs)
    return w


def _hc(cfg: ModelConfig, it: _DevInit, inject: bool = True) -> dict:
    """Hyper-connection site weights (replicated on every rank: they act on the full hidden width)."""
    S, H, r = cfg.hc_streams, cfg.hidden, cfg.hc_rank
    if cfg.hc_kind == "gated":
        w = {"norm": it.mat_common(S, H).float(), "down": it.mat_common(r, S * H), "up": it.mat_common(S * H, r)}
        if inject:
            w["inject"] = it.mat_common(S, S * H)
        return w
    n = 2 * S + S * S
    return {"fn": it.mat_common(n, S * H), "scale": torch.rand(3, device=it.device, generator=it.gc) + 0.5,
            "base": it.mat_common(n).float(), "norm": it.f32(H, val=1.0)}


def _layer(cfg: ModelConfig, lcfg: ModelConfig, it: _DevInit, i: int, kind: str, tp=(0, 1)) -> dict:
    w = {"type": kind, "in_norm": it.f32(cfg.hidden, val=1.0), "post_norm": it.f32(cfg.hidden, val=1.0),
         "mix": _mix(lcfg, it, kind), "mlp": _mlp(cfg, it, i < cfg.moe.dense_layers, tp)}
    if cfg.hc_kind != "none":
        w["hc_mix"], w["hc_mlp"] = _hc(cfg, it), _hc(cfg, it)
    return w


def build_random_model(cfg: ModelConfig, device="cuda", seed: int = 0, tp=(0, 1)) -> dict:
    """Nested weight dict on `device` in cfg.weight_format (dense | exl3 | mx).  `tp` = (rank, world): only this
    rank's shard is generated (heads, experts by id, vocabulary rows of lm_head); replicated tensors come from a
    generator that is seeded identically on every rank."""
    rank, world = tp
    from ..parallel.tp import local_config
    lcfg = local_config(cfg, world) if world > 1 else cfg
    it = _DevInit(device, seed, cfg.weight_format, cfg.exl3_bits, rank=rank)
    W = {"embed": it.mat_common(cfg.vocab, cfg.hidden), "final_norm": it.f32(cfg.hidden, val=1.0),
         "lm_head": it.mat(cfg.vocab // world, cfg.hidden),
         "layers": [_layer(cfg, lcfg, it, i, cfg.layer_types[i], tp) for i in range(cfg.n_layers)]}
    if cfg.mtp_layers:
        kind = "attn" if cfg.family == "hybrid" else "mla"
        W["mtp"] = {"fc": it.mat_common(cfg.hidden, 2 * cfg.hidden), "norm_e": it.f32(cfg.hidden, val=1.0),
                    "norm_h": it.f32(cfg.hidden, val=1.0), "final_norm": it.f32(cfg.hidden, val=1.0),
                    "layers": [_layer(cfg, lcfg, it, cfg.n_layers, kind, tp) for _ in range(cfg.mtp_layers)]}
    if cfg.hc_kind == "gated":
        W["hc_final"] = _hc(cfg, it, inject=False)
    if cfg.ngram_layers:
        W["ngram_table"] = it.mat_common(cfg.ngram_rows, cfg.ngram_dim)
        D = cfg.ngram_dim * cfg.ngram_heads
        for i in (j for j in cfg.ngram_layers if j < cfg.n_layers):
            W["layers"][i]["ngram"] = {"key": it.mat_common(cfg.hidden, D), "value": it.mat_common(cfg.hidden, D),
                                       "norm_k": it.f32(cfg.hidden, val=1.0), "norm_q": it.f32(cfg.hidden, val=1.0)}
    return W


def weight_bytes(W) -> int:
    n = 0

    def rec(x):
        nonlocal n
        if isinstance(x, dict):
            for v in x.values():
                rec(v)
        elif isinstance(x, list):
            for v in x:
                rec(v)
        elif isinstance(x, Q.QuantWeight):
            n += x.nbytes()
        elif isinstance(x, torch.Tensor):
            n += x.numel() * x.element_size()
    rec(W)
    return n


def decode_step_bytes(W, cfg: ModelConfig, rows: int) -> int:
    """Weight bytes one decode round of `rows` rows has to read from memory: every dense / attention projection,
    router, norm and lm_head once, and per MoE layer the matrices of the (row, expert) pairs (rows x top-k distinct
    experts at most, plus the shared expert).  KV / state traffic is not included."""
    def nbytes(x):
        if isinstance(x, Q.QuantWeight):
            return x.nbytes()
        if isinstance(x, torch.Tensor):
            return x.numel() * x.element_size()
        if isinstance(x, dict):
            return sum(nbytes(v) for v in x.values())
        return 0
    total = nbytes(W["lm_head"]) + nbytes(W["final_norm"]) + rows * cfg.hidden * 2
    for lw in W["layers"]:
        total += nbytes(lw["mix"]) + nbytes(lw["in_norm"]) + nbytes(lw["post_norm"])
        m = lw["mlp"]
        if "dense_gu" in m:
            total += nbytes(m)
            continue
        total += nbytes(m["gate"])
        wg = m["w_gu"]
        if isinstance(wg, Q.Exl3Weight):
            stack = wg.trellis.shape[0]
        elif isinstance(wg, torch.Tensor):
            stack = wg.shape[0]
        else:
            stack = wg.packed.shape[0] if hasattr(wg, "packed") else cfg.moe.n_experts
        per_expert = (nbytes(m["w_gu"]) + nbytes(m["w_down"])) / max(stack, 1)
        world = m.get("tp_rank", (0, 1))[1]
        pairs = min(rows * cfg.moe.top_k, cfg.moe.n_experts) / world       # this rank's share on average
        total += int(per_expert * pairs)
        if m.get("shared_in_stack"):
            total += int(per_expert * min(1.0, rows / world))
        elif "s_gu" in m:
            total += nbytes(m["s_gu"]) + nbytes(m["s_down"])
    return int(total)
