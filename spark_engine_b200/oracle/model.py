"""Full-sequence fp32 oracle model: recomputes the whole sequence from position 0.

The engine (incremental state, chunked prefill, kernels) is tested against this.  Layer order
follows the reference's Python models: plain pre-norm residual blocks, or with 4-stream
hyper-connections `[ngram] -> HC.mix -> mixer -> X += post*a -> HC.mix -> MLP -> X += post*m`
(reference/qwen38/model.py:286-300) / mHC pre-post with Sinkhorn mixing
(reference/glm53/model.py:72-96).
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from . import layers as L


def split_gdn(w, cfg: ModelConfig):
    c = cfg.gdn
    nq, nv = c.n_k_heads * c.head_dim, c.n_v_heads * c.head_dim
    return {"qkv": w["in"][: 2 * nq + nv], "z": w["in"][2 * nq + nv:], "b": w["ab"][: c.n_v_heads],
            "a": w["ab"][c.n_v_heads:], "conv": w["conv"], "A_log": w["A_log"], "dt_bias": w["dt_bias"],
            "norm": w["norm"], "o": w["o"]}


def split_attn(w, cfg: ModelConfig):
    c = cfg.attn
    nq = c.n_q_heads * c.head_dim * (2 if c.gated else 1)
    nkv = c.n_kv_heads * c.head_dim
    d = dict(w)
    d.update({"q": w["qkv"][:nq], "k": w["qkv"][nq: nq + nkv], "v": w["qkv"][nq + nkv: nq + 2 * nkv],
              "idx": w["qkv"][nq + 2 * nkv:]})
    return d


def split_kda(w, cfg: ModelConfig):
    c = cfg.kda
    n, r = c.n_heads * c.head_dim, c.gate_rank
    d = dict(w)
    d.update({"q": w["in"][:n], "k": w["in"][n:2 * n], "v": w["in"][2 * n:],
              "q_conv": w["conv"][:n], "k_conv": w["conv"][n:2 * n], "v_conv": w["conv"][2 * n:],
              "f_a": w["lr_a"][:r], "g_a": w["lr_a"][r:2 * r], "b": w["lr_a"][2 * r:],
              "dt_bias": w["dt_bias"].view(c.n_heads, c.head_dim)})
    return d


def split_mla(w, cfg: ModelConfig):
    c = cfg.mla
    d = dict(w)
    o0 = c.q_lora
    o1 = o0 + c.kv_lora + c.rope_dim
    nq = c.n_heads * (c.head_dim + c.rope_dim)
    d.update({"q_a": w["a"][:o0], "kv_a": w["a"][o0:o1], "wk": w["a"][o1: o1 + c.idx_dim],
              "cgate": w["a"][o1 + c.idx_dim: o1 + 2 * c.idx_dim], "weights_proj": w["a"][o1 + 2 * c.idx_dim:],
              "wq_b": w["q_b"][nq:], "q_b": w["q_b"][:nq]})
    return d


def split_moe(w, cfg: ModelConfig):
    c = cfg.moe
    if "dense_gu" in w:
        F = c.dense_ffn
        return {"gate": w["dense_gu"][:F], "up": w["dense_gu"][F:], "down": w["dense_down"]}
    d = {"gate": w["gate"][: c.n_experts], "w_gate": w["w_gu"][:, : c.ffn], "w_up": w["w_gu"][:, c.ffn:],
         "w_down": w["w_down"]}
    if c.shared_gate:
        d["sg"] = w["gate"][c.n_experts:]
    if "bias" in w:
        d["bias"] = w["bias"]
    if "s_gu" in w:
        Fs = w["s_gu"].shape[0] // 2
        d.update({"s_gate": w["s_gu"][:Fs], "s_up": w["s_gu"][Fs:], "s_down": w["s_down"]})
    return d


def mixer(kind: str, cfg: ModelConfig, w: dict, h: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    if kind == "gdn":
        return L.gdn_layer(h, split_gdn(w, cfg), cfg.gdn.n_k_heads, cfg.gdn.n_v_heads, cfg.gdn.head_dim,
                           cfg.norm_eps)
    if kind == "attn":
        a = cfg.attn
        inv = L.yarn_inv_freq(a.rope_dim, a.rope_theta, a.yarn_factor, a.yarn_orig_len)
        return L.gqa_layer(h, split_attn(w, cfg), pos, a.n_q_heads, a.n_kv_heads, a.head_dim, a.rope_dim,
                           a.rope_theta, inv, a.qk_norm, a.gated, a.sparse_topk_blocks, a.block, a.idx_heads,
                           a.idx_dim, cfg.norm_eps)
    if kind == "kda":
        return L.kda_layer(h, split_kda(w, cfg), cfg.kda.n_heads, cfg.kda.head_dim)
    if kind == "mla":
        m = cfg.mla
        idx = {"heads": m.idx_heads, "dim": m.idx_dim, "pool": m.pool, "topk": m.topk_pools}
        return L.mla_layer(h, split_mla(w, cfg), pos, m.n_heads, m.head_dim, m.rope_dim, m.rope_theta,
                           cfg.norm_eps, idx, m.sink, m.window)
    raise ValueError(kind)


def mlp(cfg: ModelConfig, w: dict, h: torch.Tensor) -> torch.Tensor:
    c = cfg.moe
    m = split_moe(w, cfg)
    if "down" in m:
        return L.dense_mlp(h, m, c.swiglu_limit)
    return L.moe_layer(h, m, c.top_k, c.router, c.route_scale, c.swiglu_limit, c.shared_gate)


def block(cfg: ModelConfig, lw: dict, X: torch.Tensor, pos: torch.Tensor, ids=None, table=None):
    """One decoder block on the residual X ([T,H] plain, [T,S,H] with hyper-connections)."""
    if cfg.hc_kind == "none":
        if "ngram" in lw:
            X = L.ngram_embed(X, ids, table, lw["ngram"], cfg.ngram_heads, eps=cfg.norm_eps)
        X = X + mixer(lw["type"], cfg, lw["mix"], L.rms(X, lw["in_norm"], cfg.norm_eps), pos)
        return X + mlp(cfg, lw["mlp"], L.rms(X, lw["post_norm"], cfg.norm_eps))
    if cfg.hc_kind == "gated":
        post, h = L.hc_gated_mix(X, lw["hc_mix"], cfg.norm_eps)
        X = X + post.unsqueeze(-1) * mixer(lw["type"], cfg, lw["mix"], h, pos).unsqueeze(1)
        post, h = L.hc_gated_mix(X, lw["hc_mlp"], cfg.norm_eps)
        return X + post.unsqueeze(-1) * mlp(cfg, lw["mlp"], h).unsqueeze(1)
    if cfg.hc_kind == "mhc":
        h, post, comb = L.mhc_pre(X, lw["hc_mix"], cfg.sinkhorn_iters, cfg.norm_eps)
        X = L.mhc_post(X, mixer(lw["type"], cfg, lw["mix"], h, pos), post, comb)
        h, post, comb = L.mhc_pre(X, lw["hc_mlp"], cfg.sinkhorn_iters, cfg.norm_eps)
        return L.mhc_post(X, mlp(cfg, lw["mlp"], h), post, comb)
    raise ValueError(cfg.hc_kind)


@torch.no_grad()
def forward(cfg: ModelConfig, W: dict, ids: torch.Tensor, return_hidden: bool = False):
    """ids [T] (one sequence from position 0) -> logits [T, vocab] fp32."""
    ids = ids.long()
    T = ids.shape[0]
    pos = torch.arange(T)
    X = W["embed"][ids].float()
    if cfg.hc_kind != "none":
        X = X.unsqueeze(1).repeat(1, cfg.hc_streams, 1)
    for lw in W["layers"]:
        X = block(cfg, lw, X, pos, ids, W.get("ngram_table"))
    if cfg.hc_kind == "gated":
        _, X = L.hc_gated_mix(X, W["hc_final"], cfg.norm_eps)
        hidden = X
        logits = X @ W["lm_head"].t()
    else:
        if cfg.hc_kind == "mhc":
            X = X.mean(1)
        hidden = X
        logits = L.rms(X, W["final_norm"], cfg.norm_eps) @ W["lm_head"].t()
    return (logits, hidden) if return_hidden else logits


@torch.no_grad()
def mtp_forward(cfg: ModelConfig, W: dict, ids: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
    """MTP draft head over a full sequence: position t combines the embedding of token t+1 with the
    target's hidden state at t and predicts token t+2 (reference: qwen/spec.rs, qwen/model.rs mtp_*).
    ids [T+1], hidden [T, H] -> draft logits [T, vocab]."""
    M = W["mtp"]
    T = hidden.shape[0]
    e = L.rms(W["embed"][ids[1: T + 1].long()].float(), M["norm_e"], cfg.norm_eps)
    h = L.rms(hidden, M["norm_h"], cfg.norm_eps)
    X = torch.cat((e, h), -1) @ M["fc"].t()
    pos = torch.arange(T)
    plain = ModelConfig(**{**cfg.__dict__, "hc_kind": "none", "ngram_layers": []})
    for lw in M["layers"]:
        X = block(plain, lw, X, pos)
    return L.rms(X, M["final_norm"], cfg.norm_eps) @ W["lm_head"].t()


@torch.no_grad()
def greedy_generate(cfg: ModelConfig, W: dict, prompt: torch.Tensor, n_new: int):
    """Greedy decode by full recomputation.  Returns (token ids [n_new], logits [n_new, vocab])."""
    ids = prompt.clone().long()
    outs, lg = [], []
    for _ in range(n_new):
        logits = forward(cfg, W, ids)[-1]
        nxt = int(torch.argmax(logits))
        outs.append(nxt)
        lg.append(logits)
        ids = torch.cat((ids, torch.tensor([nxt])))
    return torch.tensor(outs), torch.stack(lg)
