"""Weight layout and random initialisation for every model family.

Weights live in a nested dict.  Projections that share an input are stored fused, in the layout
the kernels consume (one GEMV/GEMM per fused matrix):

  gdn : in  = [q | k | v | z] rows,  ab = [b | a] rows (small, kept dense), conv [C,k], o
  attn: qkv = [q(+gate per head) | k | v | indexer q | indexer k] rows, o
  kda : in  = [q | k | v] rows, lr_a = [f_a | g_a | b] rows (dense), f_b, g_b, o
  mla : a   = [q_a | kv_a(+rope key) | indexer wk | cgate | weights_proj] rows, q_b(+wq_b), kv_b, o
  moe : gate [E(+1 shared-gate row), H], w_gu [E, 2F, H] (gate rows then up rows), w_down [E,H,F],
        s_gu [2Fs, H], s_down [H, Fs]

All matrices are `[out, in]`.  There is no checkpoint on the build machines, so every format is
generated: dense N(0, 0.02); EXL3 = random trellis bits + random sign/scale vectors (any bitstream
decodes to valid weights); MXFP4 = random E2M1 nibbles + E8M0 scales; FP8 = random e4m3 + block
scales.  (Reference loaders: engine-rs/src/weights.rs:627-818, qwen/load.rs:106-217,
ds41/load.rs:116-160.)
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from ..config import ModelConfig


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


class _Init:
    def __init__(self, seed: int, std: float = 0.02):
        self.g = _gen(seed)
        self.std = std

    def mat(self, *shape) -> torch.Tensor:
        return torch.randn(*shape, generator=self.g) * self.std

    def ones(self, n) -> torch.Tensor:
        return torch.ones(n)

    def zeros(self, *shape) -> torch.Tensor:
        return torch.zeros(*shape)

    def uniform(self, lo, hi, *shape) -> torch.Tensor:
        return torch.rand(*shape, generator=self.g) * (hi - lo) + lo


def gdn_weights(cfg: ModelConfig, it: _Init) -> Dict[str, torch.Tensor]:
    c, H = cfg.gdn, cfg.hidden
    nq = c.n_k_heads * c.head_dim
    nv = c.n_v_heads * c.head_dim
    return {
        "in": it.mat(2 * nq + 2 * nv, H),            # q | k | v | z
        "ab": it.mat(2 * c.n_v_heads, H),            # b | a
        "conv": it.uniform(-0.5, 0.5, 2 * nq + nv, c.conv_k),
        "A_log": torch.log(it.uniform(1.0, 8.0, c.n_v_heads)),
        "dt_bias": it.uniform(-1.0, 1.0, c.n_v_heads),
        "norm": it.ones(c.head_dim),
        "o": it.mat(H, nv),
    }


def attn_weights(cfg: ModelConfig, it: _Init) -> Dict[str, torch.Tensor]:
    c, H = cfg.attn, cfg.hidden
    nq = c.n_q_heads * c.head_dim * (2 if c.gated else 1)
    nkv = c.n_kv_heads * c.head_dim
    nidx = (c.idx_heads + 1) * c.idx_dim if c.sparse_topk_blocks else 0
    w = {"qkv": it.mat(nq + 2 * nkv + nidx, H), "o": it.mat(H, c.n_q_heads * c.head_dim)}
    if c.qk_norm:
        w["q_norm"] = it.mat(c.head_dim)
        w["k_norm"] = it.mat(c.head_dim)
    if c.sparse_topk_blocks:
        w["iq_norm"] = it.mat(c.idx_dim)
        w["ik_norm"] = it.mat(c.idx_dim)
    return w


def kda_weights(cfg: ModelConfig, it: _Init) -> Dict[str, torch.Tensor]:
    c, H = cfg.kda, cfg.hidden
    n = c.n_heads * c.head_dim
    r = c.gate_rank
    return {
        "in": it.mat(3 * n, H),                       # q | k | v
        "conv": it.uniform(-0.5, 0.5, 3 * n, c.conv_k),
        "lr_a": it.mat(2 * r + c.n_heads, H),         # f_a | g_a | b
        "f_b": it.mat(n, r) * 10, "g_b": it.mat(n, r) * 10,
        "A_log": torch.log(it.uniform(1.0, 4.0, c.n_heads)),
        "dt_bias": it.uniform(-1.0, 1.0, n),
        "o_norm": it.ones(c.head_dim),
        "o": it.mat(H, n),
    }


def mla_weights(cfg: ModelConfig, it: _Init) -> Dict[str, torch.Tensor]:
    c, H = cfg.mla, cfg.hidden
    idx_rows = 2 * c.idx_dim + c.idx_heads            # wk | cgate | weights_proj
    w = {
        "a": it.mat(c.q_lora + c.kv_lora + c.rope_dim + idx_rows, H),
        "q_a_norm": it.ones(c.q_lora), "kv_a_norm": it.ones(c.kv_lora),
        "q_b": it.mat(c.n_heads * (c.head_dim + c.rope_dim) + c.idx_heads * c.idx_dim, c.q_lora),
        "kv_b": it.mat(c.n_heads * 2 * c.head_dim, c.kv_lora),
        "k_ln_w": it.ones(c.idx_dim), "k_ln_b": it.zeros(c.idx_dim),
        "ape": it.mat(c.pool, c.idx_dim),
        "o": it.mat(H, c.n_heads * c.head_dim),
    }
    if c.sink:
        w["sink"] = it.mat(c.n_heads) * 10
    return w


def moe_weights(cfg: ModelConfig, it: _Init, dense: bool = False) -> Dict[str, torch.Tensor]:
    c, H = cfg.moe, cfg.hidden
    if dense:
        return {"dense_gu": it.mat(2 * c.dense_ffn, H), "dense_down": it.mat(H, c.dense_ffn)}
    Fs = c.shared_ffn or c.ffn * c.n_shared
    w = {
        "gate": it.mat(c.n_experts + (1 if c.shared_gate else 0), H),
        "w_gu": it.mat(c.n_experts, 2 * c.ffn, H),
        "w_down": it.mat(c.n_experts, H, c.ffn),
    }
    if c.router != "softmax":
        w["bias"] = it.mat(c.n_experts)
    if c.n_shared:
        w["s_gu"] = it.mat(2 * Fs, H)
        w["s_down"] = it.mat(H, Fs)
    return w


def hc_weights(cfg: ModelConfig, it: _Init, inject: bool = True) -> Dict[str, torch.Tensor]:
    S, H, r = cfg.hc_streams, cfg.hidden, cfg.hc_rank
    if cfg.hc_kind == "gated":
        w = {"norm": it.mat(S, H), "down": it.mat(r, S * H), "up": it.mat(S * H, r)}
        if inject:
            w["inject"] = it.mat(S, S * H)
        return w
    if cfg.hc_kind == "mhc":
        return {"fn": it.mat(2 * S + S * S, S * H), "scale": it.uniform(0.5, 1.5, 3),
                "base": it.mat(2 * S + S * S), "norm": it.ones(H)}
    return {}


MIX_INIT = {"gdn": gdn_weights, "attn": attn_weights, "kda": kda_weights, "mla": mla_weights}


def layer_weights(cfg: ModelConfig, i: int, it: _Init, kind: str = None) -> dict:
    kind = kind or cfg.layer_types[i]
    w = {"type": kind, "in_norm": it.ones(cfg.hidden), "post_norm": it.ones(cfg.hidden),
         "mix": MIX_INIT[kind](cfg, it), "mlp": moe_weights(cfg, it, dense=i < cfg.moe.dense_layers)}
    if cfg.hc_kind != "none":
        w["hc_mix"] = hc_weights(cfg, it)
        w["hc_mlp"] = hc_weights(cfg, it)
    if i in cfg.ngram_layers:
        D = cfg.ngram_dim * cfg.ngram_heads
        w["ngram"] = {"key": it.mat(cfg.hidden, D), "value": it.mat(cfg.hidden, D),
                      "norm_k": it.ones(cfg.hidden), "norm_q": it.ones(cfg.hidden)}
    return w


def init_weights(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> dict:
    """Dense fp32 weights on CPU, N(0, std), deterministic in `seed`."""
    it = _Init(seed, std)
    W = {"embed": it.mat(cfg.vocab, cfg.hidden), "final_norm": it.ones(cfg.hidden),
         "lm_head": it.mat(cfg.vocab, cfg.hidden),
         "layers": [layer_weights(cfg, i, it) for i in range(cfg.n_layers)]}
    if cfg.hc_kind != "none":
        W["hc_final"] = hc_weights(cfg, it, inject=False)
    if cfg.ngram_layers:
        W["ngram_table"] = it.mat(cfg.ngram_rows, cfg.ngram_dim)
    if cfg.mtp_layers:
        mtp_kind = "attn" if cfg.family == "hybrid" else "mla"
        W["mtp"] = {"fc": it.mat(cfg.hidden, 2 * cfg.hidden), "norm_e": it.ones(cfg.hidden),
                    "norm_h": it.ones(cfg.hidden), "final_norm": it.ones(cfg.hidden),
                    "layers": [layer_weights(cfg, cfg.n_layers, it, kind=mtp_kind)
                               for _ in range(cfg.mtp_layers)]}
    return W


def map_weights(W, fn):
    """Apply fn(tensor) to every tensor leaf of a nested weight dict."""
    if isinstance(W, dict):
        return {k: map_weights(v, fn) for k, v in W.items()}
    if isinstance(W, list):
        return [map_weights(v, fn) for v in W]
    if isinstance(W, torch.Tensor):
        return fn(W)
    return W


def count_params(W) -> int:
    n = 0

    def add(t):
        nonlocal n
        n += t.numel()
        return t
    map_weights(W, add)
    return n


FP32_KEYS = {"conv", "ape", "norm", "scale", "base", "f_b", "g_b"}


def to_device(W, device, dtype=torch.bfloat16):
    """Move a nested weight dict to `device`: matrices in `dtype`, vectors / conv taps / norm and gate
    parameters in fp32, quantised weights as they are."""
    from ..quant.formats import QuantWeight

    def rec(node, key=None):
        if isinstance(node, dict):
            return {k: rec(v, k) for k, v in node.items()}
        if isinstance(node, list):
            return [rec(v, key) for v in node]
        if isinstance(node, QuantWeight):
            return node.to(device)
        if isinstance(node, torch.Tensor):
            if node.dim() <= 1 or key in FP32_KEYS:
                return node.to(device=device, dtype=torch.float32).contiguous()
            return node.to(device=device, dtype=dtype).contiguous()
        return node
    return rec(W)
