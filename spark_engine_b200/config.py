"""Typed configuration: model hyper-parameters and engine switches.

One `ModelConfig` describes every architecture the engine serves; the layer *types*
select the code path (gated-DeltaNet, KDA, softmax/sparse GQA, MLA+indexer, compressed
sparse attention), the dimensions come from the config.  The reference reads model
hyper-parameters from `config.json` (engine-rs/src/config.rs, engine-rs/src/ds41/cfg.rs:7-76)
and spreads ~900 environment switches over the code (docs/configuration.md:3-9); here a
single `EngineConfig` carries the small set of switches that matter, with `SPARK_*`
environment fallbacks and `--flag` overrides.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass, field
from typing import List, Optional


@dataclass
class AttnConfig:
    n_q_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    rope_dim: int = 64            # NeoX rotary on the first rope_dim dims (partial when < head_dim)
    rope_theta: float = 1e4
    yarn_factor: float = 1.0      # >1: YaRN scaling beyond yarn_orig_len
    yarn_orig_len: int = 262144
    qk_norm: bool = False         # Gemma-style (1+w) RMS norm on q and k
    gated: bool = False           # per-head sigmoid output gate (q projection is 2x wide)
    sparse_topk_blocks: int = 0   # 0 = dense; else top-k blocks of `block` tokens (+ tail)
    block: int = 4
    idx_heads: int = 4
    idx_dim: int = 128


@dataclass
class GdnConfig:
    n_k_heads: int = 4
    n_v_heads: int = 4
    head_dim: int = 64
    conv_k: int = 4


@dataclass
class KdaConfig:
    n_heads: int = 4
    head_dim: int = 64
    conv_k: int = 4
    gate_rank: int = 32           # low-rank f_a/f_b and g_a/g_b projections


@dataclass
class MlaConfig:
    n_heads: int = 4
    q_lora: int = 96
    kv_lora: int = 64
    head_dim: int = 32            # dk = dv (no-rope part)
    rope_dim: int = 0             # 0: GLM-style MLA without RoPE; >0: DeepSeek-style rope part
    rope_theta: float = 1e4
    # indexer (DSA)
    idx_heads: int = 4
    idx_dim: int = 32
    pool: int = 4
    topk_pools: int = 512
    sink: bool = False            # attention sink logit in the denominator (DS-style)
    window: int = 0               # sliding window (DS-style compressed sparse attention)
    compress: int = 0             # compression ratio of the global KV (0 = none)


@dataclass
class MoeConfig:
    n_experts: int = 16
    top_k: int = 4
    ffn: int = 128
    n_shared: int = 1
    shared_ffn: int = 0           # 0 -> ffn * n_shared
    router: str = "softmax"       # softmax | sigmoid_bias | sqrt_softplus
    route_scale: float = 1.0
    shared_gate: bool = False     # sigmoid(x . w_sg) on the shared expert
    swiglu_limit: float = 0.0     # clamp-SwiGLU limit (0 = off)
    dense_layers: int = 0         # first N layers use a dense MLP of width dense_ffn
    dense_ffn: int = 0


@dataclass
class ModelConfig:
    name: str = "tiny-hybrid"
    family: str = "hybrid"        # hybrid (Qwen-style) | glm | ds4
    n_layers: int = 4
    layer_types: List[str] = field(default_factory=lambda: ["gdn", "gdn", "gdn", "attn"])
    hidden: int = 256
    vocab: int = 4096
    norm_eps: float = 1e-6
    attn: AttnConfig = field(default_factory=AttnConfig)
    gdn: GdnConfig = field(default_factory=GdnConfig)
    kda: KdaConfig = field(default_factory=KdaConfig)
    mla: MlaConfig = field(default_factory=MlaConfig)
    moe: MoeConfig = field(default_factory=MoeConfig)
    hc_streams: int = 1           # 1 = plain residual; 4 = hyper-connections (gated HC / mHC)
    hc_kind: str = "none"         # none | gated | mhc
    hc_rank: int = 32
    sinkhorn_iters: int = 20
    mtp_layers: int = 0           # MTP draft layers (chain drafter)
    mtp_depth: int = 3
    ngram_layers: List[int] = field(default_factory=list)   # layers with hashed n-gram embeddings
    ngram_rows: int = 0
    ngram_dim: int = 0
    ngram_heads: int = 16
    weight_format: str = "dense"  # dense | exl3 | mx (MXFP4 experts + FP8 dense)
    exl3_bits: int = 4
    kv_dtype: str = "bf16"        # bf16 | fp8
    kv_quant_on_cpu: bool = False  # the CPU runner keeps fp32 caches; set to model the packed FP8 latent rows there too

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1)

    @staticmethod
    def from_dict(d: dict) -> "ModelConfig":
        d = dict(d)
        for key, cls in (("attn", AttnConfig), ("gdn", GdnConfig), ("kda", KdaConfig),
                         ("mla", MlaConfig), ("moe", MoeConfig)):
            if key in d and isinstance(d[key], dict):
                d[key] = cls(**d[key])
        return ModelConfig(**d)

    @staticmethod
    def from_json(path: str) -> "ModelConfig":
        with open(path) as f:
            return ModelConfig.from_dict(json.load(f))


def _pattern(n_layers: int, period: int, a: str, b: str) -> List[str]:
    """`period-1` layers of kind `a`, then one of kind `b`, repeated."""
    return [b if (i + 1) % period == 0 else a for i in range(n_layers)]


def tiny_hybrid() -> ModelConfig:
    """Plumbing model: 3 gated-DeltaNet layers then 1 softmax GQA layer, 16-expert MoE."""
    return ModelConfig()


def qwen3next_style(n_layers: int = 48, weight_format: str = "exl3", kv_dtype: str = "bf16") -> ModelConfig:
    """Qwen3-Next-style hybrid: every 4th layer gated sparse GQA, the rest gated-DeltaNet;
    512 experts top-10 + shared; one MTP draft layer with chain depth 3."""
    return ModelConfig(
        name="qwen3next-style", family="hybrid", n_layers=n_layers,
        layer_types=_pattern(n_layers, 4, "gdn", "attn"), hidden=2048, vocab=151936,
        attn=AttnConfig(n_q_heads=16, n_kv_heads=2, head_dim=256, rope_dim=64, rope_theta=1e7,
                        yarn_factor=4.0, qk_norm=True, gated=True, sparse_topk_blocks=512, block=4,
                        idx_heads=4, idx_dim=128),
        gdn=GdnConfig(n_k_heads=16, n_v_heads=32, head_dim=128, conv_k=4),
        moe=MoeConfig(n_experts=512, top_k=10, ffn=512, n_shared=1, router="softmax", shared_gate=True),
        mtp_layers=1, mtp_depth=3, weight_format=weight_format, exl3_bits=4, kv_dtype=kv_dtype)


def glm_style(n_layers: int = 45, weight_format: str = "exl3") -> ModelConfig:
    """GLM-style: 3 KDA linear-attention layers per MLA layer with a DSA top-2048 indexer;
    288 experts top-8 (sigmoid+bias router, x2.5, clamp-SwiGLU 10) + shared expert."""
    types = ["mla" if i % 4 == 3 else "kda" for i in range(n_layers)]
    return ModelConfig(
        name="glm-style", family="glm", n_layers=n_layers, layer_types=types, hidden=4096, vocab=154880,
        norm_eps=1e-5,
        kda=KdaConfig(n_heads=64, head_dim=128, conv_k=4, gate_rank=128),
        mla=MlaConfig(n_heads=64, q_lora=1536, kv_lora=512, head_dim=256, rope_dim=64, idx_heads=32,
                      idx_dim=128, pool=4, topk_pools=512),
        moe=MoeConfig(n_experts=288, top_k=8, ffn=1536, n_shared=1, router="sigmoid_bias", route_scale=2.5,
                      swiglu_limit=10.0, dense_layers=3, dense_ffn=12288),
        hc_streams=1, hc_kind="none", mtp_layers=2, mtp_depth=5, weight_format=weight_format)


def ds4_style(n_layers: int = 40, weight_format: str = "mx") -> ModelConfig:
    """DeepSeek-V4-style: compressed sparse MLA with hierarchical top-k indexer, 384 experts
    top-6 (MXFP4) + shared (FP8), hashed n-gram tables streamed from host, FP8 KV."""
    return ModelConfig(
        name="ds4-style", family="ds4", n_layers=n_layers, layer_types=["mla"] * n_layers, hidden=4096,
        vocab=129280,
        mla=MlaConfig(n_heads=64, q_lora=1536, kv_lora=512, head_dim=128, rope_dim=64, idx_heads=16, idx_dim=128,
                      pool=4, topk_pools=512, sink=True, window=128, compress=4),
        moe=MoeConfig(n_experts=384, top_k=6, ffn=2048, n_shared=1, router="sqrt_softplus", route_scale=1.5,
                      swiglu_limit=10.0),
        mtp_layers=1, mtp_depth=3, ngram_layers=[1, 14], ngram_rows=1 << 22, ngram_dim=1024,
        weight_format=weight_format, kv_dtype="fp8")


def scaled_down(cfg: ModelConfig, hidden: int = 256, n_layers: int = 4, vocab: int = 1024) -> ModelConfig:
    """Same layer types, small dimensions: the CPU test shape of a large config."""
    c = dataclasses.replace(cfg)
    per = 4
    c.n_layers = n_layers
    c.layer_types = [cfg.layer_types[i % max(per, 1)] if i < len(cfg.layer_types) else cfg.layer_types[-1]
                     for i in range(n_layers)]
    c.hidden, c.vocab = hidden, vocab
    c.attn = dataclasses.replace(cfg.attn, n_q_heads=4, n_kv_heads=2, head_dim=64,
                                 rope_dim=min(cfg.attn.rope_dim, 32), idx_heads=2, idx_dim=32,
                                 sparse_topk_blocks=min(cfg.attn.sparse_topk_blocks, 8))
    c.gdn = dataclasses.replace(cfg.gdn, n_k_heads=2, n_v_heads=4, head_dim=32)
    c.kda = dataclasses.replace(cfg.kda, n_heads=4, head_dim=32, gate_rank=16)
    c.mla = dataclasses.replace(cfg.mla, n_heads=4, q_lora=64, kv_lora=32, head_dim=32,
                                rope_dim=16 if cfg.mla.rope_dim else 0, idx_heads=2, idx_dim=16,
                                topk_pools=min(cfg.mla.topk_pools, 8),
                                window=min(cfg.mla.window, 16))
    c.moe = dataclasses.replace(cfg.moe, n_experts=16, top_k=min(cfg.moe.top_k, 4), ffn=128,
                                dense_layers=min(cfg.moe.dense_layers, 1), dense_ffn=256 if cfg.moe.dense_layers else 0)
    c.ngram_layers = [i for i in cfg.ngram_layers if i < n_layers]
    c.ngram_rows = 4096 if cfg.ngram_rows else 0
    c.ngram_dim = 64 if cfg.ngram_dim else 0
    c.weight_format = "dense"
    c.name = cfg.name + "-small"
    return c


def _env(name: str, default, cast=str):
    v = os.environ.get("SPARK_" + name.upper())
    if v is None:
        return default
    if cast is bool:
        return v not in ("0", "false", "False", "")
    return cast(v)


@dataclass
class EngineConfig:
    """Engine switches (CLI `--flag`, JSON file, `SPARK_<NAME>` environment fallback)."""
    model: str = "tiny-hybrid"
    numerics: str = "deterministic"      # deterministic | fast (multimem hardware reductions)
    tp: int = 1
    ep: int = 1
    max_seqs: int = 8
    max_rows: int = 64                   # rows per decode/verify forward
    prefill_chunk: int = 8192            # larger chunks amortise the one-off expert reconstruction (16K prompt: 14.7k tok/s at 4096, 17.1k at 8192)
    kv_tokens: int = 1 << 20             # KV budget in tokens
    kv_granule: int = 16384
    kv_backing: str = "dense"            # dense (one allocation of the whole budget) | vmm (address space reserved, backed on demand)
    cuda_graphs: bool = True
    spec: str = "mtp"                    # none | mtp | lookup | feature (tap-conditioned drafter) | stage (staged drafter)
    spec_depth: int = 3
    spec_policy: str = "theta"           # tau | theta | rate | cost
    spec_tree_widths: str = ""           # e.g. "3,2,1": verify a tree (widths per depth) built from the feature drafter's candidates
    comm: str = "fused"                  # fused (peer-memory kernels) | nccl (baseline)
    comm_wait_ms: float = 1000.0         # bound of every device-side wait
    step_deadline_s: float = 0.0         # > 0: a watchdog aborts the process when one engine step runs longer
    pcache_dir: Optional[str] = None
    pcache_bytes: int = 64 << 30
    host_mem_floor_gb: float = 2.0       # > 0: below this much available host memory the server sheds load
    meminfo_path: str = ""               # where the memory guard reads MemAvailable ("" = /proc/meminfo)
    socket: str = "/tmp/spark-b200.sock"
    host: str = "127.0.0.1"
    port: int = 8000
    profile: bool = False
    prewarm: bool = False         # run synthetic requests for 1..max_seqs streams before serving (captures the graphs)
    serve_log: bool = False       # one stderr line per admission / prefill forward / round ([serve-admit], [serve-round] ...)
    draft_trace: str = ""         # file ("-" = stderr) that gets one JSON line per speculative round
    nvtx: bool = False
    log_rounds: bool = False
    seed: int = 0

    @staticmethod
    def from_env(**over) -> "EngineConfig":
        c = EngineConfig()
        for f in dataclasses.fields(c):
            cur = getattr(c, f.name)
            cast = type(cur) if cur is not None else str
            setattr(c, f.name, _env(f.name, cur, cast))
        for k, v in over.items():
            if v is not None:
                setattr(c, k, v)
        return c

    def signature(self) -> str:
        """Flag signature: captured graphs are keyed on it so a changed switch forces a
        re-capture (reference: spec_probe.rs:316-327)."""
        keys = ("numerics", "tp", "ep", "comm", "spec", "spec_depth", "cuda_graphs")
        return "|".join(f"{k}={getattr(self, k)}" for k in keys)


PRESETS = {
    "tiny-hybrid": tiny_hybrid,
    "qwen3next-style": qwen3next_style,
    "glm-style": glm_style,
    "ds4-style": ds4_style,
}


def get_model_config(name: str, **kw) -> ModelConfig:
    if name.endswith(".json"):
        return ModelConfig.from_json(name)
    return PRESETS[name](**kw)
