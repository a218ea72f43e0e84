"""Microbenchmarks of the prefill-side kernels on shapes of the three model families (CUDA-event timed, L2 flushed
between iterations): chunked gated-DeltaNet, chunked KDA, fused grouped EXL3 expert GEMM, flash-style prefill
attention, latent attention.  `python -m spark_engine_b200.ops.bench_prefill_kernels [name ...] [--small]`;
`--small` shrinks the shapes to a few hundred MB and `--once` launches every kernel exactly once (profiler captures).
"""
from __future__ import annotations

import dataclasses
import sys

import torch

from .. import ops
from ..config import AttnConfig, GdnConfig, KdaConfig, MlaConfig, ModelConfig, MoeConfig
from ..models.plan import make_plan
from ..quant import formats as Q

DEV = "cuda"


ONCE = False          # --once: a single launch per kernel and no A/B variant (profiler captures)


def _time(fn, iters=5):
    if ONCE:
        if iters == 5:
            fn()
            torch.cuda.synchronize()
        return float("nan")
    flush = torch.empty(160 << 20, dtype=torch.uint8, device=DEV)
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return sorted(ts)[len(ts) // 2]


def bench_gdn(small):
    from ..models.model import GdnMixer
    T = 1024 if small else 4096
    cfg = dataclasses.replace(ModelConfig(), gdn=GdnConfig(n_k_heads=16, n_v_heads=32, head_dim=128))
    c = cfg.gdn
    g = torch.Generator(device=DEV).manual_seed(1)
    nq, nv = c.n_k_heads * 128, c.n_v_heads * 128
    w = {"conv": torch.rand(2 * nq + nv, 4, device=DEV, generator=g) - 0.5, "A_log": torch.zeros(c.n_v_heads, device=DEV),
         "dt_bias": torch.zeros(c.n_v_heads, device=DEV), "norm": torch.ones(128, device=DEV)}
    proj = torch.randn(T, 2 * nq + 2 * nv, device=DEV, generator=g).bfloat16()
    ab = torch.randn(T, 2 * c.n_v_heads, device=DEV, generator=g).bfloat16()
    m = GdnMixer(cfg, w, 1, DEV, torch.bfloat16)
    plan = make_plan([(0, [1] * T, 0)], device=DEV)
    cu = ops.cuda_ops()
    us = _time(lambda: cu.gdn_mixer(m, proj, ab, plan, True))
    cu.GDN_CHUNKED = False
    us_seq = _time(lambda: cu.gdn_mixer(m, proj, ab, plan, True), 2)
    cu.GDN_CHUNKED = True
    print(f"gdn_chunk  T={T} heads=32x128: chunked {us:9.1f} us   sequential {us_seq:9.1f} us")


def bench_kda(small):
    from ..models.model import KdaMixer
    T = 1024 if small else 4096
    c = KdaConfig(n_heads=64, head_dim=128, gate_rank=128)
    cfg = dataclasses.replace(ModelConfig(), kda=c)
    n, r = 64 * 128, 128
    g = torch.Generator(device=DEV).manual_seed(1)
    rnd = lambda *s: torch.randn(*s, device=DEV, generator=g)
    w = {"conv": torch.rand(3 * n, 4, device=DEV, generator=g) - 0.5, "f_b": rnd(n, r) * 0.1, "g_b": rnd(n, r) * 0.1,
         "A_log": torch.zeros(64, device=DEV), "dt_bias": torch.zeros(n, device=DEV), "o_norm": torch.ones(128, device=DEV)}
    pre, lr = rnd(T, 3 * n).bfloat16(), rnd(T, 2 * r + 64).bfloat16()
    m = KdaMixer(cfg, w, 1, DEV, torch.bfloat16)
    plan = make_plan([(0, [1] * T, 0)], device=DEV)
    cu = ops.cuda_ops()
    us = _time(lambda: cu.kda_mixer(m, pre, lr, plan, True))
    cu.KDA_CHUNKED = False
    us_seq = _time(lambda: cu.kda_mixer(m, pre, lr, plan, True), 2)
    cu.KDA_CHUNKED = True
    print(f"kda_chunk  T={T} heads=64x128: chunked {us:9.1f} us   sequential {us_seq:9.1f} us (incl. gate GEMMs)")


def bench_moe(small):
    from . import exl3_moe
    E, H, F, T = (64, 2048, 512, 128) if small else (512, 2048, 512, 1024)
    c = MoeConfig(n_experts=E, top_k=10, ffn=F, router="softmax", shared_gate=False, n_shared=0)
    g = torch.Generator(device=DEV).manual_seed(2)
    w = {"gate": (torch.randn(E, H, device=DEV, generator=g) * 0.1).bfloat16(),
         "w_gu": Q.random_exl3(2 * F, H, 4, E, 0.05, 1, DEV), "w_down": Q.random_exl3(H, F, 4, E, 0.05, 2, DEV)}
    h = torch.randn(T, H, device=DEV, generator=g).bfloat16()
    us = _time(lambda: ops.moe(h, w, c))
    exl3_moe.EXL3_MOE_FUSED = False
    us_ref = _time(lambda: ops.moe(h, w, c), 3)
    exl3_moe.EXL3_MOE_FUSED = True
    wb = w["w_gu"].nbytes() + w["w_down"].nbytes()
    print(f"exl3 moe   T={T} E={E} top10 H={H} F={F}: fused {us:9.1f} us ({wb / us / 1e6:5.2f} TB/s of packed weights)"
          f"   reconstruct + tcgen05 {us_ref:9.1f} us")


def bench_attn(small):
    from ..models.model import AttnMixer, SeqInfo
    T = 1024 if small else 4096
    a = AttnConfig(n_q_heads=16, n_kv_heads=2, head_dim=256, rope_dim=64, gated=True, qk_norm=True, sparse_topk_blocks=0)
    cfg = dataclasses.replace(ModelConfig(), attn=a, hidden=2048)
    g = torch.Generator(device=DEV).manual_seed(3)
    w = {"q_norm": torch.zeros(256, device=DEV), "k_norm": torch.zeros(256, device=DEV)}
    m = AttnMixer(cfg, w, T + 64, DEV, torch.bfloat16)
    qkv = torch.randn(T, 16 * 512 + 2 * 2 * 256, device=DEV, generator=g).bfloat16()
    plan = make_plan([(0, [1] * T, 0)], device=DEV)
    seqs = [SeqInfo(0, T + 64)]
    cu = ops.cuda_ops()
    us = _time(lambda: cu.attn_mixer(m, qkv, plan, seqs))
    flops = 4 * T * T / 2 * 256 * 16
    cu.ATTN_PREFILL_KERNEL = False
    us_row = _time(lambda: cu.attn_mixer(m, qkv, plan, seqs), 2)
    cu.ATTN_PREFILL_KERNEL = True
    print(f"attn_prefill T={T} 16q/2kv x256: flash {us:9.1f} us ({flops / us / 1e6:6.1f} TFLOP/s incl. prep)   per-row kernel {us_row:9.1f} us")


BENCHES = {"gdn": bench_gdn, "kda": bench_kda, "moe": bench_moe, "attn": bench_attn}

if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    small = "--small" in sys.argv
    ONCE = "--once" in sys.argv
    for name in (args or list(BENCHES)):
        BENCHES[name](small)
