"""Decode-kernel microbenchmarks: every launch is replayed from a CUDA graph (no host overhead) over weight copies
larger than L2.  `python -m spark_engine_b200.ops.bench_decode_kernels [dense|moe|gemv|all]`"""
import sys, os, torch
sys.path.insert(0, os.getcwd())
from spark_engine_b200.ops import cuda as cu
from spark_engine_b200.quant import formats as Q
dev = "cuda"
def gtime(fns, reps=10):
    for f in fns: f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns: f()
    g.replay(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps): g.replay()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (reps * len(fns)) * 1e3
H = 2048
out = []
which = sys.argv[1] if len(sys.argv) > 1 else "all"
if which in ("all", "dense"):
    for name, N, K in (("in_proj", 12288, 2048), ("o_proj", 2048, 4096), ("shared_gu", 1024, 2048), ("shared_dn", 2048, 512)):
        ncopy = max(4, int(400e6 / (N * K / 2)))
        ncopy = min(ncopy, 64)
        ws = [Q.random_exl3(N, K, 4, 0, 0.02, i, dev) for i in range(ncopy)]
        for R in (1, 4):
            x = torch.randn(R, K, device=dev).bfloat16()
            t = gtime([(lambda w=w: cu.exl3_gemv(x, w)) for w in ws])
            out.append((f"exl3_gemv {name} R={R}", t, N * K / 2 / t / 1e6))
if which in ("all", "moe"):
    E, F = 512, 512
    wgu = Q.random_exl3(2 * F, H, 4, E, 0.02, 100, dev)
    wd = Q.random_exl3(H, F, 4, E, 0.02, 101, dev)
    for streams in (1, 2, 4):
        Pn = streams * 10
        x = torch.randn(streams, H, device=dev).bfloat16()
        pes = [torch.randperm(E, device=dev)[:Pn].int() for _ in range(16)]
        pr = torch.arange(streams, device=dev).repeat_interleave(10).int()
        t = gtime([(lambda pe=pe: cu.exl3_gemv(x, wgu, items=Pn, rows_per_item=1, pair_expert=pe, pair_row=pr)) for pe in pes])
        out.append((f"moe gate_up pairs={Pn}", t, Pn * 2 * F * H / 2 / t / 1e6))
        gu = torch.randn(Pn, 2 * F, device=dev).bfloat16()
        t = gtime([(lambda pe=pe: cu.exl3_gemv(gu, wd, items=Pn, rows_per_item=1, pair_expert=pe, act=1, out_f32=True)) for pe in pes])
        out.append((f"moe down pairs={Pn}", t, Pn * F * H / 2 / t / 1e6))
if which in ("all", "gemv"):
    V = 151936
    lm = [torch.randn(V, H, device=dev).bfloat16() for _ in range(2)]
    for R in (1, 4, 8, 16):
        x = torch.randn(R, H, device=dev).bfloat16()
        t = gtime([(lambda w=w: cu.gemv_bf16(x, w, out_f32=True)) for w in lm])
        out.append((f"lm_head gemv R={R}", t, V * H * 2 / t / 1e6))
    for name, N in (("router", 513), ("ab", 64)):
        ws = [torch.randn(N, H, device=dev).bfloat16() for _ in range(64)]
        x = torch.randn(4, H, device=dev).bfloat16()
        t = gtime([(lambda w=w: cu.gemv_bf16(x, w, out_f32=True)) for w in ws])
        out.append((f"gemv {name} R=4", t, N * H * 2 / t / 1e6))
    res = torch.randn(4, H, device=dev); d = torch.randn(4, H, device=dev).bfloat16(); w = torch.ones(H, device=dev)
    t = gtime([lambda: cu.add_rmsnorm(d, res, w, 1e-6)] * 32)
    out.append(("add_rmsnorm R=4", t, 0))
for k, t, bw in out:
    print(f"{k:32s} {t:8.1f} us  {bw:8.2f} TB/s")
