"""Microbenchmark of the MXFP4 expert kernels at the DS-style shapes (hidden 4096, expert FFN 2048).

    python -m spark_engine_b200.ops.bench_mx_experts [--pairs 24] [--tokens 1024] [--experts 64]

Decode: `pairs` (token, expert) pairs with distinct experts through the GEMV (gate/up, then SwiGLU + down) and,
with --tc, through the block-scaled tensor-core kernel.  Prefill: `tokens` x top-6 rows in expert order through
the fused grouped kernel and the tensor-core kernel.  CUDA-event timed, median of the iterations, L2 flushed by a
256 MB write before every timed launch.  One JSON line per measurement.  The tensor-core calls are four launches
(activation quantiser, work items, scale blocks, GEMM): time them with --graph, without it the host launch path of the
small decode case is what the events see.
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pairs", type=int, default=24)
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tc", action="store_true", help="also time the block-scaled tcgen05 path")
    ap.add_argument("--once", action="store_true", help="one launch of each kernel, no timing (profiler runs)")
    ap.add_argument("--graph", action="store_true", help="time each call as a captured CUDA graph (as the decode "
                    "rounds run it): removes the host launch path of multi-kernel calls from the measurement")
    a = ap.parse_args()
    from . import cuda as cu
    from . import mx
    from ..quant import formats as Q
    dev = "cuda"
    E, F, H = a.experts, 2048, 4096
    wgu = Q.random_mxfp4(2 * F, H, E, 0.02, 1, dev)
    wd = Q.random_mxfp4(H, F, E, 0.02, 2, dev)
    P = a.pairs
    x = torch.randn(4, H, device=dev).bfloat16()
    pe = torch.randperm(E, device=dev)[:P].int()
    pr = (torch.arange(P, device=dev) % 4).int()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def run(fn):
        if a.once:
            fn()
            torch.cuda.synchronize()
            return float("nan")
        for _ in range(3):
            fn()
        if a.graph:
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                fn()
            fn = gr.replay
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    def report(name, us, nbytes=None, flops=None):
        d = {"kernel": name, "us": round(us, 1)}
        if nbytes:
            d["weight_TBps"] = round(nbytes / us / 1e6, 2)
        if flops:
            d["TFLOPs"] = round(flops / us / 1e6, 1)
        print(json.dumps(d), flush=True)

    b_gu = P * 2 * F * H / 2 * (1 + 1 / 16)
    b_d = P * H * F / 2 * (1 + 1 / 16)
    gu = mx.gemv(x, wgu, items=P, rows_per_item=1, pair_expert=pe, pair_row=pr)
    report("gemv gate/up %d pairs" % P, run(lambda: mx.gemv(x, wgu, items=P, rows_per_item=1, pair_expert=pe, pair_row=pr)), b_gu)
    report("gemv swiglu+down %d pairs" % P,
           run(lambda: mx.gemv(gu, wd, items=P, rows_per_item=1, pair_expert=pe, act=1, limit=10.0, out_f32=True)), b_d)
    if a.tc:
        report("tcgen05 gate/up %d pairs" % P, run(lambda: mx.moe_mxfp4_tc(x, wgu, P, P, pair_expert=pe, pair_row=pr)), b_gu)
        report("tcgen05 swiglu+down %d pairs" % P,
               run(lambda: mx.moe_mxfp4_tc(gu, wd, P, P, pair_expert=pe, act=1, limit=10.0, out_f32=True)), b_d)
    T = a.tokens
    ids = torch.stack([torch.randperm(E, device=dev)[:6] for _ in range(T)]).int()
    perm, inv, offs, tiles, ntile, max_tiles = cu.moe_sort(ids.view(-1), E)
    act = torch.randn(T * 6, H, device=dev).bfloat16()
    fl = 2 * T * 6 * 2 * F * H
    report("fused grouped gate/up %d rows" % (T * 6), run(lambda: mx.mx_mgemm(act, wgu, tiles, ntile, max_tiles)), flops=fl)
    if a.tc:
        report("tcgen05 grouped gate/up %d rows" % (T * 6),
               run(lambda: mx.moe_mxfp4_tc(act, wgu, T * 6, max_tiles, tiles=tiles, ntile=ntile)), flops=fl)
    print(json.dumps({"status": cu.read_status(torch.device(dev))}))


if __name__ == "__main__":
    main()
