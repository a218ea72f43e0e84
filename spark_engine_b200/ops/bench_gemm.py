"""Throughput of the tcgen05 GEMM against torch.matmul (cuBLAS) on the same shapes.

  python -m spark_engine_b200.ops.bench_gemm [--ncu-case] [--mx]

CUDA-event timing, 3 warm-ups, operands rotated through copies larger than L2 for the small shapes.  Prints one JSON
line per shape with TFLOP/s and the fraction of the measured bf16 peak (MEASURED_PEAKS.json when present).
`--ncu-case` runs a single 8192x4096x4096 launch pair (the case captured under ncu).  `--mx` adds the block-scaled MXFP8
GEMM (e4m3 operands, E8M0 scale per 32 along K, scales applied by the tensor core) on the same shapes."""
from __future__ import annotations

import json
import os
import sys

import torch

from . import cuda as cu


def main():
    ncu_case = "--ncu-case" in sys.argv
    dev = "cuda"
    peak = 1651.4
    try:
        with open(os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")) as f:
            peak = json.load(f)["bf16_tflops"]
    except Exception:
        pass
    shapes = [(8192, 4096, 4096)] if ncu_case else [(4096, 4096, 4096), (8192, 8192, 8192), (8192, 4096, 4096),
                                                     (4096, 12288, 2048), (4096, 2048, 4096), (16384, 1024, 2048), (512, 4096, 4096)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for M, N, K in shapes:
        ncopy = max(2, int(300e6 // ((M * K + N * K) * 2)) + 1)
        a = [torch.randn(M, K, device=dev).bfloat16() for _ in range(ncopy)]
        b = [torch.randn(N, K, device=dev).bfloat16() for _ in range(ncopy)]
        res = {}
        for name, fn in (("tcgen05", lambda i: cu.gemm_bf16(a[i % ncopy], b[i % ncopy])),
                         ("cublas", lambda i: torch.matmul(a[i % ncopy], b[i % ncopy].t()))):
            iters = 1 if ncu_case else 20
            for i in range(0 if ncu_case else 3):
                fn(i)
            torch.cuda.synchronize()
            e0.record()
            for i in range(iters):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            res[name] = {"ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)}
        if "--mx" in sys.argv and K % 128 == 0:
            from ..quant import formats as Q
            from . import mx
            wq = [Q.random_mxfp8(N, K, 0.02, i, dev) for i in range(ncopy)]
            aq = [(torch.randn(M, K, device=dev) * 50).clamp(-448, 448).to(torch.float8_e4m3fn) for _ in range(ncopy)]
            asf = torch.full((M, K // 32), 120, dtype=torch.uint8, device=dev)
            ab = mx.sf_blocks(asf)
            for w in wq:
                w._sf_blocks = mx.sf_blocks(w.scales)
            lib = mx._lib()
            out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

            def run_mx(i):
                w = wq[i % ncopy]
                lib.spark_gemm_mxfp8(cu.P(aq[i % ncopy]), cu.P(w.q), cu.P(ab), cu.P(w._sf_blocks), cu.P(out), M, N, K, K, K, N, 0,
                                     cu.P(cu.status_word(torch.device(dev))), cu.stream())
            iters = 1 if ncu_case else 20
            for i in range(0 if ncu_case else 3):
                run_mx(i)
            torch.cuda.synchronize()
            e0.record()
            for i in range(iters):
                run_mx(i)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / iters
            res["tcgen05_mxfp8"] = {"ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 1)}
        c = cu.gemm_bf16(a[0], b[0]).float()
        ref = torch.matmul(a[0], b[0].t()).float()
        print(json.dumps({"M": M, "N": N, "K": K, **res, "frac_of_measured_peak": round(res["tcgen05"]["tflops"] / peak, 3),
                          "vs_cublas": round(res["tcgen05"]["tflops"] / res["cublas"]["tflops"], 3),
                          "rel_err_vs_cublas": float(((c - ref).norm() / ref.norm()).item()),
                          "status": list(cu.read_status(torch.device(dev)))}))


if __name__ == "__main__":
    main()
