"""Microbenchmark of the fused compute+collective kernels against the NCCL + cuBLAS path.

  torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m spark_engine_b200.parallel.bench_fused

(a) row-parallel bf16 GEMM [M, K/tp] x [K/tp, N], K = N = 4096, M in {1,4,16,64,512,4096}, fused with
    all-reduce + residual add + RMSNorm;
(b) MoE expert-parallel dispatch + combine, T in {1,16,256,4096} tokens per rank, hidden 4096, 256 experts
    top-8, uniform-random router logits, FP8 e4m3 payload with 1x128 scales.
All inputs N(0,1) bf16, seed 0.  Device-timed with CUDA events, max over ranks; every case also reports its
roofline: the slower of FLOPs / measured GEMM peak and NVLink bytes / measured link bandwidth.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist


def main():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from spark_engine_b200.ops import cuda as cu
    from spark_engine_b200.parallel import symm

    peaks = {"bf16_tflops": 1651.4, "link_gbs": 770.0}
    try:
        with open(os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")) as f:
            peaks["bf16_tflops"] = json.load(f)["bf16_tflops"]
    except Exception:
        pass
    arena = symm.Arena(1 << 30)
    iters, warm = 20, 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    g = torch.Generator(device=dev).manual_seed(0)
    results = []
    # ------------------------------------------------------------------ (a) row-parallel GEMM + AR + residual + RMSNorm
    K = N = 4096
    Ks = K // world
    w = torch.randn(N, Ks, device=dev, generator=g).bfloat16()
    nw = torch.ones(N, device=dev)
    far = symm.FusedAllReduce(arena, "bench_ar", 64, N)
    rp = symm.RowParallelGemm(arena, "bench_rp", 4096, N)
    for M in (1, 4, 16, 64, 512, 4096):
        x = torch.randn(M, Ks, device=dev, generator=g).bfloat16()
        res = torch.zeros(M, N, device=dev)
        rpr = (M + world - 1) // world
        res_owned = torch.zeros(rpr, N, device=dev)

        def ours():
            if M <= 16:
                part = cu.gemv_bf16(x, w, out_f32=True)
                return far(part, res=res, norm_w=nw)
            return rp(x, w, res_owned=res_owned, norm_w=nw, fused=True)

        def base():
            y = torch.matmul(x, w.t()).float()
            dist.all_reduce(y)
            r = res + y
            return (r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + 1e-6) * nw).bfloat16()

        t_ours, t_base = timed(ours), timed(base)
        flops = 2.0 * M * N * Ks
        nv_bytes = (world - 1) / world * M * N * (4 + 2) if world > 1 else 0.0
        roof_us = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (peaks["link_gbs"] * 1e9)) * 1e6
        results.append({"case": "rowpar_gemm_ar_residual_norm", "M": M, "K": K, "N": N, "tp": world, "ours_us": round(t_ours, 2),
                        "nccl_cublas_us": round(t_base, 2), "speedup": round(t_base / t_ours, 2),
                        "roofline_us": round(roof_us, 3), "frac_of_roofline": round(roof_us / t_ours, 3)})
    # ------------------------------------------------------------------ (b) EP dispatch + combine
    H, E, k = 4096, 256, 8
    for T in (1, 16, 256, 4096):
        ep = symm.ExpertParallel(arena, f"bench_ep{T}", T, H, E, k)
        x = torch.randn(T, H, device=dev, generator=g).bfloat16()
        logits = torch.rand(T, E, device=dev, generator=g)

        def ours_ep():
            wts, ids = ep.dispatch(x, logits)
            return ep.combine(ep.a_rows, wts, T)

        epr = E // world

        def base_ep():
            p = torch.softmax(logits, -1)
            wt, idx = torch.topk(p, k, -1)
            wt = wt / wt.sum(-1, keepdim=True)
            xb = x.float().view(T, H // 128, 128)
            sc = xb.abs().amax(-1).clamp_min(1e-4) / 448.0
            q = (xb / sc.unsqueeze(-1)).to(torch.float8_e4m3fn).view(T, H)
            dst = (idx // epr).flatten()
            order = torch.argsort(dst, stable=True)
            tok = order // k
            send_q = q[tok].view(torch.uint8)
            send_s = sc[tok]
            counts = torch.bincount(dst, minlength=world)
            rcounts = torch.empty_like(counts)
            dist.all_to_all_single(rcounts, counts)
            sc_l, rc_l = counts.tolist(), rcounts.tolist()
            recv_q = torch.empty(sum(rc_l), H, dtype=torch.uint8, device=dev)
            recv_s = torch.empty(sum(rc_l), H // 128, device=dev)
            dist.all_to_all_single(recv_q, send_q, rc_l, sc_l)
            dist.all_to_all_single(recv_s, send_s, rc_l, sc_l)
            y = (recv_q.view(torch.float8_e4m3fn).float().view(-1, H // 128, 128) * recv_s.unsqueeze(-1)).view(-1, H).bfloat16()
            back = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
            dist.all_to_all_single(back, y, sc_l, rc_l)
            out = torch.zeros(T * k, H, dtype=torch.bfloat16, device=dev)
            out[order] = back
            return (out.view(T, k, H).float() * wt.unsqueeze(-1)).sum(1).bfloat16()

        t_ours, t_base = timed(ours_ep), timed(base_ep)
        frac_remote = (world - 1) / world
        nv_bytes = T * k * frac_remote * (H + H // 128 * 4 + 16) + T * k * frac_remote * H * 2      # dispatch + return
        roof_us = nv_bytes / (peaks["link_gbs"] * 1e9) * 1e6
        results.append({"case": "ep_dispatch_combine", "T": T, "H": H, "E": E, "top_k": k, "ep": world,
                        "ours_us": round(t_ours, 2), "nccl_torch_us": round(t_base, 2), "speedup": round(t_base / t_ours, 2),
                        "roofline_us": round(roof_us, 3), "frac_of_roofline": round(roof_us / t_ours, 3) if t_ours else None})
    st = arena.status()
    if rank == 0:
        for r in results:
            print(json.dumps(r))
        print(json.dumps({"device_status": list(st), "world": world, "peaks": peaks}))
    arena.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
