"""Microbenchmark of the fused compute+collective kernels against the NCCL + cuBLAS path.

  torchrun --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m spark_engine_b200.parallel.bench_fused

(a) row-parallel bf16 GEMM [M, K/tp] x [K/tp, N], K = N = 4096, M in {1,4,16,64,512,4096}, fused with
    all-reduce + residual add + RMSNorm;
(b) MoE expert-parallel dispatch + combine, T in {1,16,256,4096} tokens per rank, hidden 4096, 256 experts
    top-8, uniform-random router logits, FP8 e4m3 payload with 1x128 scales.
(c) all-gather fused into a column-parallel GEMM: x row-sharded [M/tp, 4096], W [4096/tp, 4096];
(d) sequence-parallel residual update: reduce-scatter of fp32 partial rows [M, 2048] to the row owners + residual +
    RMSNorm + bf16 all-gather, against the full-row all-reduce kernel and NCCL;
(e) decode-round collectives inside a captured CUDA graph (32 back-to-back launches per replay): all-reduce + residual
    + RMSNorm of 1 / 4 / 16 rows x 2048 in the low-latency wire format and in the flag format, the row-parallel EXL3
    GEMV with the all-reduce in its epilogue, the packet arg-max; NCCL + ATen beside them.
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
    arena = symm.Arena(2 << 30)
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
    # ------------------------------------------------------------------ (c) all-gather + column-parallel GEMM
    Kc, Nc = 4096, 4096 // world
    wc = torch.randn(Nc, Kc, device=dev, generator=g).bfloat16()
    agg = symm.AllGatherGemm(arena, "bench_ag", 4096, Kc)
    for M in (64 * world, 512, 4096):
        rows = M // world
        xl = torch.randn(rows, Kc, device=dev, generator=g).bfloat16()

        def ours_ag():
            return agg(xl, wc)

        def base_ag():
            full = torch.empty(M, Kc, dtype=torch.bfloat16, device=dev)
            dist.all_gather_into_tensor(full, xl)
            return torch.matmul(full, wc.t())

        t_ours, t_base = timed(ours_ag), timed(base_ag)
        flops = 2.0 * M * Nc * Kc
        nv_bytes = (world - 1) * rows * Kc * 2
        roof_us = max(flops / (peaks["bf16_tflops"] * 1e12), nv_bytes / (peaks["link_gbs"] * 1e9)) * 1e6
        results.append({"case": "allgather_colpar_gemm", "M": M, "K": Kc, "N_shard": Nc, "tp": world, "ours_us": round(t_ours, 2),
                        "nccl_cublas_us": round(t_base, 2), "speedup": round(t_base / t_ours, 2),
                        "roofline_us": round(roof_us, 3), "frac_of_roofline": round(roof_us / t_ours, 3)})
    # ------------------------------------------------------------------ (d) sequence-parallel residual update of prefill rows
    Hs = 2048
    nws = torch.ones(Hs, device=dev)
    sp = symm.RowParallelGemm(arena, "bench_sp", 4096, Hs)
    far_big = symm.FusedAllReduce(arena, "bench_ar_big", 1024, Hs)
    for M in (1024, 4096):
        part = torch.randn(M, Hs, device=dev, generator=g)
        resf = torch.zeros(M, Hs, device=dev)
        rpr = M // world

        def ours_sp():
            return sp.rows(part, resf[rank * rpr:(rank + 1) * rpr], nws, 1e-6)

        def ours_ar():
            return far_big(part, res=resf, norm_w=nws)

        def base_sp():
            y = part.clone()
            dist.all_reduce(y)
            r = resf + y
            return (r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + 1e-6) * nws).bfloat16()

        t_sp, t_base = timed(ours_sp), timed(base_sp)
        t_ar = timed(ours_ar) if M <= 1024 else float("nan")
        nv_bytes = (world - 1) / world * M * Hs * (4 + 2)
        roof_us = nv_bytes / (peaks["link_gbs"] * 1e9) * 1e6
        results.append({"case": "seqpar_rs_norm_ag_rows", "M": M, "N": Hs, "tp": world, "ours_us": round(t_sp, 2),
                        "full_row_allreduce_kernel_us": round(t_ar, 2) if t_ar == t_ar else None, "nccl_aten_us": round(t_base, 2),
                        "speedup": round(t_base / t_sp, 2), "roofline_us": round(roof_us, 3),
                        "frac_of_roofline": round(roof_us / t_sp, 3)})
    # ------------------------------------------------------------------ (e) decode-round collectives inside a CUDA graph
    from spark_engine_b200.quant import formats as Q

    def gtimed(fn, n=32, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(n):
                fn()
        gr.replay()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / (reps * n) * 1e3], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    for R in (1, 4, 16):
        far_ll = symm.FusedAllReduce(arena, f"bench_ll{R}", 64, Hs)
        far_fl = symm.FusedAllReduce(arena, f"bench_fl{R}", 64, Hs)
        far_fl.ll_off = -1                                   # the flag format (push, fence, arrival counter, flags, poll)
        xr = torch.randn(R, Hs, device=dev, generator=g).bfloat16()
        rr = torch.zeros(R, Hs, device=dev)
        wq = Q.random_exl3(Hs, 4096 // world, 4, 0, 0.02, 3, dev)
        xo = torch.randn(R, 4096 // world, device=dev, generator=g).bfloat16()

        def nccl_ar():
            y = xr.float()
            dist.all_reduce(y)
            r = rr + y
            return (r * torch.rsqrt(r.pow(2).mean(-1, keepdim=True) + 1e-6) * nws).bfloat16()

        results.append({"case": "graph_decode_allreduce_residual_norm", "rows": R, "N": Hs, "tp": world,
                        "low_latency_us": round(gtimed(lambda: far_ll(xr, res=rr, norm_w=nws)), 2),
                        "flags_us": round(gtimed(lambda: far_fl(xr, res=rr, norm_w=nws)), 2),
                        "nccl_aten_us": round(gtimed(nccl_ar), 2),
                        "exl3_gemv_fused_low_latency_us": round(gtimed(lambda: far_ll.gemv_fused(xo, wq, res=rr, norm_w=nws)), 2),
                        "exl3_gemv_fused_flags_us": round(gtimed(lambda: far_fl.gemv_fused(xo, wq, res=rr, norm_w=nws)), 2),
                        "exl3_gemv_alone_us": round(gtimed(lambda: cu.exl3_gemv(xo, wq)), 2)})
    pk = symm.PacketArgmax(arena, "bench_pk", 64)
    lg = torch.randn(4, 151936 // world, device=dev, generator=g)
    results.append({"case": "graph_decode_packet_argmax", "rows": 4, "vocab": 151936, "tp": world,
                    "ours_us": round(gtimed(lambda: pk(lg, rank * lg.shape[1])), 2),
                    "local_argmax_us": round(gtimed(lambda: cu.argmax(lg)), 2)})
    st = arena.status()
    if rank == 0:
        for r in results:
            print(json.dumps(r))
        print(json.dumps({"device_status": list(st), "world": world, "peaks": peaks}))
    arena.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
