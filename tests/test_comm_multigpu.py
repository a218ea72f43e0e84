"""Peer-memory collectives and fused compute+collective kernels on >= 2 GPUs (child processes, one per GPU,
NCCL only as plumbing and as the reference; NVLS off), plus the bounded-wait timeout path on one GPU."""
import os
import socket

import pytest
import torch

pytestmark = [pytest.mark.gpu]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, what):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", RANK=str(rank),
                      WORLD_SIZE=str(world))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from spark_engine_b200.parallel import symm
    from spark_engine_b200.ops import cuda as cu
    from spark_engine_b200.quant import formats as Q
    dev = torch.device("cuda", rank)
    arena = symm.Arena(256 << 20)
    g = torch.Generator(device=dev).manual_seed(100 + rank)

    def gather(t):
        out = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(out, t.contiguous())
        return out

    def ordered_sum(parts):
        acc = torch.zeros_like(parts[0], dtype=torch.float32)
        for p in parts:
            acc = acc + p.float()
        return acc

    if what in ("allreduce", "all"):
        ar = symm.FusedAllReduce(arena, "ar", 16, 2048)
        for it in range(3):
            x = torch.randn(4, 2048, device=dev, generator=g)
            ref = ordered_sum(gather(x))
            out = ar(x, out_dtype=torch.float32)
            assert torch.equal(out, ref), "one-shot all-reduce is not the rank-ordered sum"
            res = torch.randn(4, 2048, device=dev, generator=torch.Generator(device=dev).manual_seed(7 + it))
            w = torch.rand(2048, device=dev, generator=torch.Generator(device=dev).manual_seed(9)) + 0.5
            r2 = res.clone()
            xb = x.bfloat16()
            outn = ar(xb, res=r2, norm_w=w)
            full = ordered_sum(gather(xb)) + res
            assert torch.equal(r2, full)
            refn = (full * torch.rsqrt(full.pow(2).mean(-1, keepdim=True) + 1e-6) * w)
            assert ((outn.float() - refn).norm() / refn.norm()) < 5e-3
            outs = gather(outn)
            assert all(torch.equal(o, outs[0]) for o in outs), "ranks disagree"
    if what in ("gemv_ar", "all"):
        N, K = 2048, 1024
        w = Q.random_exl3(N, K, 4, 0, 0.05, 300 + rank, dev)
        far = symm.FusedAllReduce(arena, "gemv_ar", 16, N)
        for R in (1, 4):
            x = torch.randn(R, K, device=dev, generator=g).bfloat16()
            res = torch.zeros(R, N, device=dev)
            nw = torch.ones(N, device=dev)
            y_part = cu.exl3_gemv(x, w, out_f32=True)
            full = ordered_sum(gather(y_part))
            out = far.gemv_fused(x, w, res=res, norm_w=nw)
            assert torch.equal(res, full), "fused GEMV + all-reduce differs from GEMV then rank-ordered sum"
            refn = full * torch.rsqrt(full.pow(2).mean(-1, keepdim=True) + 1e-6)
            assert ((out.float() - refn).norm() / refn.norm()) < 5e-3
    if what in ("gemm_rs", "all"):
        M, N, K = 300, 512, 256
        rp = symm.RowParallelGemm(arena, "rp", 512, N)
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        wt = (torch.randn(N, K, device=dev, generator=g) * 0.1).bfloat16()
        part = x.float() @ wt.float().t()
        ref = ordered_sum(gather(part))
        for fused in (True, False):
            out = rp(x, wt, fused=fused).float().clone()
            torch.cuda.synchronize()
            assert ((out - ref).norm() / ref.norm()) < 6e-3, f"fused={fused}"
            outs = gather(out)
            assert all(torch.equal(o, outs[0]) for o in outs)
    if what in ("ag_gemm", "all"):
        rows, K, N = 96, 512, 384
        agg = symm.AllGatherGemm(arena, "agg", rows * world, K)
        xl = torch.randn(rows, K, device=dev, generator=g).bfloat16()
        wt = (torch.randn(N, K, device=dev, generator=g) * 0.1).bfloat16()
        out = agg(xl, wt, out_f32=True)
        ref = torch.cat(gather(xl)).float() @ wt.float().t()
        assert ((out - ref).norm() / ref.norm()) < 1e-4
    if what in ("ep", "all"):
        H, E, k = 1024, 64, 4
        for T in (1, 16, 200):
            ep = symm.ExpertParallel(arena, f"ep{T}", T, H, E, k)
            x = torch.randn(T, H, device=dev, generator=g).bfloat16()
            logits = torch.randn(T, E, device=dev, generator=g)
            wts, ids = ep.dispatch(x, logits)
            # "expert" = identity scaled by (global expert id + 1): checks routing, payload and return addressing
            torch.cuda.synchronize()
            n = int(ep.total.item())
            eglob = ep.expert_local[:n].long() + rank * (E // world)
            y = (ep.a_rows[:n].float() * (eglob + 1).unsqueeze(1) / E).bfloat16()
            ypad = torch.zeros(ep.max_rows, H, dtype=torch.bfloat16, device=dev)
            ypad[:n] = y
            out = ep.combine(ypad, wts, T)
            p = torch.softmax(logits, -1)
            rw, ri = torch.topk(p, k, -1)
            rw = rw / rw.sum(-1, keepdim=True)
            assert torch.equal(ids.long().sort(-1).values, ri.sort(-1).values)
            xq, sc = Q.act_quant_fp8(x.float().cpu(), 128)
            xd = (xq.float().view(T, H // 128, 128) * sc.unsqueeze(-1)).view(T, H).to(dev)
            ref = torch.zeros(T, H, device=dev)
            for j in range(k):
                ref += wts[:, j:j + 1] * (xd * ((ids[:, j:j + 1].float() + 1) / E)).bfloat16().float()
            assert ((out.float() - ref).norm() / ref.norm()) < 1e-2, T
    torch.cuda.synchronize()
    assert arena.status()[0] == 0, arena.status()
    arena.close()
    dist.destroy_process_group()


@pytest.mark.multigpu
@pytest.mark.parametrize("what", ["allreduce", "gemv_ar", "gemm_rs", "ag_gemm", "ep"])
def test_peer_memory_collectives(what):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_worker, args=(world, _free_port(), what), nprocs=world, join=True)


def test_wait_times_out_with_status_and_context_stays_usable():
    """A flag that nothing sets: the kernel gives up after its budget, records the status, returns."""
    import ctypes as C
    from spark_engine_b200.parallel import symm
    from spark_engine_b200.ops import cuda as cu
    arena = symm.Arena(1 << 20, wait_ms=5.0)
    off = arena.region("never", 32)
    cu.clear_status(arena.device)
    rc = symm._lib()._dll.spark_wait_flags(C.byref(arena.ctx), off, 1, cu.stream())
    assert rc == 0
    torch.cuda.synchronize()
    st = arena.status()
    assert st[0] == 5 and st[2] == 1, st          # ST_TIMEOUT_PEER_FLAG, expected seq 1
    cu.clear_status(arena.device)
    x = torch.ones(4, device=arena.device) * 2      # the context still works
    assert float(x.sum()) == 8.0
    arena.close()
