"""Micro-scaled formats on the device (FP8 128x128-block dense, MXFP4 experts, activation quantisers) against
plain fp32 PyTorch on the dequantised weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from spark_engine_b200 import ops
from spark_engine_b200.quant import formats as Q

DEV = "cuda"


def mx():
    from spark_engine_b200.ops import mx as m
    return m


def rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _swiglu(gu, limit):
    F = gu.shape[1] // 2
    g, u = gu[:, :F].float(), gu[:, F:].float()
    if limit > 0:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return torch.nn.functional.silu(g) * u


@pytest.mark.parametrize("fmt", ["fp8", "mxfp4", "mxfp8"])
@pytest.mark.parametrize("R", [1, 3, 4, 8, 13, 16])
@pytest.mark.parametrize("N,K", [(256, 512), (1024, 2048)])
def test_mx_gemv_matches_dequant_matmul(fmt, R, N, K):
    if fmt == "mxfp8":
        w = Q.random_mxfp8(N, K, 0.02, 5, DEV)
    else:
        w = (Q.random_fp8_block if fmt == "fp8" else Q.random_mxfp4)(N, K, 0, 0.02, 5, DEV)
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.randn(R, K, device=DEV, generator=g).bfloat16()
    y = mx().gemv(x, w, out_f32=True)
    y2 = mx().gemv(x, w, out_f32=True)
    ref = x.float().cpu() @ w.dequant().t()
    assert torch.equal(y, y2)
    assert rel_err(y.cpu(), ref) < 2e-3          # activations pass through fp16, weights are exact
    # a row's result does not depend on its neighbours
    y1 = mx().gemv(x[:1].contiguous(), w, out_f32=True)
    assert torch.equal(y1[0], y[0])


@pytest.mark.parametrize("fmt", ["fp8", "mxfp4"])
def test_mx_expert_pairs_with_swiglu_input(fmt):
    E, F, H = 6, 256, 512
    mk = Q.random_fp8_block if fmt == "fp8" else Q.random_mxfp4
    wd = mk(H, F, E, 0.02, 9, DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    P = 10
    gu = torch.randn(P, 2 * F, device=DEV, generator=g).bfloat16()
    pe = torch.tensor([0, 5, 2, -1, 3, 3, 1, 4, -1, 0], dtype=torch.int32, device=DEV)
    y = mx().gemv(gu, wd, items=P, rows_per_item=1, pair_expert=pe, act=1, limit=7.0, out_f32=True)
    # the serving entry point: MXFP4 pairs go through the block-scaled tensor-core kernel, which quantises the
    # activations to MXFP8 (3 mantissa bits) on the way in
    y_tc = mx().expert_gemv(gu, wd, P, pe, None, 1, 7.0, True)
    a = _swiglu(gu.cpu(), 7.0)
    for p in range(P):
        e = int(pe[p])
        if e < 0:
            continue
        ref = a[p] @ wd.dequant_expert(e).t()
        assert rel_err(y[p].cpu(), ref) < 3e-3
        assert rel_err(y_tc[p].cpu(), ref) < 5e-2


@pytest.mark.parametrize("fmt", ["fp8", "mxfp4"])
def test_mx_dequant_is_exact(fmt):
    E, N, K = 3, 256, 384
    w = (Q.random_fp8_block if fmt == "fp8" else Q.random_mxfp4)(N, K, E, 0.02, 4, DEV)
    d = mx().dequant_bf16(w)
    for e in range(E):
        assert torch.equal(d[e].float().cpu(), w.dequant_expert(e).bfloat16().float())


def test_mx_prefill_linear_through_tcgen05():
    w = Q.random_fp8_block(512, 1024, 0, 0.02, 6, DEV)
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(200, 1024, device=DEV, generator=g).bfloat16()
    y = ops.linear(x, w)
    ref = x.float().cpu() @ w.dequant().bfloat16().float().t()
    assert rel_err(y.cpu(), ref) < 5e-3


@pytest.mark.parametrize("block,pow2", [(128, False), (128, True), (32, True)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_act_quant_matches_reference(block, pow2, dtype):
    g = torch.Generator(device=DEV).manual_seed(8)
    x = (torch.randn(37, 512, device=DEV, generator=g) * 3).to(dtype)
    q, sc = mx().act_quant(x, block=block, pow2=pow2)
    qr, scr = Q.act_quant_fp8(x.float().cpu(), block=block, pow2=pow2)
    scf = sc.cpu().float() if block == 128 else Q.e8m0_to_float(sc.cpu())
    assert torch.allclose(scf, scr, rtol=1e-6)
    deq = q.cpu().float().view(37, -1, block) * scf.unsqueeze(-1)
    ref = qr.float().view(37, -1, block) * scr.unsqueeze(-1)
    # identical up to round-to-nearest ties of the division on the two devices
    assert (deq - ref).abs().max() <= 0.07 * ref.abs().max()
    assert (deq != ref).float().mean() < 1e-3


def test_mx_model_matches_cpu_runner_on_the_same_weights():
    """A hybrid MoE model in the mx weight format (FP8 dense projections, MXFP4 experts): device prefill and decode
    rows against the CPU fp32 runner on the dequantised weights."""
    from spark_engine_b200.config import qwen3next_style, scaled_down
    from spark_engine_b200.models.build import build_random_model
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import to_device
    from spark_engine_b200.quant.formats import QuantWeight
    cfg = scaled_down(qwen3next_style())
    cfg.weight_format = "mx"
    cfg.mtp_layers = 0
    W = build_random_model(cfg, DEV, 3)
    kinds = set()

    def walk(n):
        if isinstance(n, dict):
            for v in n.values():
                walk(v)
        elif isinstance(n, list):
            for v in n:
                walk(v)
        elif isinstance(n, QuantWeight):
            kinds.add(type(n).__name__)
    walk(W)
    assert kinds == {"Mxfp8Weight", "Mxfp4Weight"}
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    ref_m = Model(cfg, to_device(W, "cpu", torch.float32), n_slots=1, kv_tokens=128)
    ref = ref_m.forward(make_plan([(0, ids, 0)]))
    m = Model(cfg, W, device=DEV, dtype=torch.bfloat16, n_slots=1, kv_tokens=128)
    lg = m.forward(make_plan([(0, ids[:32], 0)], device=DEV)).float().cpu()          # prefill rows (GEMM path)
    # prefill quantises the activations of the dense projections to MXFP8 (3 mantissa bits) for the block-scaled
    # tensor-core GEMM, as the reference's FP8 prefill does; decode rows keep bf16 activations
    assert rel_err(lg, ref[:32]) < 0.12, rel_err(lg, ref[:32])
    rows = [m.forward(make_plan([(0, [ids[t]], t)], device=DEV)).float().cpu()[0] for t in range(32, 40)]   # GEMV path
    assert rel_err(torch.stack(rows), ref[32:]) < 0.12, rel_err(torch.stack(rows), ref[32:])


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 128, 512), (256, 384, 1024), (77, 200, 256), (1000, 640, 2048)])
def test_block_scaled_fp8_gemm_matches_dequantised_product(M, N, K):
    """tcgen05 block-scaled MMA (scales applied by the tensor core) against the fp32 product of the dequantised
    operands: equal up to fp32 summation order."""
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g))          # rows of different magnitude
    w = torch.randn(N, K, generator=g) * 0.05 * torch.exp(torch.randn(N, K // 32, generator=g).repeat_interleave(32, 1))
    wq = Q.Mxfp8Weight.encode(w).to(DEV)
    aq, asf = Q.quant_mxfp8(a)
    c = mx().gemm_mxfp8(aq.to(DEV), asf.to(DEV), wq, out_f32=True)
    torch.cuda.synchronize()
    st = ops.cuda_ops().read_status(torch.device(DEV))
    assert st[0] == 0, st
    ref = Q.dequant_mxfp8(aq, asf).double() @ wq.dequant().double().t()
    assert rel_err(c.cpu().double(), ref) < 1e-5
    assert torch.equal(c, mx().gemm_mxfp8(aq.to(DEV), asf.to(DEV), wq, out_f32=True))


def test_mxfp8_linear_quantises_activations_on_the_device():
    g = torch.Generator().manual_seed(5)
    w = torch.randn(256, 512, generator=g) * 0.05
    wq = Q.Mxfp8Weight.encode(w).to(DEV)
    x = torch.randn(150, 512, generator=g).bfloat16().to(DEV)
    y = ops.linear(x, wq)
    ref = x.float().cpu() @ wq.dequant().t()
    assert rel_err(y.cpu(), ref) < 4e-2              # e4m3 activations: ~2^-4 relative per element, averaged over K
