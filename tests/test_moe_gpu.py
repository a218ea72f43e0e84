"""MoE block on the device (decode pairs path and prefill grouped-GEMM path, dense and EXL3 experts)
against the fp32 reference computed from the dequantised weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from spark_engine_b200 import ops
from spark_engine_b200.config import MoeConfig
from spark_engine_b200.quant import formats as Q

DEV = "cuda"


def _ref(h, w, c):
    """fp32 CPU reference with dequantised experts."""
    wc = {}
    for k, v in w.items():
        if isinstance(v, Q.QuantWeight):
            if v.experts:
                wc[k] = torch.stack([v.dequant_expert(e) for e in range(c.n_experts)])
            else:
                wc[k] = v.dequant()
        else:
            wc[k] = v.float().cpu()
    return ops.moe(h.float().cpu(), wc, c)


def _weights(c, H, fmt, g):
    E, F = c.n_experts, c.ffn
    if fmt == "exl3":
        return {"gate": (torch.randn(E + 1, H, device=DEV, generator=g) * 0.1).bfloat16(),
                "w_gu": Q.random_exl3(2 * F, H, 4, E, 0.05, 1, DEV), "w_down": Q.random_exl3(H, F, 4, E, 0.05, 2, DEV),
                "s_gu": Q.random_exl3(2 * F, H, 4, 0, 0.05, 3, DEV), "s_down": Q.random_exl3(H, F, 4, 0, 0.05, 4, DEV)}
    return {"gate": (torch.randn(E + 1, H, device=DEV, generator=g) * 0.1).bfloat16(),
            "w_gu": (torch.randn(E, 2 * F, H, device=DEV, generator=g) * 0.05).bfloat16(),
            "w_down": (torch.randn(E, H, F, device=DEV, generator=g) * 0.05).bfloat16(),
            "s_gu": (torch.randn(2 * F, H, device=DEV, generator=g) * 0.05).bfloat16(),
            "s_down": (torch.randn(H, F, device=DEV, generator=g) * 0.05).bfloat16()}


@pytest.mark.parametrize("fmt", ["dense", "exl3"])
@pytest.mark.parametrize("R", [3, 300])
def test_moe_block(fmt, R):
    g = torch.Generator(device=DEV).manual_seed(11)
    c = MoeConfig(n_experts=16, top_k=4, ffn=128, router="softmax", shared_gate=True)
    H = 256
    w = _weights(c, H, fmt, g)
    h = torch.randn(R, H, device=DEV, generator=g).bfloat16()
    out = ops.moe(h, w, c)
    torch.cuda.synchronize()
    st = ops.cuda_ops().read_status(torch.device(DEV))
    assert st[0] == 0, st
    ref = _ref(h, w, c)
    err = ((out.float().cpu() - ref).norm() / ref.norm()).item()
    assert err < 2e-2, err
    out2 = ops.moe(h, w, c)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("H,F,R", [(2048, 256, 300), (1024, 512, 77), (4096, 128, 130)])
def test_exl3_prefill_experts_fused_kernel_vs_reconstruct_path(H, F, R):
    """The fused grouped EXL3 kernel (packed trellis -> MMA, clusters along K) against the reconstruct + tcgen05
    path and the fp32 reference."""
    from spark_engine_b200.ops import exl3_moe
    g = torch.Generator(device=DEV).manual_seed(5)
    c = MoeConfig(n_experts=16, top_k=4, ffn=F, router="softmax", shared_gate=True)
    w = _weights(c, H, "exl3", g)
    h = torch.randn(R, H, device=DEV, generator=g).bfloat16()
    outs = []
    for fused in (True, False):
        exl3_moe.EXL3_MOE_FUSED = fused
        try:
            outs.append(ops.moe(h, w, c))
            if fused:
                assert torch.equal(outs[0], ops.moe(h, w, c))
        finally:
            exl3_moe.EXL3_MOE_FUSED = True
    torch.cuda.synchronize()
    ref = _ref(h, w, c)
    for o in outs:
        err = ((o.float().cpu() - ref).norm() / ref.norm()).item()
        assert err < 2e-2, err
    assert ((outs[0].float() - outs[1].float()).norm() / outs[1].float().norm()).item() < 1e-2


@pytest.mark.parametrize("H,F,R", [(512, 256, 300), (1024, 128, 77), (256, 384, 40)])
def test_mxfp4_prefill_experts_fused_kernel_vs_dequant_path(H, F, R):
    """Fused grouped MXFP4 kernel (packed experts -> MMA fragments) against the dequantise + tcgen05 path and the
    fp32 reference."""
    from spark_engine_b200.ops import mx
    g = torch.Generator(device=DEV).manual_seed(6)
    c = MoeConfig(n_experts=16, top_k=4, ffn=F, router="sqrt_softplus", route_scale=1.5, swiglu_limit=10.0, n_shared=0)
    w = {"gate": (torch.randn(16, H, device=DEV, generator=g) * 0.1).bfloat16(), "bias": torch.zeros(16, device=DEV),
         "w_gu": Q.random_mxfp4(2 * F, H, 16, 0.05, 1, DEV), "w_down": Q.random_mxfp4(H, F, 16, 0.05, 2, DEV)}
    h = torch.randn(R, H, device=DEV, generator=g).bfloat16()
    outs = []
    mx.MX_MOE_TC = mx.MX_DECODE_TC = False           # bf16-activation paths first
    try:
        for fused in (True, False):
            mx.MX_MOE_FUSED = fused
            outs.append(ops.moe(h, w, c))
            if fused:
                assert torch.equal(outs[0], ops.moe(h, w, c))
    finally:
        mx.MX_MOE_FUSED = True
        mx.MX_MOE_TC = mx.MX_DECODE_TC = True
    ref = _ref(h, w, c)
    for o in outs:
        err = ((o.float().cpu() - ref).norm() / ref.norm()).item()
        assert err < 2e-2, err
    # block-scaled tensor-core path: same experts, activations quantised to MXFP8 on the way in
    tc = ops.moe(h, w, c)
    assert torch.equal(tc, ops.moe(h, w, c))
    err = ((tc.float().cpu() - ref).norm() / ref.norm()).item()
    assert err < 6e-2, err
    assert ops.cuda_ops().read_status(torch.device(DEV))[0] == 0


@pytest.mark.parametrize("mode", ["tiles", "pairs"])
@pytest.mark.parametrize("N,K", [(256, 128), (512, 1024), (128, 4096)])
def test_grouped_mxfp4_tensor_core_gemm_matches_dequantised_product(mode, N, K):
    """tcgen05 block-scaled grouped GEMM (MXFP8 activations x packed MXFP4 experts, scales applied by the tensor
    core) against the fp32 product of the dequantised operands, for expert-sorted tiles and for (token, expert)
    pairs."""
    from spark_engine_b200.ops import mx
    E = 6
    w = Q.random_mxfp4(N, K, E, 0.05, 3, DEV)
    g = torch.Generator(device=DEV).manual_seed(9)
    if mode == "tiles":
        counts = [150, 0, 3, 17, 128, 40]                    # rows per expert, in expert order
        P = sum(counts)
        x = (torch.randn(P, K, device=DEV, generator=g) * torch.exp(torch.randn(P, 1, device=DEV, generator=g))).bfloat16()
        tl, r0 = [], 0
        for e, n in enumerate(counts):
            for a in range(r0, r0 + n, 128):
                tl.append([a, r0 + n, e, 0])
            r0 += n
        max_items = len(tl) + 3
        tiles = torch.tensor(tl + [[0, 0, 0, 0]] * 3, dtype=torch.int32, device=DEV)
        ntile = torch.tensor([len(tl)], dtype=torch.int32, device=DEV)
        y = mx.moe_mxfp4_tc(x, w, P, max_items, tiles=tiles, ntile=ntile, out_f32=True)
        rows = [(p, p, e) for e, n in enumerate(counts) for p in range(sum(counts[:e]), sum(counts[:e]) + n)]
    else:
        T, P = 4, 10
        x = torch.randn(T, K, device=DEV, generator=g).bfloat16()
        pe = torch.tensor([0, 5, 2, -1, 3, 3, 1, 4, -1, 0], dtype=torch.int32, device=DEV)
        pr = torch.tensor([0, 0, 1, 1, 2, 3, 3, 2, 0, 1], dtype=torch.int32, device=DEV)
        y = mx.moe_mxfp4_tc(x, w, P, P, pair_expert=pe, pair_row=pr, out_f32=True)
        rows = [(p, int(pr[p]), int(pe[p])) for p in range(P) if int(pe[p]) >= 0]
    torch.cuda.synchronize()
    assert ops.cuda_ops().read_status(torch.device(DEV))[0] == 0
    aq, asf = mx.act_quant(x, block=32)
    xd = Q.dequant_mxfp8(aq.cpu(), asf.cpu()).double()
    for out_row, a_row, e in rows:
        ref = xd[a_row] @ w.dequant_expert(e).double().t()
        err = ((y[out_row].cpu().double() - ref).norm() / ref.norm().clamp_min(1e-12)).item()
        assert err < 1e-5, (out_row, a_row, e, err)
