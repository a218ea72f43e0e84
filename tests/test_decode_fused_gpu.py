"""Decode-round kernels with deferred RMSNorm, residual epilogues, the fused router and device-fed rounds, each
against a plain PyTorch fp32 restatement of the same op."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from spark_engine_b200 import ops
from spark_engine_b200.config import EngineConfig, MoeConfig, qwen3next_style
from spark_engine_b200.models.build import build_random_model
from spark_engine_b200.quant import formats as Q
from spark_engine_b200.serving.engine import LLMEngine

DEV = "cuda"


def cu():
    return ops.cuda_ops()


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def test_gemv_bf16_wide_grid():
    g = torch.Generator(device=DEV).manual_seed(4)
    H, N = 1024, 40003                         # wide, and not a multiple of the 16 weight rows a warp owns
    W = (torch.randn(N, H, device=DEV, generator=g) * 0.05).bfloat16()
    x = torch.randn(13, H, device=DEV, generator=g).bfloat16()
    outs = {}
    for R in (1, 4, 9, 13):
        outs[R] = y = cu().gemv_bf16(x[:R].contiguous(), W, out_f32=True)
        assert rel_err(y, x[:R].float() @ W.float().t()) < 1e-4
        assert torch.isfinite(y).all()
        assert torch.equal(y[0], outs[1][0])                    # a row's logits do not depend on the batch
    yb = cu().gemv_bf16(x[:4].contiguous(), W, out_f32=False)
    assert rel_err(yb, x[:4].float() @ W.float().t()) < 8e-3
    # a reduction too long for 16 staged rows (the n-gram value projection: 16 heads x 1024) stays on the streaming kernel
    W2 = (torch.randn(2048, 16384, device=DEV, generator=g) * 0.02).bfloat16()
    x2 = torch.randn(4, 16384, device=DEV, generator=g).bfloat16()
    y2 = cu().gemv_bf16(x2, W2, out_f32=True)
    assert rel_err(y2, x2.float() @ W2.float().t()) < 1e-4
    assert torch.equal(cu().gemv_bf16(x2[:1].contiguous(), W2, out_f32=True)[0], y2[0])


@pytest.mark.parametrize("kind,E,k", [("softmax", 512, 10), ("sigmoid_bias", 288, 8), ("sqrt_softplus", 384, 6)])
def test_fused_router_matches_reference(kind, E, k):
    g = torch.Generator(device=DEV).manual_seed(7)
    c = MoeConfig(n_experts=E, top_k=k, router=kind, route_scale=2.5 if kind != "softmax" else 1.0,
                  shared_gate=(kind == "softmax"))
    H, R = 256, 7
    gate = (torch.randn(E + (1 if c.shared_gate else 0), H, device=DEV, generator=g) * 0.1).bfloat16()
    bias = torch.randn(E, device=DEV, generator=g) * 0.01
    h = torch.randn(R, H, device=DEV, generator=g).bfloat16()
    lib = cu().lib()
    ld = (E + 8) // 8 * 8
    for slots, (e_lo, e_hi), (rank, world) in ((k, (0, E), (0, 1)), (k + 1, (E // 4, E // 2), (1, 4))):
        logits = torch.zeros(16, ld, device=DEV)
        counter = torch.zeros(4, dtype=torch.int32, device=DEV)
        wts = torch.zeros(R, slots, device=DEV)
        ids = torch.zeros(R, slots, dtype=torch.int32, device=DEV)
        prow = torch.zeros(R, slots, dtype=torch.int32, device=DEV)
        sg = torch.zeros(R, device=DEV)
        for rep in range(2):               # the arrival counter must be back at zero after a launch
            rc = lib.spark_moe_router_topk(h.data_ptr(), h.stride(0), gate.data_ptr(), gate.stride(0), logits.data_ptr(), ld,
                                           R, H, E, k, cu().ROUTER_KIND[kind], bias.data_ptr(), float(c.route_scale),
                                           int(c.shared_gate), slots, e_hi - e_lo, e_lo, e_hi, rank, world, wts.data_ptr(),
                                           ids.data_ptr(), prow.data_ptr(), sg.data_ptr(), counter.data_ptr(),
                                           torch.cuda.current_stream().cuda_stream)
            assert rc == 0
        torch.cuda.synchronize()
        assert counter[0].item() == 0
        rw, ri, rsg = ops.route(h.float().cpu(), {"gate": gate.float().cpu(), "bias": bias.cpu()}, c)
        loc = torch.where((ri >= e_lo) & (ri < e_hi), ri - e_lo, torch.full_like(ri, -1))
        got = ids[:, :k].long().cpu()
        # same experts per row (order may differ on exact ties only), same weights
        assert torch.equal(got.sort(-1).values, loc.sort(-1).values), kind
        full = torch.where(got >= 0, got + e_lo, got)
        for r in range(R):
            for j in range(k):
                if full[r, j] >= 0:
                    jj = (ri[r] == full[r, j]).nonzero()[0, 0]
                    assert abs(wts[r, j].item() - rw[r, jj].item()) < 2e-3 * abs(rw[r, jj].item()) + 1e-5
        assert prow[:, :k].cpu().tolist() == [[r] * k for r in range(R)]
        if c.shared_gate:
            assert torch.allclose(sg.cpu(), rsg[:, 0], rtol=2e-3, atol=1e-4)
        if slots > k:
            own = [(e_hi - e_lo) if r % world == rank else -1 for r in range(R)]
            assert ids[:, k].cpu().tolist() == own
            want = rsg[:, 0] if c.shared_gate else torch.ones(R)
            assert torch.allclose(wts[:, k].cpu(), want, rtol=2e-3, atol=1e-4)


def _moe_weights(c, H, g, stacked):
    E, F = c.n_experts, c.ffn
    gu, dn = Q.random_exl3(2 * F, H, 4, E + 1, 0.05, 1, DEV), Q.random_exl3(H, F, 4, E + 1, 0.05, 2, DEV)
    gate = (torch.randn(E + 1, H, device=DEV, generator=g) * 0.1).bfloat16()
    s_gu = Q.Exl3Weight(gu.trellis[E], gu.suh[E], gu.svh[E], 4, gu.kind)
    s_dn = Q.Exl3Weight(dn.trellis[E], dn.suh[E], dn.svh[E], 4, dn.kind)
    if stacked:
        return {"gate": gate, "w_gu": gu, "w_down": dn, "s_gu": s_gu, "s_down": s_dn, "shared_in_stack": True}
    sl = lambda w: Q.Exl3Weight(w.trellis[:E].contiguous(), w.suh[:E].contiguous(), w.svh[:E].contiguous(), 4, w.kind)
    return {"gate": gate, "w_gu": sl(gu), "w_down": sl(dn), "s_gu": s_gu, "s_down": s_dn}


def test_shared_expert_as_a_pair_and_deferred_combine():
    g = torch.Generator(device=DEV).manual_seed(11)
    c = MoeConfig(n_experts=16, top_k=4, ffn=128, router="softmax", shared_gate=True)
    H, R = 256, 5
    h = torch.randn(R, H, device=DEV, generator=g).bfloat16()
    ws = _moe_weights(c, H, torch.Generator(device=DEV).manual_seed(12), True)
    wp = _moe_weights(c, H, torch.Generator(device=DEV).manual_seed(12), False)
    a = ops.moe(h, ws, c)                       # shared expert = pair of the stack
    b = ops.moe(h, wp, c)                       # shared expert = two separate GEMVs
    assert rel_err(a, b) < 1e-2
    # fp32 reference from the dequantised weights
    wc = {"gate": wp["gate"].float().cpu(),
          "w_gu": torch.stack([wp["w_gu"].dequant_expert(e) for e in range(16)]),
          "w_down": torch.stack([wp["w_down"].dequant_expert(e) for e in range(16)]),
          "s_gu": wp["s_gu"].dequant(), "s_down": wp["s_down"].dequant()}
    ref = ops.moe(h.float().cpu(), wc, c)
    assert rel_err(a.cpu(), ref) < 2e-2
    # deferred: the expert outputs are combined inside the residual update + RMSNorm launch
    cm = cu()
    res = torch.randn(R, H, device=DEV, generator=g)
    wn = torch.rand(H, device=DEV, generator=g) + 0.5
    pend = ops.moe(h, ws, c, defer=True)
    hn, res2 = cm.add_rmsnorm(pend, res.clone(), wn, 1e-6)
    assert rel_err((res2 - res).cpu(), ref) < 2e-2
    want = res2 * torch.rsqrt(res2.pow(2).mean(-1, keepdim=True) + 1e-6) * wn
    assert rel_err(hn, want) < 5e-3
    # and on its own: same sum as the fused launch added
    assert rel_err(pend.tensor().float(), (res2 - res)) < 1e-2


def _small_model():
    cfg = qwen3next_style(n_layers=4)
    cfg.moe.n_experts, cfg.vocab, cfg.mtp_layers = 32, 4096, 0
    return cfg, build_random_model(cfg, DEV, seed=0)


def test_fused_decode_round_matches_the_unfused_kernels():
    cfg, W = _small_model()
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab, (2, 96), generator=g).tolist()
    c = cu()
    logits = {}
    for fused in (True, False):
        c.FUSED_DECODE = fused
        try:
            eng = LLMEngine(cfg, W, EngineConfig(cuda_graphs=False), max_seqs=2, kv_tokens_per_seq=256)
            cur = [int(eng.model.greedy(eng.prefill(s, p).unsqueeze(0))[0]) for s, p in enumerate(prompts)]
            from spark_engine_b200.models.plan import make_plan
            lg = []
            for step in range(4):
                plan = make_plan([(s, [cur[s]], 96 + step) for s in range(2)], device=DEV)
                out = eng.model.forward(plan)
                lg.append(out.float().clone())
                cur = out.argmax(-1).tolist()
            logits[fused] = torch.stack(lg)
        finally:
            c.FUSED_DECODE = True
    torch.cuda.synchronize()
    assert c.read_status(torch.device(DEV))[0] == 0
    assert rel_err(logits[True], logits[False]) < 2e-2


def test_device_fed_steps_equal_host_fed_rounds():
    cfg, W = _small_model()
    g = torch.Generator().manual_seed(6)
    prompts = torch.randint(0, cfg.vocab, (2, 80), generator=g).tolist()
    outs = []
    for fed in (False, True):
        eng = LLMEngine(cfg, W, EngineConfig(cuda_graphs=True), max_seqs=2, kv_tokens_per_seq=256)
        cur = [int(eng.model.greedy(eng.prefill(s, p).unsqueeze(0))[0]) for s, p in enumerate(prompts)]
        toks = []
        if fed:
            first = eng.decode_steps([0, 1], cur, 3)            # captures the round, then replays with device feedback
            toks = first + eng.decode_steps([0, 1], first[-1], 4)
            cur = toks[-1]
            for _ in range(2):                                  # plain rounds after fed replays read their own outputs
                cur = eng.decode_round([0, 1], cur)
                toks.append(cur)
        else:
            for _ in range(9):
                cur = eng.decode_round([0, 1], cur)
                toks.append(cur)
        assert [eng.model.seqs[s].length for s in (0, 1)] == [89, 89]
        outs.append(toks)
    assert outs[0] == outs[1]


@pytest.mark.parametrize("D,Hq,Hkv,fp8", [(256, 16, 2, False), (128, 8, 8, False), (64, 4, 2, True), (256, 16, 2, True)])
def test_decode_attention_tensor_core_kernel(D, Hq, Hkv, fp8):
    """Split-KV decode attention (dense context, selected-token lists, tree ancestor masks, FP8 KV) against fp32 softmax
    attention over the same cache contents."""
    import math
    g = torch.Generator(device=DEV).manual_seed(9)
    c = cu()
    lib = c.lib()
    tokens, R = 700, 5
    kv_base = torch.tensor([0, 0, 0, 300, 300], dtype=torch.int64, device=DEV)       # two sequences
    pos0 = torch.tensor([200, 200, 200, 310, 310], dtype=torch.int32, device=DEV)     # first in-flight position
    row_j = torch.tensor([0, 1, 2, 0, 1], dtype=torch.int32, device=DEV)
    pos = pos0 + row_j
    K = torch.randn(tokens, Hkv, D, device=DEV, generator=g)
    V = torch.randn(tokens, Hkv, D, device=DEV, generator=g)
    q = torch.randn(R, Hq, D, device=DEV, generator=g).bfloat16()
    if fp8:
        ks = K.abs().amax(-1).clamp_min(1e-8) / 448.0
        vs = V.abs().amax(-1).clamp_min(1e-8) / 448.0
        Kc, Vc = (K / ks.unsqueeze(-1)).to(torch.float8_e4m3fn), (V / vs.unsqueeze(-1)).to(torch.float8_e4m3fn)
        Kd, Vd = Kc.float() * ks.unsqueeze(-1), Vc.float() * vs.unsqueeze(-1)
    else:
        ks = vs = None
        Kc, Vc = K.bfloat16(), V.bfloat16()
        Kd, Vd = Kc.float(), Vc.float()
    rep = Hq // Hkv
    scale = 1.0 / math.sqrt(D)
    qkv = torch.zeros(R, 8, device=DEV).bfloat16()

    def run(sel=None, sel_n=None, tree=False, anc=None, max_ctx=None, chunks=1):
        nsplit = ((max_ctx + 63) // 64 + chunks - 1) // chunks
        part_o = torch.empty(R * Hq * nsplit * D, device=DEV)
        part_ml = torch.empty(R * Hq * nsplit * 2, device=DEV)
        out = torch.empty(R, Hq * D, dtype=torch.bfloat16, device=DEV)
        rc = lib.spark_attn_decode(q.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), c.P(ks), c.P(vs), int(fp8), pos.data_ptr(),
                                   kv_base.data_ptr(), c.P(sel), c.P(sel_n), 0 if sel is None else sel.shape[1], part_o.data_ptr(),
                                   part_ml.data_ptr(), nsplit, qkv.data_ptr(), qkv.stride(0), 0, R, Hq, Hkv, D, scale,
                                   out.data_ptr(), c.stream(), pos0.data_ptr() if tree else None,
                                   row_j.data_ptr() if tree else None, c.P(anc), chunks)
        assert rc == 0
        return out.float().view(R, Hq, D)

    def ref(visible):                           # visible: list of token-index tensors per row
        o = torch.empty(R, Hq, D, device=DEV)
        for r in range(R):
            idx = visible[r] + int(kv_base[r])
            kk = Kd[idx].repeat_interleave(rep, 1)          # [n, Hq, D]
            vv = Vd[idx].repeat_interleave(rep, 1)
            sc = torch.einsum("hd,nhd->hn", q[r].float(), kk) * scale
            o[r] = torch.einsum("hn,nhd->hd", torch.softmax(sc, -1), vv)
        return o

    # dense causal context
    got = run(max_ctx=int(pos.max()) + 1)
    want = ref([torch.arange(int(p) + 1, device=DEV) for p in pos])
    assert rel_err(got, want) < 2e-2
    # selected-token lists of different lengths
    sel_n = torch.tensor([70, 129, 64, 5, 200], dtype=torch.int32, device=DEV)
    sel = torch.zeros(R, 200, dtype=torch.int32, device=DEV)
    vis = []
    for r in range(R):
        ch = torch.randperm(int(pos[r]) + 1, device=DEV, generator=g)[: int(sel_n[r])].sort().values
        sel[r, : int(sel_n[r])] = ch.int()
        vis.append(ch)
    got = run(sel=sel, sel_n=sel_n, max_ctx=200)
    assert rel_err(got, ref(vis)) < 2e-2
    # several 64-token tiles per split with a running softmax (what prefill-size batches use): 2 tiles per split, and
    # the whole row in one split
    for chunks in (2, 4):
        got = run(sel=sel, sel_n=sel_n, max_ctx=200, chunks=chunks)
        assert rel_err(got, ref(vis)) < 2e-2, chunks
    got = run(max_ctx=int(pos.max()) + 1, chunks=(int(pos.max()) + 64) // 64)
    assert rel_err(got, want) < 2e-2
    # tree rows: sequence 0 has three in-flight rows, row 2 is a sibling of row 1 (both children of row 0)
    anc = torch.tensor([0b001, 0b011, 0b101, 0b01, 0b11], dtype=torch.int32, device=DEV)
    got = run(tree=True, anc=anc, max_ctx=int((pos0 + row_j).max()) + 1)
    vis = []
    for r in range(R):
        own = [j for j in range(3) if (int(anc[r]) >> j) & 1]
        vis.append(torch.cat((torch.arange(int(pos0[r]), device=DEV), torch.tensor(own, device=DEV) + int(pos0[r]))))
    assert rel_err(got, ref(vis)) < 2e-2
    torch.cuda.synchronize()
    assert c.read_status(torch.device(DEV))[0] == 0


def test_gumbel_perturb_kernel_matches_the_host_oracle():
    """Device Gumbel noise (hash of seed, position, GLOBAL vocabulary id) against the fp32 host formula, for a
    vocabulary slice that starts at a non-zero offset; greedy rows stay untouched; the sampled tokens agree."""
    from spark_engine_b200.spec.sampling import gumbel_noise_ref
    torch.manual_seed(3)
    R, V, off, vocab = 5, 37_991, 75_982, 151_964
    lg = torch.randn(R, V, device="cuda") * 3
    temps, seeds, poss = [0.7, 0.0, 1.3, 0.0, 0.2], [11, 12, 2 ** 40 + 5, 14, 15], [0, 5, 123456, 7, 2 ** 33]
    got = ops.gumbel_perturb(lg, temps, seeds, poss, off, vocab)
    want = lg.clone()
    for r, T in enumerate(temps):
        if T > 0:
            want[r] = lg[r] / T + gumbel_noise_ref(seeds[r], poss[r], vocab, "cuda")[off: off + V]
    assert got.data_ptr() != lg.data_ptr()
    assert torch.equal(got[1], lg[1]) and torch.equal(got[3], lg[3])
    assert (got - want).abs().max().item() < 1e-4
    assert ops.argmax(got).tolist() == want.argmax(-1).tolist()


def test_checked_mode_rejects_bad_tables_before_launch(monkeypatch):
    """SPARK_CHECK: an expert id or a token id outside its table raises in Python and nothing is launched (the device
    status word stays clear and the context stays usable); valid tables pass; poisoned scratch does not leak into
    results."""
    from spark_engine_b200.utils import debug as dbg
    monkeypatch.setattr(dbg, "CHECK", True)
    monkeypatch.setattr(dbg, "POISON", True)
    g = torch.Generator(device=DEV).manual_seed(9)
    E, N, K = 4, 64, 128
    # views of larger allocations: should a check ever miss, the launch would still read memory that exists
    w = (torch.randn(E + 2, N, K, device=DEV, generator=g) * 0.05).bfloat16()[:E]
    x = torch.randn(4, K, device=DEV, generator=g).bfloat16()[:2]
    rows = torch.tensor([0, 1, 1], dtype=torch.int32, device=DEV)
    good = torch.tensor([3, 0, -1], dtype=torch.int32, device=DEV)
    y = cu().gemv_bf16(x, w, items=3, rows_per_item=1, pair_expert=good, pair_row=rows, out_f32=True, expert_stride=N * K, n=N, k=K)
    assert rel_err(y[0], x[0].float() @ w[3].float().t()) < 1e-4
    bad = torch.tensor([3, 4, 0], dtype=torch.int32, device=DEV)
    with pytest.raises(dbg.IndexTableError):
        cu().gemv_bf16(x, w, items=3, rows_per_item=1, pair_expert=bad, pair_row=rows, out_f32=True, expert_stride=N * K, n=N, k=K)
    with pytest.raises(dbg.IndexTableError):
        cu().gemv_bf16(x, w, items=3, rows_per_item=1, pair_expert=good, pair_row=rows + 1, out_f32=True, expert_stride=N * K, n=N, k=K)
    table = torch.randn(52, 64, device=DEV).bfloat16()[:50]
    with pytest.raises(dbg.IndexTableError):
        cu().embed(table, torch.tensor([1, 50], dtype=torch.int32, device=DEV))
    torch.cuda.synchronize()
    assert cu().read_status(torch.device(DEV))[0] == 0
    # a whole model step under both modes: finite logits, same tokens as the plain run
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights, to_device
    cfg = tiny_hybrid()
    W = to_device(init_weights(cfg, seed=0), DEV)
    ids = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    outs = []
    for on in (True, False):
        monkeypatch.setattr(dbg, "CHECK", on)
        monkeypatch.setattr(dbg, "POISON", on)
        m = Model(cfg, W, device=DEV, dtype=torch.bfloat16, n_slots=1, kv_tokens=256)
        a = m.forward(make_plan([(0, ids[:36], 0)], device=DEV, all_logits=False), commit=True)
        b = m.forward(make_plan([(0, ids[36:40], 36)], device=DEV), commit=True)
        outs.append(torch.cat((a, b)).float())
    assert torch.isfinite(outs[0]).all()
    assert torch.equal(outs[0], outs[1])
    assert dbg.stats["checked"] > 0 and dbg.stats["poisoned"] > 0
