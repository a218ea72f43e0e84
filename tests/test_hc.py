"""Hyper-connection models (gated HC, mHC): the runner's fused sites (previous block's write-back + this block's mixed
row in one pass) against the fp32 oracle model on CPU, and the CUDA site kernels against the oracle layer math."""
import pytest
import torch

from spark_engine_b200.config import tiny_hybrid
from spark_engine_b200.models.model import Model
from spark_engine_b200.models.plan import make_plan
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.oracle import layers as L
from spark_engine_b200.oracle import model as oracle


def _cfg(kind):
    cfg = tiny_hybrid()
    cfg.hc_kind, cfg.hc_streams, cfg.hc_rank, cfg.mtp_layers = kind, 4, 32, 0
    return cfg


@pytest.mark.parametrize("kind", ["gated", "mhc"])
def test_hc_model_matches_the_oracle_on_cpu(kind):
    cfg = _cfg(kind)
    W = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (24,), generator=g)
    ref = oracle.forward(cfg, W, ids)
    m = Model(cfg, W, n_slots=1, kv_tokens=64)
    got = m.forward(make_plan([(0, ids[:16].tolist(), 0)]))
    got2 = m.forward(make_plan([(0, ids[16:].tolist(), 16)]))
    assert (torch.cat((got, got2)) - ref).abs().max() < 2e-4


@pytest.mark.gpu
def test_mhc_site_kernel_matches_the_oracle():
    from spark_engine_b200.ops import cuda as cu
    torch.manual_seed(0)
    T, S, D = 5, 4, 1536
    g = torch.Generator().manual_seed(1)
    w = {"fn": torch.randn(2 * S + S * S, S * D, generator=g) * 0.05, "scale": torch.rand(3, generator=g) + 0.5,
         "base": torch.randn(2 * S + S * S, generator=g) * 0.3, "norm": torch.rand(D, generator=g) + 0.5}
    w = {k: (v.bfloat16().float() if v.dim() == 2 else v) for k, v in w.items()}
    res = torch.randn(T, S, D, generator=g)
    x = torch.randn(T, D, generator=g)
    h0, post0, comb0 = L.mhc_pre(res, w, 20, 1e-5)
    res1 = L.mhc_post(res, x, post0, comb0)
    h1, post1, comb1 = L.mhc_pre(res1, w, 20, 1e-5)
    wd = {k: v.cuda() for k, v in w.items()}
    X = res.cuda().contiguous()
    Xn, h, post, comb = cu.mhc_site(X, None, wd, 20, 1e-5)
    assert Xn is X
    assert (h.float().cpu() - h0).abs().max() < 2e-2 * h0.abs().max()
    assert (post.cpu() - post0).abs().max() < 1e-4 and (comb.cpu() - comb0).abs().max() < 1e-4
    assert torch.equal(X.cpu(), res)                     # no pending update: the streams are untouched
    for xdev in (x.cuda(), x.cuda().bfloat16()):
        X = res.cuda().contiguous()
        Xn, h, post2, comb2 = cu.mhc_site(X, (xdev, post, comb), wd, 20, 1e-5)
        tol = 1e-4 if xdev.dtype == torch.float32 else 3e-2
        assert (Xn.cpu() - res1).abs().max() < tol and torch.equal(X.cpu(), res)
        assert (post2.cpu() - post1).abs().max() < tol and (comb2.cpu() - comb1).abs().max() < tol
        assert (h.float().cpu() - h1).abs().max() < 2e-2 * h1.abs().max() + tol
    # final site: update, mean over streams, RMSNorm
    X = res.cuda().contiguous()
    _, hn, mean = cu.mhc_site(X, (x.cuda(), post, comb), None, 0, 1e-5, mode=2, norm=wd["norm"])
    assert (mean.cpu() - res1.mean(1)).abs().max() < 1e-4
    assert (hn.float().cpu() - L.rms(res1.mean(1), w["norm"], 1e-5)).abs().max() < 3e-2
    # run twice: bitwise identical (partials are summed in chunk order by the last CTA)
    Xa, Xb = res.cuda().contiguous(), res.cuda().contiguous()
    a = cu.mhc_site(Xa, (x.cuda(), post, comb), wd, 20, 1e-5)
    b = cu.mhc_site(Xb, (x.cuda(), post, comb), wd, 20, 1e-5)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


@pytest.mark.gpu
def test_gated_hc_site_kernel_matches_the_oracle():
    from spark_engine_b200.ops import cuda as cu
    T, S, D, r = 3, 4, 1024, 32
    g = torch.Generator().manual_seed(2)
    w = {"norm": torch.randn(S, D, generator=g) * 0.1, "down": torch.randn(r, S * D, generator=g) * 0.05,
         "up": torch.randn(S * D, r, generator=g) * 0.3, "inject": torch.randn(S, S * D, generator=g) * 0.05}
    w = {k: (v.bfloat16().float() if k != "norm" else v) for k, v in w.items()}
    res = torch.randn(T, S, D, generator=g)
    x = torch.randn(T, D, generator=g)
    post0, mixed0 = L.hc_gated_mix(res, w, 1e-6)
    res1 = res + post0.unsqueeze(-1) * x.unsqueeze(1)
    post1, mixed1 = L.hc_gated_mix(res1, w, 1e-6)
    wd = {k: v.cuda() for k, v in w.items()}
    X = res.cuda().contiguous()
    _, h, hf, post = cu.hc_gated_site(X, None, wd, 1e-6)
    assert (hf.cpu() - mixed0).abs().max() < 1e-4 and (post.cpu() - post0).abs().max() < 1e-4
    Xn, h, hf, post2 = cu.hc_gated_site(X, (x.cuda(), post), wd, 1e-6)
    assert (Xn.cpu() - res1).abs().max() < 1e-4
    assert (hf.cpu() - mixed1).abs().max() < 1e-4 and (post2.cpu() - post1).abs().max() < 1e-4
    assert (h.float().cpu() - mixed1).abs().max() < 2e-2
    wf = {k: v for k, v in wd.items() if k not in ("inject", "_dev")}
    _, h, hf, none = cu.hc_gated_site(res.cuda().contiguous(), None, wf, 1e-6)
    assert none is None and (hf.cpu() - mixed0).abs().max() < 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["gated", "mhc"])
def test_hc_model_on_the_device_matches_cpu(kind):
    from spark_engine_b200.models.weights import map_weights, to_device
    cfg = _cfg(kind)
    W = init_weights(cfg, seed=0)
    Wr = map_weights(W, lambda t: t.bfloat16().float() if t.dim() >= 2 else t)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    ref = Model(cfg, Wr, n_slots=1, kv_tokens=128).forward(make_plan([(0, ids, 0)]))
    m = Model(cfg, to_device(W, "cuda"), device="cuda", dtype=torch.bfloat16, n_slots=1, kv_tokens=128)
    lg = m.forward(make_plan([(0, ids[:32], 0)], device="cuda"))
    lg2 = torch.cat([m.forward(make_plan([(0, [ids[t]], t)], device="cuda")) for t in range(32, 40)])
    got = torch.cat((lg, lg2)).float().cpu()
    err = (got - ref).norm() / ref.norm()
    assert err < 4e-2, err


@pytest.mark.gpu
def test_ngram_gate_kernel():
    from spark_engine_b200.ops import cuda as cu
    g = torch.Generator().manual_seed(3)
    R, H = 6, 1024
    x, key, val = (torch.randn(R, H, generator=g) for _ in range(3))
    nk, nq = torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g) + 0.5
    d = (L.rms(key, nk, 1e-6) * L.rms(x, nq, 1e-6)).sum(-1, keepdim=True) / H ** 0.5
    want = x + torch.sigmoid(torch.sign(d) * torch.sqrt(d.abs().clamp_min(1e-6))) * val
    got = cu.ngram_gate(x.cuda().contiguous(), key.cuda(), val.cuda(), nk.cuda(), nq.cuda(), 1e-6)
    assert (got.cpu() - want).abs().max() < 1e-4
