"""Operator layer: one Python entry point per op; the sm_100a kernels run on a B200, plain PyTorch
runs on CPU (fp32 plumbing and oracle tests).

On a CUDA device the kernel library MUST be present: an op whose kernel is missing raises instead of
silently running an eager fallback (set SPARK_ALLOW_TORCH_FALLBACK=1 to run the PyTorch/ATen
baseline path on purpose, e.g. for A/B timing against the library path).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from ..oracle import layers as L
from ..quant.formats import QuantWeight

_FALLBACK = os.environ.get("SPARK_ALLOW_TORCH_FALLBACK", "0") == "1"
_cuda_ops = None


def cuda_ops():
    """The kernel bindings (loaded on first use on a CUDA device)."""
    global _cuda_ops
    if _cuda_ops is None:
        from . import cuda as _c
        _cuda_ops = _c
    return _cuda_ops


def use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and not _FALLBACK


def set_fallback(on: bool):
    """Route CUDA tensors through PyTorch/ATen ops (the library baseline) instead of the kernels."""
    global _FALLBACK
    _FALLBACK = on


# ----------------------------------------------------------------------------- basic ops
def embed(table: torch.Tensor, ids: torch.Tensor, dtype) -> torch.Tensor:
    """Token embedding rows.  On the device the residual stream is fp32 (activations bf16)."""
    if use_kernels(table):
        return cuda_ops().embed(table, ids.to(torch.int32))
    return table[ids].to(dtype)


def to_tensor(x):
    """Plain tensor of a block output that may still be deferred (uncombined MoE of a decode round, row-parallel
    product)."""
    if x is None or isinstance(x, torch.Tensor):
        return x
    if isinstance(x, Partial):
        return linear(x.x, x.w)
    return x.tensor()


def residual_add(res, delta) -> torch.Tensor:
    res, delta = to_tensor(res), to_tensor(delta)
    if use_kernels(res) and res.dtype == torch.float32 and res.dim() == 2:
        return cuda_ops().residual_add(res, delta)
    return res + delta.to(res.dtype)


def argmax(logits: torch.Tensor) -> torch.Tensor:
    """Greedy token per row (ties -> lowest id), int32."""
    if use_kernels(logits):
        return cuda_ops().argmax(logits)
    return torch.argmax(logits, -1).to(torch.int32)


def gumbel_perturb(logits: torch.Tensor, temps, seeds, positions, offset: int, vocab: int) -> torch.Tensor:
    """fp32 logits [R, V_local] of vocabulary ids [offset, offset + V_local): rows with temperature > 0 become
    logits / T + g(seed, position, global id); greedy rows are returned unchanged.  The arg-max of the result (over
    all ranks' slices) is the sampled token.  temps/seeds/positions are Python sequences of length R."""
    if not any(t > 0 for t in temps):
        return logits
    x = logits.float() if logits.dtype != torch.float32 else logits.clone()
    if use_kernels(x):
        dev = x.device
        t = torch.tensor(list(temps), dtype=torch.float32).to(dev, non_blocking=True)
        sd = torch.tensor([int(v) for v in seeds], dtype=torch.int64).to(dev, non_blocking=True)
        ps = torch.tensor([int(v) for v in positions], dtype=torch.int64).to(dev, non_blocking=True)
        return cuda_ops().gumbel_perturb(x.contiguous(), t, sd, ps, offset)
    from ..spec.sampling import gumbel_noise_ref
    V = x.shape[1]
    for r, T in enumerate(temps):
        if T > 0:
            x[r] = x[r] / T + gumbel_noise_ref(int(seeds[r]), int(positions[r]), vocab, x.device)[offset: offset + V]
    return x


def lm_head(h, w) -> torch.Tensor:
    """Logits in fp32."""
    if use_kernels(h) and not isinstance(w, QuantWeight):
        return cuda_ops().dense_linear(h, w, out_f32=True)
    return linear(h, w).float()


def linear(x: torch.Tensor, w) -> torch.Tensor:
    """y = x @ W^T for a dense `[N,K]` tensor or a quantised weight object."""
    if isinstance(w, QuantWeight):
        if use_kernels(x):
            return cuda_ops().quant_linear(x, w)
        return (x.float() @ w.dequant().to(x.device).t()).to(x.dtype)
    if use_kernels(x):
        return cuda_ops().dense_linear(x, w)
    return x @ w.to(x.dtype).t()


def linear_pair(x, w_a, w_b):
    """Two independent projections of the same rows.  On the device, decode-size batches run the second one on a
    side stream next to the first (parallel branches of the captured graph)."""
    if use_kernels(x) and x.shape[0] <= 16 and cuda_ops().SIDE_STREAMS:
        c = cuda_ops()
        main = torch.cuda.current_stream()
        side = c._side_stream(x.device)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            b = linear(x, w_b)
        a = linear(x, w_a)
        main.wait_stream(side)
        return a, b
    return linear(x, w_a), linear(x, w_b)


def rmsnorm(x, w, eps):
    x = to_tensor(x)
    if use_kernels(x):
        return cuda_ops().rmsnorm(x, w, eps)
    return L.rms(x.float(), w.float(), eps).to(x.dtype)


class Partial:
    """A row-parallel product x @ W_shard^T that has not been computed yet: under tensor parallelism the
    GEMV, the all-reduce, the residual add and the next RMSNorm run as one kernel."""

    def __init__(self, x, w):
        self.x, self.w = x, w


def row_parallel(x, w, tp=None):
    """Output projection of a mixer.  Without tensor parallelism: the product.  With it: this rank's partial
    product, deferred when the fused GEMV + all-reduce kernel can take it (EXL3 weights, <= 16 rows)."""
    if tp is not None and tp.can_fuse_gemv(x, w):
        return Partial(x, w)
    return linear(x, w)


def add_rmsnorm(delta, res, w, eps, tp=None):
    """res' = res + delta (delta may be None); returns (rmsnorm(res') * w, res').  With `tp`, delta is this
    rank's partial sum and is all-reduced first (one fused kernel on the device)."""
    if tp is not None and delta is not None:
        return tp.add_rmsnorm(delta, res, w, eps)
    if use_kernels(res):
        return cuda_ops().add_rmsnorm(delta, res, w, eps)
    delta = to_tensor(delta)
    if delta is not None:
        res = res + delta
    return L.rms(res.float(), w.float(), eps).to(res.dtype), res


def swiglu(gu: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    """gu = [gate | up] halves along the last axis."""
    if use_kernels(gu):
        return cuda_ops().swiglu(gu, limit)
    F_ = gu.shape[-1] // 2
    return L.swiglu(gu[..., :F_].float(), gu[..., F_:].float(), limit).to(gu.dtype)


# ----------------------------------------------------------------------------- MoE
def route(h, w, c):
    """Router: returns (weights [R,k] fp32, expert ids [R,k] int64, shared gate [R,1] or None)."""
    logits = linear(h, w["gate"]).float()
    sg = None
    if c.shared_gate:
        sg = torch.sigmoid(logits[:, c.n_experts:])
        logits = logits[:, : c.n_experts]
    if c.router == "softmax":
        p = torch.softmax(logits, -1)
        sel = p
    elif c.router == "sigmoid_bias":
        p = torch.sigmoid(logits)
        sel = p + w["bias"].float().to(p.device)
    else:
        p = torch.sqrt(F.softplus(logits))
        sel = p + w["bias"].float().to(p.device)
    idx = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, : c.top_k]
    wts = torch.gather(p, 1, idx)
    wts = wts / wts.sum(-1, keepdim=True).clamp_min(1e-20) * c.route_scale
    return wts, idx, sg


def moe(h, w, c, defer: bool = False):
    """Routed experts (slot-order weighted sum) + shared expert.  `defer` (decode rounds on the device): the
    uncombined expert outputs are returned and the combine runs fused with the next residual update."""
    if use_kernels(h):
        return cuda_ops().moe(h, w, c, defer)
    R = h.shape[0]
    wts, idx, sg = route(h, w, c)
    out = torch.zeros(R, h.shape[1], dtype=torch.float32, device=h.device)
    hf = h.float()
    wgu, wd = w["w_gu"], w["w_down"]
    lo, hi = w.get("ep", (0, c.n_experts))       # expert-parallel rank: only its own experts, partial output
    for slot in range(c.top_k):
        for e in idx[:, slot].unique().tolist():
            if not lo <= e < hi:
                continue
            rows = (idx[:, slot] == e).nonzero(as_tuple=True)[0]
            gu = hf[rows] @ _expert(wgu, e - lo).t()
            y = L.swiglu(gu[:, : c.ffn], gu[:, c.ffn:], c.swiglu_limit) @ _expert(wd, e - lo).t()
            out[rows] += wts[rows, slot].unsqueeze(1) * y
    if "s_gu" in w:
        gu = linear(h, w["s_gu"]).float()
        Fs = gu.shape[1] // 2
        sh = linear(L.swiglu(gu[:, :Fs], gu[:, Fs:], c.swiglu_limit).to(h.dtype), w["s_down"]).float()
        out = out + (sg * sh if sg is not None else sh)
    return out.to(h.dtype)


def _expert(w, e):
    if isinstance(w, QuantWeight):
        return w.dequant_expert(e)
    return w[e].float()


# ----------------------------------------------------------------------------- mixers (fast paths)
def gdn_mixer(mixer, proj, ab, plan, commit) -> Optional[torch.Tensor]:
    if use_kernels(proj):
        return cuda_ops().gdn_mixer(mixer, proj, ab, plan, commit)
    return None


def gdn_commit(mixer, proj, ab, plan, accepted) -> bool:
    if use_kernels(proj):
        return cuda_ops().gdn_commit(mixer, proj, ab, plan, accepted)
    return False


def kda_mixer(mixer, pre, lr, plan, commit) -> Optional[torch.Tensor]:
    if use_kernels(pre):
        return cuda_ops().kda_mixer(mixer, pre, lr, plan, commit)
    return None


def kda_commit(mixer, pre, lr, plan, accepted) -> bool:
    if use_kernels(pre):
        return cuda_ops().kda_commit(mixer, pre, lr, plan, accepted)
    return False


def mla_mixer(mixer, h, plan, seqs) -> Optional[torch.Tensor]:
    if use_kernels(h):
        return cuda_ops().mla_mixer(mixer, h, plan, seqs)
    return None


def attn_mixer(mixer, qkv, plan, seqs) -> Optional[torch.Tensor]:
    if use_kernels(qkv):
        return cuda_ops().attn_mixer(mixer, qkv, plan, seqs)
    return None


# ----------------------------------------------------------------------------- hyper-connections
def _reduced(x, tp):
    """Block output as a plain tensor; under tensor parallelism this rank's partial sum is all-reduced first."""
    if x is None:
        return None
    if tp is not None:
        return tp.reduce(x)
    return to_tensor(x)


def hc_gated_site(X, pend, w, eps, tp=None):
    """Gated hyper-connection site.  `pend` = (block output, post) of the previous site, applied to the streams first:
    X[:, s] += post[:, s] * x.  Returns (X, mixed row h, hidden copy in fp32 or None, post for this site's block)."""
    if pend is not None:
        pend = (_reduced(pend[0], tp), pend[1])
    if use_kernels(X) and X.shape[1] == 4 and w["down"].shape[0] == 32 and X.dtype == torch.float32:
        return cuda_ops().hc_gated_site(X, pend, w, eps)
    if pend is not None:
        X = X + pend[1].unsqueeze(-1).to(X.dtype) * pend[0].to(X.dtype).unsqueeze(1)
    post, mixed = L.hc_gated_mix(X.float(), {k: v.float() for k, v in w.items() if torch.is_tensor(v)}, eps)
    return X, mixed.to(X.dtype), None, post


def mhc_site(X, pend, w, iters, eps, tp=None):
    """mHC site.  `pend` = (block output, post, comb) of the previous site, applied first.  Returns (X, h, post, comb)."""
    if pend is not None:
        pend = (_reduced(pend[0], tp),) + tuple(pend[1:])
    if use_kernels(X) and X.shape[1] == 4 and X.dtype == torch.float32:
        return cuda_ops().mhc_site(X, pend, w, iters, eps)
    if pend is not None:
        X = L.mhc_post(X.float(), pend[0].float(), pend[1], pend[2]).to(X.dtype)
    h, post, comb = L.mhc_pre(X.float(), {k: v.float() for k, v in w.items() if torch.is_tensor(v)}, iters, eps)
    return X, h.to(X.dtype), post, comb


def mhc_final(X, pend, norm_w, eps, tp=None):
    """Last update, then the mean over streams and its RMSNorm.  Returns (hidden fp32-or-input dtype [T,D], normed row)."""
    if pend is not None:
        pend = (_reduced(pend[0], tp),) + tuple(pend[1:])
    if use_kernels(X) and X.shape[1] == 4 and X.dtype == torch.float32:
        _, h, mean = cuda_ops().mhc_site(X, pend, None, 0, eps, mode=2, norm=norm_w)
        return mean, h
    if pend is not None:
        X = L.mhc_post(X.float(), pend[0].float(), pend[1], pend[2]).to(X.dtype)
    m = X.mean(1)
    return m, rmsnorm(m, norm_w, eps)


def ngram_embed(model, X, plan, w):
    """Hashed n-gram rows need the token history of each sequence: the model keeps it per slot."""
    from ..models.ngram import ngram_rows_for_plan
    cfg = model.cfg
    emb = ngram_rows_for_plan(model, plan)                   # [R, heads*dim] fp32 on X.device
    if use_kernels(X):                                       # the two projections on the GEMV / tcgen05 GEMM kernels
        eb = emb.to(torch.bfloat16)
        key_raw = linear(eb, w["key"]).float()
        val = linear(eb, w["value"]).float()
    else:
        key_raw = emb @ w["key"].float().t()
        val = emb @ w["value"].float().t()
    if use_kernels(X) and X.dtype == torch.float32 and X.dim() == 2:
        return cuda_ops().ngram_gate(X.contiguous(), key_raw, val, w["norm_k"], w["norm_q"], cfg.norm_eps)
    key = L.rms(key_raw, w["norm_k"].float(), cfg.norm_eps)
    d = (key * L.rms(X.float(), w["norm_q"].float(), cfg.norm_eps)).sum(-1, keepdim=True) / math.sqrt(X.shape[-1])
    gate = torch.sigmoid(torch.sign(d) * torch.sqrt(d.abs().clamp_min(cfg.norm_eps)))
    return (X.float() + gate * val).to(X.dtype)
