"""CPU fp32 full-sequence oracles for every layer type the engine serves.

Plain, slow, readable PyTorch.  Each function restates the layer math with configurable
dimensions; kernels and the incremental engine are tested against these.  The math follows the
reference's Python models (reference/qwen38/model.py:46-202, reference/glm53/{kda,mla,dsa,mhc,moe}.py,
reference/ds41/kernel.py:59-181), which hard-code dimensions and cannot be imported without a
checkpoint.  Weights are `[out, in]` matrices; `x @ w.t()` is a projection.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ----------------------------------------------------------------------------- norms / rope
def rms(x: torch.Tensor, w: Optional[torch.Tensor] = None, eps: float = 1e-6, one_plus: bool = False):
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    if w is None:
        return y
    return y * ((1.0 + w) if one_plus else w)


def layer_norm(x, w, b, eps=1e-6):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps) * w + b


def yarn_inv_freq(rot: int, theta: float, factor: float = 1.0, orig_len: int = 262144,
                  beta_fast: float = 32.0, beta_slow: float = 1.0) -> torch.Tensor:
    """Inverse frequencies in fp64; `factor` > 1 applies YaRN's per-band interpolation
    (reference: qwen_qsa.cu:22-29 inv_freq_init_kernel)."""
    half = rot // 2
    inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2 / rot)
    if factor <= 1.0:
        return inv

    def dim_of(n_rot):
        return rot * math.log(orig_len / (n_rot * 2 * math.pi)) / (2 * math.log(theta))

    lo = max(math.floor(dim_of(beta_fast)), 0)
    hi = min(math.ceil(dim_of(beta_slow)), half - 1)
    ramp = ((torch.arange(half, dtype=torch.float64) - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
    return inv / factor * ramp + inv * (1 - ramp)


def rope_neox(x: torch.Tensor, pos: torch.Tensor, rot: int, theta: float, inv: Optional[torch.Tensor] = None):
    """NeoX (half-split) rotary on the first `rot` dims of the last axis; x [T, ..., D], pos [T]."""
    if rot == 0:
        return x
    half = rot // 2
    if inv is None:
        inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2 / rot)
    ang = (pos.to(x.device).double().unsqueeze(1) * inv.to(x.device).unsqueeze(0)).float()
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    cos, sin = ang.cos().view(shape), ang.sin().view(shape)
    x1, x2, rest = x[..., :half], x[..., half:rot], x[..., rot:]
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin, rest), -1)


def causal_conv(x: torch.Tensor, w: torch.Tensor, dilation: int = 1, tail: Optional[torch.Tensor] = None):
    """Depthwise causal conv over time.  x [T, C]; w [C, k] (w[:, -1] multiplies the current step);
    `tail` [(k-1)*dilation, C] = inputs before x (zeros when None)."""
    T, C = x.shape
    k = w.shape[1]
    pad = (k - 1) * dilation
    if tail is None:
        tail = x.new_zeros(pad, C)
    xp = torch.cat((tail, x), 0)
    out = x.new_zeros(T, C)
    for j in range(k):
        out = out + xp[j * dilation: j * dilation + T] * w[:, j]
    return out


# ----------------------------------------------------------------------------- linear attention
def gdn_recurrence(q, k, v, g, beta, S0=None):
    """Gated delta rule, sequential in time.  q,k [T,H,Dk] (already normalised/scaled, one per value
    head), v [T,H,Dv], g [T,H] log-decay, beta [T,H].  State S [H, Dv, Dk].  Returns (o [T,H,Dv], S)."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    S = q.new_zeros(H, Dv, Dk) if S0 is None else S0.clone()
    o = q.new_empty(T, H, Dv)
    for t in range(T):
        S = S * torch.exp(g[t]).view(H, 1, 1)
        vp = beta[t].view(H, 1) * (v[t] - torch.einsum("hvk,hk->hv", S, k[t]))
        S = S + vp.unsqueeze(2) * k[t].unsqueeze(1)
        o[t] = torch.einsum("hvk,hk->hv", S, q[t])
    return o, S


def gdn_layer(x, w: dict, n_k: int, n_v: int, D: int, eps: float = 1e-6):
    """Gated-DeltaNet block (reference/qwen38/model.py:92-122).  x [T, hidden] -> [T, hidden]."""
    T = x.shape[0]
    y = F.silu(causal_conv(x @ w["qkv"].t(), w["conv"]))
    q = y[:, : n_k * D].view(T, n_k, D)
    k = y[:, n_k * D: 2 * n_k * D].view(T, n_k, D)
    v = y[:, 2 * n_k * D:].view(T, n_v, D)
    g = -torch.exp(w["A_log"]) * F.softplus(x @ w["a"].t() + w["dt_bias"])
    beta = torch.sigmoid(x @ w["b"].t())
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + eps) * D ** -0.5
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + eps)
    rep = n_v // n_k
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    o, _ = gdn_recurrence(q, k, v, g, beta)
    z = (x @ w["z"].t()).view(T, n_v, D)
    o = rms(o, w["norm"], eps) * torch.sigmoid(z)
    return o.reshape(T, n_v * D) @ w["o"].t()


def kda_recurrence(q, k, v, lam, beta, S0=None):
    """Kimi-delta-attention recurrence: per-channel log-decay lam [T,H,Dk] applied on the K columns
    of the state h [H,Dv,Dk] (reference/glm53/kda.py:52-77)."""
    T, H, Dk = q.shape
    Dv = v.shape[-1]
    S = q.new_zeros(H, Dv, Dk) if S0 is None else S0.clone()
    o = q.new_empty(T, H, Dv)
    for t in range(T):
        S = S * torch.exp(lam[t]).unsqueeze(1)
        vp = beta[t].view(H, 1) * (v[t] - torch.einsum("hvk,hk->hv", S, k[t]))
        S = S + vp.unsqueeze(2) * k[t].unsqueeze(1)
        o[t] = torch.einsum("hvk,hk->hv", S, q[t])
    return o, S


def kda_layer(x, w: dict, H: int, D: int):
    T = x.shape[0]

    def branch(name):
        return F.silu(causal_conv(x @ w[name].t(), w[name + "_conv"])).view(T, H, D)

    q, k, v = branch("q"), branch("k"), branch("v")
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(x @ w["b"].t())
    g1 = ((x @ w["f_a"].t()) @ w["f_b"].t()).view(T, H, D)
    lam = -5.0 / (1.0 + torch.exp(-torch.exp(w["A_log"]).view(1, H, 1) * (g1 + w["dt_bias"].view(1, H, D))))
    o, _ = kda_recurrence(q, k, v, lam, beta)
    g2 = ((x @ w["g_a"].t()) @ w["g_b"].t()).view(T, H, D)
    o = w["o_norm"] * (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-5)) * torch.sigmoid(g2)
    return o.reshape(T, H * D) @ w["o"].t()


# ----------------------------------------------------------------------------- softmax attention
def block_sparse_mask(score: Optional[torch.Tensor], T: int, block: int, topk: int) -> torch.Tensor:
    """Query p sees `vis=(p+1)//block` complete blocks: all if <= topk else the top-k by score
    (ties -> lowest index), plus the tail tokens vis*block..p (reference/qwen38/model.py:133-152)."""
    mask = torch.zeros(T, T, dtype=torch.bool)
    for p in range(T):
        vis = (p + 1) // block
        if vis:
            if vis <= topk:
                blocks = torch.arange(vis)
            else:
                blocks = stable_topk(score[p, :vis], topk)
            tok = (blocks.unsqueeze(1) * block + torch.arange(block)).flatten()
            mask[p, tok] = True
        mask[p, vis * block: p + 1] = True
    return mask


def stable_topk(v: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest entries; ties resolved toward the lowest index."""
    order = torch.sort(v, descending=True, stable=True).indices
    return order[:k]


def gqa_layer(x, w: dict, pos, n_q: int, n_kv: int, D: int, rope_dim: int, theta: float, inv=None,
              qk_norm: bool = False, gated: bool = False, sparse_topk: int = 0, block: int = 4,
              idx_heads: int = 4, idx_dim: int = 128, eps: float = 1e-6):
    """Softmax GQA block; optional Gemma-RMS q/k norm, sigmoid output gate and block-sparse
    selection driven by an indexer over mean-pooled keys (reference/qwen38/model.py:125-170)."""
    T = x.shape[0]
    qg = (x @ w["q"].t()).view(T, n_q, D * (2 if gated else 1))
    q = qg[..., :D]
    k = (x @ w["k"].t()).view(T, n_kv, D)
    v = (x @ w["v"].t()).view(T, n_kv, D)
    if qk_norm:
        q, k = rms(q, w["q_norm"], eps, True), rms(k, w["k_norm"], eps, True)
    q, k = rope_neox(q, pos, rope_dim, theta, inv), rope_neox(k, pos, rope_dim, theta, inv)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    if sparse_topk:
        qk = x @ w["idx"].t()
        qi = rope_neox(rms(qk[:, : idx_heads * idx_dim].view(T, idx_heads, idx_dim), w["iq_norm"], eps, True),
                       pos, min(rope_dim, idx_dim), theta, inv)
        kr = qk[:, idx_heads * idx_dim:]
        nb = T // block
        score = None
        if nb:
            pooled = kr[: nb * block].view(nb, block, idx_dim).mean(1)
            kc = rope_neox(rms(pooled, w["ik_norm"], eps, True), pos[torch.arange(nb) * block],
                           min(rope_dim, idx_dim), theta, inv)
            score = F.relu(torch.einsum("thd,nd->thn", qi, kc)).sum(1) / math.sqrt(idx_dim)
        mask = block_sparse_mask(score, T, block, sparse_topk)
    rep = n_q // n_kv
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("thd,shd->hts", q, kk) / math.sqrt(D)
    s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
    o = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)
    if gated:
        o = o * torch.sigmoid(qg[..., D:])
    return o.reshape(T, n_q * D) @ w["o"].t()


def dsa_select(x, cq, w: dict, H: int, Di: int, pool: int, topk_pools: int):
    """DSA indexer (reference/glm53/dsa.py:45-96): returns a bool mask [T,T].  Keys are LayerNorm'ed,
    pooled per `pool` tokens with a softmax-gated (gate + APE) mean; scores relu(q.pool)/sqrt(Di)
    weighted per head; a pool is selectable iff its last token <= the query."""
    T = x.shape[0]
    q = (cq @ w["wq_b"].t()).view(T, H, Di)
    k = layer_norm(x @ w["wk"].t(), w["k_ln_w"], w["k_ln_b"])
    gate = x @ w["cgate"].t()                                   # [T, Di]
    hw = (x @ w["weights_proj"].t()) * H ** -0.5                # [T, H]
    nb = T // pool
    mask = torch.zeros(T, T, dtype=torch.bool)
    score = None
    if nb:
        kb = k[: nb * pool].view(nb, pool, Di)
        gb = gate[: nb * pool].view(nb, pool, Di) + w["ape"].view(1, pool, Di)
        pk = (torch.softmax(gb, 1) * kb).sum(1)                 # [nb, Di]
        sc = F.relu(torch.einsum("thd,nd->thn", q, pk) * Di ** -0.5)
        score = torch.einsum("th,thn->tn", hw, sc)
    for p in range(T):
        vis = (p + 1) // pool
        if vis:
            blocks = torch.arange(vis) if vis <= topk_pools else stable_topk(score[p, :vis], topk_pools)
            tok = (blocks.unsqueeze(1) * pool + torch.arange(pool)).flatten()
            mask[p, tok] = True
        mask[p, vis * pool: p + 1] = True
    return mask


def mla_layer(x, w: dict, pos, H: int, D: int, rope_dim: int = 0, theta: float = 1e4, eps: float = 1e-5,
              idx: Optional[dict] = None, sink: bool = False, window: int = 0):
    """Multi-head latent attention (reference/glm53/mla.py:31-65), unabsorbed form:
    cq = rmsnorm(x q_a), q = cq q_b; ckv = rmsnorm(x kv_a) -> kv_b -> per head [k | v].
    Optional decoupled rope key (DeepSeek-style) shared by all heads, DSA mask, attention sink
    (logit added to the denominator only, reference/ds41/kernel.py:142-164) and sliding window
    (window tokens are always visible in addition to the selected ones)."""
    T = x.shape[0]
    cq = rms(x @ w["q_a"].t(), w["q_a_norm"], eps)
    q = (cq @ w["q_b"].t()).view(T, H, D + rope_dim)
    kva = x @ w["kv_a"].t()
    kv_lora = w["kv_b"].shape[1]
    ckv = rms(kva[:, :kv_lora], w["kv_a_norm"], eps)
    kv = (ckv @ w["kv_b"].t()).view(T, H, 2 * D)
    k, v = kv[..., :D], kv[..., D:]
    s = torch.einsum("thd,shd->hts", q[..., :D], k)
    if rope_dim:
        qr = rope_neox(q[..., D:], pos, rope_dim, theta)
        kr = rope_neox(kva[:, kv_lora:].view(T, 1, rope_dim), pos, rope_dim, theta)[:, 0]
        s = s + torch.einsum("thd,sd->hts", qr, kr)
    s = s / math.sqrt(D + rope_dim)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    if idx is not None:
        mask = dsa_select(x, cq, w, idx["heads"], idx["dim"], idx["pool"], idx["topk"])
        if window:
            ar = torch.arange(T)
            mask = mask | ((ar.view(T, 1) - ar.view(1, T) < window) & (ar.view(T, 1) >= ar.view(1, T)))
    s = s.masked_fill(~mask.unsqueeze(0), float("-inf"))
    if sink:
        m = torch.maximum(s.max(-1, keepdim=True).values, w["sink"].view(H, 1, 1))
        e = torch.exp(s - m)
        p = e / (e.sum(-1, keepdim=True) + torch.exp(w["sink"].view(H, 1, 1) - m))
    else:
        p = torch.softmax(s, -1)
    o = torch.einsum("hts,shd->thd", p, v)
    return o.reshape(T, H * D) @ w["o"].t()


# ----------------------------------------------------------------------------- MoE
def route(x, w_gate, top_k: int, kind: str = "softmax", bias: Optional[torch.Tensor] = None,
          scale: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Routers: `softmax` -> top-k -> renormalise (reference/qwen38/model.py:193-195);
    `sigmoid_bias`: select by sigmoid+bias, weights = selected sigmoid renormalised x scale
    (reference/glm53/moe.py:72-82); `sqrt_softplus`: s = sqrt(softplus(logit)), select by s+bias,
    weights s/sum(s) x scale (engine-rs/shim/ds41_ops.cu:375-421).  Ties -> lowest expert id."""
    logits = x @ w_gate.t()
    if kind == "softmax":
        p = torch.softmax(logits, -1)
        sel = p
    elif kind == "sigmoid_bias":
        p = torch.sigmoid(logits)
        sel = p + (bias if bias is not None else 0)
    elif kind == "sqrt_softplus":
        p = torch.sqrt(F.softplus(logits))
        sel = p + (bias if bias is not None else 0)
    else:
        raise ValueError(kind)
    idx = torch.sort(sel, dim=-1, descending=True, stable=True).indices[:, :top_k]
    wts = torch.gather(p, 1, idx)
    wts = wts / wts.sum(-1, keepdim=True).clamp_min(1e-20) * scale
    return wts, idx


def swiglu(g, u, limit: float = 0.0):
    if limit > 0:
        return F.silu(g.clamp(max=limit)) * u.clamp(-limit, limit)
    return F.silu(g) * u


def moe_layer(x, w: dict, top_k: int, kind: str = "softmax", scale: float = 1.0, limit: float = 0.0,
              shared_gate: bool = False):
    """Routed experts combined in slot order + shared expert (reference/qwen38/model.py:173-202)."""
    wts, idx = route(x, w["gate"], top_k, kind, w.get("bias"), scale)
    out = torch.zeros_like(x)
    for slot in range(top_k):
        for t in range(x.shape[0]):
            e = int(idx[t, slot])
            h = swiglu(x[t] @ w["w_gate"][e].t(), x[t] @ w["w_up"][e].t(), limit)
            out[t] = out[t] + wts[t, slot] * (h @ w["w_down"][e].t())
    if "s_gate" in w:
        sh = swiglu(x @ w["s_gate"].t(), x @ w["s_up"].t(), limit) @ w["s_down"].t()
        if shared_gate:
            sh = torch.sigmoid(x @ w["sg"].t()) * sh
        out = out + sh
    return out


def dense_mlp(x, w: dict, limit: float = 0.0):
    return swiglu(x @ w["gate"].t(), x @ w["up"].t(), limit) @ w["down"].t()


# ----------------------------------------------------------------------------- hyper-connections
def hc_gated_mix(X, w: dict, eps: float = 1e-6):
    """Gated hyper-connection site (reference/qwen38/model.py:65-82): X [T,S,D] ->
    (post [T,S] or None, mixed [T,D])."""
    S = X.shape[1]
    n = rms(X, eps=eps) * (1.0 + w["norm"])
    flat = n.flatten(1)
    t = F.silu(flat @ w["down"].t() / S)
    g = torch.sigmoid(t @ w["up"].t()).view_as(n)
    mixed = (g * n).mean(1)
    post = 2 * torch.sigmoid(flat @ w["inject"].t() / S) if "inject" in w else None
    return post, mixed


def sinkhorn(comb: torch.Tensor, iters: int, eps: float = 1e-6):
    """comb [..., S, S] positive; column-normalise, then (iters-1) x (row, column) normalisations
    (reference/glm53/mhc.py:31-60)."""
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(iters - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return comb


def mhc_pre(res, w: dict, iters: int = 20, eps: float = 1e-5):
    """mHC pre: res [T,S,D] -> (layer_in [T,D], post [T,S], comb [T,S,S])."""
    T, S, D = res.shape
    flat = res.flatten(1)
    m = (flat @ w["fn"].t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + eps)
    pre = torch.sigmoid(m[:, :S] * w["scale"][0] + w["base"][:S]) + 1e-6
    post = 2 * torch.sigmoid(m[:, S:2 * S] * w["scale"][1] + w["base"][S:2 * S])
    comb = torch.softmax((m[:, 2 * S:] * w["scale"][2] + w["base"][2 * S:]).view(T, S, S), -1) + 1e-6
    comb = sinkhorn(comb, iters)
    layer_in = rms((pre.unsqueeze(-1) * res).sum(1), w["norm"], eps)
    return layer_in, post, comb


def mhc_post(res, x, post, comb):
    """res'[j] = sum_i comb[i,j] res[i] + post[j] x."""
    return torch.einsum("tij,tid->tjd", comb, res) + post.unsqueeze(-1) * x.unsqueeze(1)


# ----------------------------------------------------------------------------- n-gram embeddings
NGRAM_MULT = (0x9E3779B97F4A7C15, 0xC2B2AE3D27D4EB4F, 0x165667B19E3779F9)


def _wrap64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def ngram_ids(ids: torch.Tensor, n_heads: int, head_rows: int, eos: int = -1,
              mult: Tuple[int, int, int] = NGRAM_MULT) -> torch.Tensor:
    """Hashed bigram / trigram table rows per position (reference/qwen38/model.py:224-242):
    first half of the heads bigram `t0*m0 ^ t1*m1`, second half trigram `... ^ t2*m2` with int64
    wrap-around; tokens before a segment start (EOS) read as `eos`; row = hash mod head_rows +
    head*head_rows."""
    T = ids.shape[0]
    ids = ids.long()
    pos = torch.arange(T)
    eos_pos = torch.where(ids == eos, pos, torch.full_like(pos, -1))
    prev = torch.cat((torch.tensor([-1]), torch.cummax(eos_pos, 0).values[:-1]))
    in_seg = pos - (prev + 1)

    def shifted(s):
        src = pos - s
        val = ids[src.clamp_min(0)]
        return torch.where((in_seg >= s) & (src >= 0), val, torch.full_like(val, eos))

    m = [torch.tensor(_wrap64(v), dtype=torch.int64) for v in mult]
    t0, t1, t2 = shifted(0), shifted(1), shifted(2)
    bi = (t0 * m[0]) ^ (t1 * m[1])
    tri = bi ^ (t2 * m[2])
    half = n_heads // 2
    mixed = torch.stack([bi] * half + [tri] * (n_heads - half), 1)
    return torch.remainder(mixed, head_rows) + torch.arange(n_heads).view(1, -1) * head_rows


def ngram_embed(x, ids, table, w: dict, n_heads: int, eos: int = -1, eps: float = 1e-6):
    """DS-style engram: gather hashed rows, concatenate heads, gate against the hidden state:
    gate = sigmoid(sign(d) sqrt|d|), d = <rms(key), rms(x)>/sqrt(D); out = x + gate * value."""
    head_rows = table.shape[0] // n_heads
    rows = ngram_ids(ids, n_heads, head_rows, eos)
    emb = table[rows].flatten(1).float()                      # [T, heads*dim]
    key = rms(emb @ w["key"].t(), w["norm_k"], eps)
    val = emb @ w["value"].t()
    d = (key * rms(x, w["norm_q"], eps)).sum(-1, keepdim=True) / math.sqrt(x.shape[-1])
    gate = torch.sigmoid(torch.sign(d) * torch.sqrt(d.abs().clamp_min(eps)))
    return x + gate * val


# ----------------------------------------------------------------------------- sampling / speculation
def gumbel_noise(seed: int, position: int, vocab: int) -> torch.Tensor:
    """Noise keyed by (seed, position, vocab id) only, so target and drafter share it and
    speculative sampling stays exact (reference: sampling.rs:1-8,20-97)."""
    from ..spec.sampling import gumbel_noise_ref
    return gumbel_noise_ref(seed, position, vocab)


def greedy_accept(draft: list, target_argmax: list) -> int:
    """Longest prefix of the draft chain that the target reproduces (qwen/spec.rs:89-96):
    target_argmax[i] is the target's prediction after consuming draft[:i]."""
    n = 0
    while n < len(draft) and draft[n] == target_argmax[n]:
        n += 1
    return n
