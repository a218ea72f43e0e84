"""Seed-determined sampling that keeps speculative decoding exact.

Gumbel-max: token = argmax_v (logit_v / T + g_v) with g_v = -log(-log u_v) and u_v a hash of
(seed, position, vocab id) only.  Target and drafter draw the SAME noise for a position, so "the drafter's pick
equals the target's pick" is a deterministic comparison exactly as in greedy decoding, and the emitted text
depends only on (model, prompt, seed).  Under vocabulary parallelism each rank reduces its slice to one
(value, index) packet and the packets are combined (ties -> lowest index).
Reference: engine-rs/src/sampling.rs:1-8,20-170, head_select.rs:1-101, shim/latent.cu:840-940.
"""
from __future__ import annotations

import torch

_M1, _M2, _M3 = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_MASK = (1 << 64) - 1


def _mix64(x: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on int64 tensors (wrap-around arithmetic)."""
    def c(v):
        v &= _MASK
        return v - (1 << 64) if v >= (1 << 63) else v
    x = (x ^ ((x >> 30) & ((1 << 34) - 1))) * c(_M2)
    x = (x ^ ((x >> 27) & ((1 << 37) - 1))) * c(_M3)
    return x ^ ((x >> 31) & ((1 << 33) - 1))


def uniform_ref(seed: int, position: int, vocab: int, device="cpu") -> torch.Tensor:
    """u in (0,1), one per vocab id, a pure function of (seed, position, id)."""
    def c(v):
        v &= _MASK
        return v - (1 << 64) if v >= (1 << 63) else v
    ids = torch.arange(vocab, dtype=torch.int64, device=device)
    key = c(seed * _M1) ^ c((position + 1) * _M2)
    h = _mix64(ids * c(_M1) + key)
    top = (h >> 11) & ((1 << 53) - 1)
    return (top.double() + 0.5) / float(1 << 53)


def gumbel_noise_ref(seed: int, position: int, vocab: int, device="cpu") -> torch.Tensor:
    u = uniform_ref(seed, position, vocab, device)
    return (-torch.log(-torch.log(u))).float()


def sample(logits: torch.Tensor, temperature: float, seed: int, position: int) -> int:
    """One token from fp32 logits [V]; temperature 0 = greedy (ties -> lowest id)."""
    if temperature <= 0:
        return int(torch.argmax(logits))
    g = gumbel_noise_ref(seed, position, logits.shape[0], logits.device)
    return int(torch.argmax(logits.float() / temperature + g))


def packet(logits_slice: torch.Tensor, offset: int, temperature: float, seed: int, position: int, vocab: int):
    """(value, global index) of the best entry of a vocabulary slice."""
    x = logits_slice.float()
    if temperature > 0:
        g = gumbel_noise_ref(seed, position, vocab, x.device)[offset: offset + x.shape[0]]
        x = x / temperature + g
    v, i = x.max(0)
    return float(v), int(i) + offset


def combine_packets(packets) -> int:
    """Winner over ranks: highest value, ties -> lowest index; NaN values lose."""
    best_v, best_i = float("-inf"), None
    for v, i in packets:
        if v != v:
            continue
        if best_i is None or v > best_v or (v == best_v and i < best_i):
            best_v, best_i = v, i
    return best_i if best_i is not None else min(i for _, i in packets)
