"""Load-time re-codings of dense (non-expert) weights: smaller resident copies for the decode GEMVs.

    C12   lossless 12-bit coding of bf16 values: sign + 7 mantissa bits in one byte, a 4-bit code into a per-row table
          of the 15 most frequent exponents, code 15 = escape (exact values in a CSR side list).  0.75 of the bf16 bytes.
    Q8    int8 + fp32 scale per (row, 128 k).
    Q4    4-bit codes + (scale, minimum) per (row, 64 k), affine.
    FP8R  weight-only e4m3 + fp32 scale per row.
    SPX   INT-b (2..8 bits, little-endian bitstream per row) + fp16 scale per (row, 64 k) after a random-sign
          block-Hadamard rotation of the input dimension (round-to-nearest here; the reference calibrates with GPTQ).

Every class follows the `QuantWeight` contract (dequant() -> fp32 [N, K] on CPU), so the oracle, the CPU runner and
the device ops treat them like the checkpoint formats.  Reference: engine-rs/src/c12.rs:1-10,215-364 (C12/Q8/Q4),
dense_fp8.rs, spx.rs:1-22, weights.rs:445-530; shim/c12.cuh, q8.cuh, q4d.cuh, spx.cu.
"""
from __future__ import annotations

import math

import torch

from .formats import QuantWeight, hadamard128


# ----------------------------------------------------------------------------------------------- C12
class C12Weight(QuantWeight):
    """m8 [N,K] u8 (sign<<7 | mantissa), e4 [N,K/2] u8 (two 4-bit exponent codes, low nibble = even k),
    eb [N,15] u8 exponent table, CSR escapes (ptr [N+1] i32, col i32, val i16 = exact bf16 bits)."""
    experts = False

    def __init__(self, m8, e4, eb, ptr, col, val):
        self.m8, self.e4, self.eb, self.ptr, self.col, self.val = m8, e4, eb, ptr, col, val
        self.n, self.k = m8.shape

    @staticmethod
    def encode(w: torch.Tensor) -> "C12Weight":
        wb = w.to(torch.bfloat16).contiguous().cpu()
        bits = wb.view(torch.int16).to(torch.int32) & 0xFFFF
        N, K = bits.shape
        assert K % 2 == 0
        sign, exp, man = (bits >> 15) & 1, (bits >> 7) & 0xFF, bits & 0x7F
        m8 = ((sign << 7) | man).to(torch.uint8)
        eb = torch.zeros(N, 15, dtype=torch.uint8)
        code = torch.full((N, K), 15, dtype=torch.int32)
        for r in range(N):
            cnt = torch.bincount(exp[r], minlength=256)
            top = torch.sort(cnt, descending=True, stable=True).indices[:15]
            top = top[cnt[top] > 0]
            eb[r, : top.numel()] = top.to(torch.uint8)
            lut = torch.full((256,), 15, dtype=torch.int32)
            lut[top] = torch.arange(top.numel(), dtype=torch.int32)
            code[r] = lut[exp[r]]
        esc = code == 15
        ptr = torch.zeros(N + 1, dtype=torch.int32)
        ptr[1:] = torch.cumsum(esc.sum(1), 0).to(torch.int32)
        rows, cols = esc.nonzero(as_tuple=True)
        val = wb.view(torch.int16)[rows, cols].clone()
        e4 = (code[:, 0::2] | (code[:, 1::2] << 4)).to(torch.uint8)
        return C12Weight(m8, e4, eb, ptr, cols.to(torch.int32), val)

    def dequant_bf16(self) -> torch.Tensor:
        m8 = self.m8.cpu().to(torch.int32)
        e4 = self.e4.cpu().to(torch.int32)
        code = torch.stack((e4 & 0xF, e4 >> 4), -1).flatten(-2)
        ebx = torch.cat((self.eb.cpu().to(torch.int32), torch.zeros(self.n, 1, dtype=torch.int32)), 1)
        exp = torch.gather(ebx, 1, code.long())
        bits = ((m8 >> 7) << 15) | (exp << 7) | (m8 & 0x7F)
        out = bits.to(torch.int16)
        ptr = self.ptr.cpu().long()
        rows = torch.repeat_interleave(torch.arange(self.n), ptr[1:] - ptr[:-1])
        out[rows, self.col.cpu().long()] = self.val.cpu()
        return out.view(torch.bfloat16)

    def dequant(self):
        return self.dequant_bf16().float()

    def to(self, device):
        return C12Weight(*(t.to(device) for t in (self.m8, self.e4, self.eb, self.ptr, self.col, self.val)))

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in (self.m8, self.e4, self.eb, self.ptr, self.col, self.val))


# ----------------------------------------------------------------------------------------------- Q8 / Q4 / FP8 per row
class Q8Weight(QuantWeight):
    """int8 [N,K] + fp32 scale [N, K/128]."""
    experts = False

    def __init__(self, q, scales, group=128):
        self.q, self.scales, self.group = q, scales, group
        self.n, self.k = q.shape

    @staticmethod
    def encode(w: torch.Tensor, group: int = 128) -> "Q8Weight":
        N, K = w.shape
        blk = w.float().view(N, K // group, group)
        sc = blk.abs().amax(-1).clamp_min(1e-12) / 127.0
        q = torch.round(blk / sc.unsqueeze(-1)).clamp(-127, 127).to(torch.int8).view(N, K)
        return Q8Weight(q, sc, group)

    def dequant(self):
        q = self.q.cpu().float().view(self.n, self.k // self.group, self.group)
        return (q * self.scales.cpu().unsqueeze(-1)).view(self.n, self.k)

    def to(self, device):
        return Q8Weight(self.q.to(device), self.scales.to(device), self.group)

    def nbytes(self):
        return self.q.numel() + self.scales.numel() * 4


class Q4Weight(QuantWeight):
    """nibbles [N, K/2] (low nibble = even k) + (scale, minimum) fp32 [N, K/64, 2]: w = code * scale + minimum."""
    experts = False

    def __init__(self, q, sm, group=64):
        self.q, self.sm, self.group = q, sm, group
        self.n, self.k = q.shape[0], q.shape[1] * 2

    @staticmethod
    def encode(w: torch.Tensor, group: int = 64) -> "Q4Weight":
        N, K = w.shape
        blk = w.float().view(N, K // group, group)
        lo, hi = blk.amin(-1), blk.amax(-1)
        sc = ((hi - lo) / 15.0).clamp_min(1e-12)
        code = torch.round((blk - lo.unsqueeze(-1)) / sc.unsqueeze(-1)).clamp(0, 15).to(torch.int32).view(N, K)
        q = (code[:, 0::2] | (code[:, 1::2] << 4)).to(torch.uint8)
        return Q4Weight(q, torch.stack((sc, lo), -1).contiguous(), group)

    def dequant(self):
        q = self.q.cpu().to(torch.int32)
        code = torch.stack((q & 0xF, q >> 4), -1).flatten(-2).float().view(self.n, self.k // self.group, self.group)
        sm = self.sm.cpu()
        return (code * sm[..., 0:1] + sm[..., 1:2]).view(self.n, self.k)

    def to(self, device):
        return Q4Weight(self.q.to(device), self.sm.to(device), self.group)

    def nbytes(self):
        return self.q.numel() + self.sm.numel() * 4


class Fp8RowWeight(QuantWeight):
    """Weight-only e4m3 [N,K] + fp32 scale per row."""
    experts = False

    def __init__(self, q, scales):
        self.q, self.scales = q, scales
        self.n, self.k = q.shape

    @staticmethod
    def encode(w: torch.Tensor) -> "Fp8RowWeight":
        sc = w.float().abs().amax(-1).clamp_min(1e-12) / 448.0
        return Fp8RowWeight((w.float() / sc.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn), sc)

    def dequant(self):
        return self.q.cpu().float() * self.scales.cpu().unsqueeze(-1)

    def to(self, device):
        return Fp8RowWeight(self.q.to(device), self.scales.to(device))

    def nbytes(self):
        return self.q.numel() + self.scales.numel() * 4


# ----------------------------------------------------------------------------------------------- SPX
def _block_hadamard(x: torch.Tensor, block: int) -> torch.Tensor:
    """Orthonormal Sylvester Hadamard on consecutive `block`-wide pieces of the last axis."""
    H = hadamard128() if block == 128 else _sylvester(block)
    return (x.reshape(*x.shape[:-1], -1, block) @ H.t().to(x.dtype)).reshape(x.shape)


def _sylvester(n: int) -> torch.Tensor:
    assert n & (n - 1) == 0
    H = torch.ones(1, 1)
    while H.shape[0] < n:
        H = torch.cat((torch.cat((H, H), 1), torch.cat((H, -H), 1)), 0)
    return H / math.sqrt(n)


def pack_bits(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """[N, K] ints in [0, 2^bits) -> u8 [N, ceil(K*bits/8)], little-endian bitstream per row."""
    N, K = codes.shape
    b = ((codes.long().unsqueeze(-1) >> torch.arange(bits)) & 1).reshape(N, K * bits)
    pad = (-b.shape[1]) % 8
    if pad:
        b = torch.cat((b, torch.zeros(N, pad, dtype=b.dtype)), 1)
    return (b.view(N, -1, 8) << torch.arange(8)).sum(-1).to(torch.uint8)


def unpack_bits(packed: torch.Tensor, bits: int, K: int) -> torch.Tensor:
    N = packed.shape[0]
    b = ((packed.long().unsqueeze(-1) >> torch.arange(8)) & 1).reshape(N, -1)[:, : K * bits]
    return (b.view(N, K, bits) << torch.arange(bits)).sum(-1)


class SpxWeight(QuantWeight):
    """q u8 [N, ceil(K*bits/8)], s fp16 [N, K/64], sign int8 [K]; W_rot = (c - (2^b-1)/2) * s,
    y = W_rot . H_B(sign * x)."""
    experts = False

    def __init__(self, q, s, sign, bits, n, k, rot_block=128, group=64):
        self.q, self.s, self.sign, self.bits, self.n, self.k = q, s, sign, bits, n, k
        self.rot_block, self.group = rot_block, group

    @staticmethod
    def encode(w: torch.Tensor, bits: int = 4, rot_block: int = 128, group: int = 64, seed: int = 0) -> "SpxWeight":
        N, K = w.shape
        g = torch.Generator().manual_seed(seed)
        sign = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).to(torch.int8)
        w_rot = _block_hadamard(w.float() * sign.float(), rot_block)        # W R, so that W x = W_rot (R^T x)
        blk = w_rot.view(N, K // group, group)
        half = (2 ** bits - 1) / 2.0
        sc = (blk.abs().amax(-1) / half).clamp_min(1e-8).half().float()
        code = torch.round(blk / sc.unsqueeze(-1) + half).clamp(0, 2 ** bits - 1).view(N, K)
        return SpxWeight(pack_bits(code, bits), sc.half(), sign, bits, N, K, rot_block, group)

    def w_rot(self) -> torch.Tensor:
        code = unpack_bits(self.q.cpu(), self.bits, self.k).float()
        half = (2 ** self.bits - 1) / 2.0
        return ((code - half).view(self.n, self.k // self.group, self.group)
                * self.s.cpu().float().unsqueeze(-1)).view(self.n, self.k)

    def rotate_input(self, x: torch.Tensor) -> torch.Tensor:
        return _block_hadamard(x.float() * self.sign.to(x.device).float(), self.rot_block)

    def dequant(self):
        # W = W_rot R^T with R = diag(sign) H (H symmetric orthonormal): undo the rotation on the weight side
        return _block_hadamard(self.w_rot(), self.rot_block) * self.sign.cpu().float()

    def to(self, device):
        return SpxWeight(self.q.to(device), self.s.to(device), self.sign.to(device), self.bits, self.n, self.k,
                         self.rot_block, self.group)

    def nbytes(self):
        return self.q.numel() + self.s.numel() * 2 + self.sign.numel()


RECODERS = {"c12": C12Weight.encode, "q8": Q8Weight.encode, "q4": Q4Weight.encode, "fp8": Fp8RowWeight.encode,
            "spx": SpxWeight.encode}


def recode_dense(W: dict, kind: str, min_numel: int = 1 << 16, keys=("in", "qkv", "o", "a", "q_b", "dense_gu", "dense_down",
                                                                    "s_gu", "s_down", "lm_head")) -> dict:
    """Replace the large dense projections of a nested weight dict by their `kind` coding (load-time option,
    engine-rs/src/weights.rs:445-530)."""
    enc = RECODERS[kind]

    def rec(node, key=None):
        if isinstance(node, dict):
            return {k: rec(v, k) for k, v in node.items()}
        if isinstance(node, list):
            return [rec(v, key) for v in node]
        if (isinstance(node, torch.Tensor) and node.dim() == 2 and key in keys and node.numel() >= min_numel
                and node.shape[1] % 128 == 0):
            return enc(node.float().cpu()).to(node.device)
        return node
    return rec(W)
