"""Checkpoint weight formats: EXL3 trellis, MXFP4 (E2M1 + E8M0/32), FP8 e4m3 block-scaled.

Each format has (a) a CPU/torch decoder that defines the numerics (the oracle the kernels are tested
against), (b) a random generator (no checkpoints exist on the build machines; any EXL3 bitstream
decodes to valid weights, so random bits + random sign/scale vectors are a valid random-init model),
(c) the packed tensors the kernels read.

EXL3 contract (reference/qwen38/exl3.py:1-110, reference/glm53/exl3.py:24-46; kernels
engine-rs/shim/qwen_exl3.cuh:17-117): inner weight [K,N] stored as trellis[K/16, N/16, 16*bits] int16,
one 256-weight tile per (k-tile, n-tile).  A tile's words, viewed as little-endian uint32 and read
MSB-first, form a tail-biting ring of 256*bits bits; the 16-bit state of stream position t starts at
bit ((t+1)*bits - 16) mod (256*bits); position t holds tile element PERM[t] (tensor-core fragment
order).  Codebooks: `mul1`  x = state*0x83DCD12D; s = sum of the 4 bytes of x;
value = fp16(fp16(1024+s) * fp16(bits 0x1eee) + fp16(bits 0xc931)) (one rounding);
`mcg`  y = state*0xCBAC1FED; y = (y & 0x8FFF8FFF) ^ 0x3B603B60; value = fp16(lo16) + fp16(hi16).
Full weight: y = had128(had128(x * suh) @ inner) * svh, had128 = blockwise 128-point Hadamard / sqrt(128).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

MUL1 = 0x83DCD12D
MCG = 0xCBAC1FED


class QuantWeight:
    """Base of quantised weights: logical shape [N, K] (out, in)."""
    n: int
    k: int

    def dequant(self) -> torch.Tensor:          # -> [N, K] fp32 on CPU
        raise NotImplementedError

    def dequant_expert(self, e: int) -> torch.Tensor:
        raise NotImplementedError

    @property
    def shape(self):
        return (self.n, self.k)


# ----------------------------------------------------------------------------- EXL3
def fragment_perm() -> torch.Tensor:
    """PERM[t]: tile element (row*16+col, row = k, col = n) held by stream position t.  Positions
    are grouped by lane of an m16n8k16 B fragment: lane l owns rows {2(l%4), +1, +8, +9} of columns
    l//4 and l//4+8."""
    t = torch.arange(256)
    lane, j = t // 8, t % 8
    row = (lane % 4) * 2 + (j % 2) + ((j % 4) // 2) * 8
    col = lane // 4 + (j // 4) * 8
    return row * 16 + col


_CB = {}


def codebook(kind: str) -> torch.Tensor:
    """All 65536 decoded values as fp32 (exact fp16 values)."""
    if kind in _CB:
        return _CB[kind]
    s = torch.arange(65536, dtype=torch.int64)
    if kind == "mul1":
        x = (s * MUL1) & 0xFFFFFFFF
        bsum = (x & 255) + ((x >> 8) & 255) + ((x >> 16) & 255) + ((x >> 24) & 255)
        a = (1024 + bsum).double()
        inv = torch.tensor([0x1EEE], dtype=torch.int16).view(torch.float16).double()
        bias = torch.tensor([0xC931 - 0x10000], dtype=torch.int16).view(torch.float16).double()
        v = (a * inv + bias).to(torch.float16).float()
    elif kind == "mcg":
        y = (s * MCG) & 0xFFFFFFFF
        y = (y & 0x8FFF8FFF) ^ 0x3B603B60
        lo = (y & 0xFFFF)
        hi = (y >> 16) & 0xFFFF

        def h(bits):
            b = torch.where(bits >= 0x8000, bits - 0x10000, bits).to(torch.int16)
            return b.view(torch.float16)
        v = (h(lo) + h(hi)).float()          # fp16 add: one rounding
    else:
        raise ValueError(kind)
    _CB[kind] = v
    return v


def hadamard128() -> torch.Tensor:
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.shape[0] < 128:
        h = torch.cat((torch.cat((h, h), 1), torch.cat((h, -h), 1)), 0)
    return (h / math.sqrt(128)).float()


def trellis_states(trellis: torch.Tensor, bits: int) -> torch.Tensor:
    """trellis [..., 16*bits] int16 -> [..., 256] int64 states in stream order."""
    lead = trellis.shape[:-1]
    w16 = trellis.reshape(-1, 16 * bits).to(torch.int64) & 0xFFFF
    w32 = w16[:, 0::2] | (w16[:, 1::2] << 16)
    n_words, n_bits = 8 * bits, 256 * bits
    t = torch.arange(256, device=trellis.device)
    first = ((t + 1) * bits - 16) % n_bits
    wi = first >> 5
    win = (w32[:, wi] << 32) | w32[:, (wi + 1) % n_words]
    return ((win >> (48 - (first & 31))) & 0xFFFF).reshape(*lead, 256)


def exl3_inner(trellis: torch.Tensor, kind: str = "mul1") -> torch.Tensor:
    """trellis [Kt, Nt, 16*bits] int16 -> codebook values [Kt*16, Nt*16] fp32 (inner weight, [K,N])."""
    Kt, Nt, Wd = trellis.shape
    bits = Wd // 16
    cb = codebook(kind).to(trellis.device)
    vals = cb[trellis_states(trellis, bits)]                       # [Kt, Nt, 256] stream order
    tile = torch.empty_like(vals)
    tile[..., fragment_perm().to(trellis.device)] = vals
    return tile.view(Kt, Nt, 16, 16).permute(0, 2, 1, 3).reshape(Kt * 16, Nt * 16)


def exl3_full(trellis, suh, svh, kind="mul1") -> torch.Tensor:
    """-> W_kn [K, N] fp32 with y = x @ W_kn."""
    w = exl3_inner(trellis, kind)
    K, N = w.shape
    h = hadamard128().to(w.device)
    w = (h @ w.view(K // 128, 128, N)).view(K, N) * suh.float().view(K, 1)
    w = (w.view(K, N // 128, 128) @ h).view(K, N) * svh.float().view(1, N)
    return w


class Exl3Weight(QuantWeight):
    """One linear [N,K] (trellis [K/16, N/16, 16*bits]) or a stack of experts (leading E dim)."""

    def __init__(self, trellis, suh, svh, bits: int, kind: str = "mul1"):
        self.trellis, self.suh, self.svh, self.bits, self.kind = trellis, suh, svh, bits, kind
        self.experts = trellis.dim() == 4
        self.k = trellis.shape[-3] * 16
        self.n = trellis.shape[-2] * 16

    def dequant(self):
        assert not self.experts
        return exl3_full(self.trellis.cpu(), self.suh.cpu(), self.svh.cpu(), self.kind).t().contiguous()

    def dequant_expert(self, e):
        return exl3_full(self.trellis[e].cpu(), self.suh[e].cpu(), self.svh[e].cpu(), self.kind).t().contiguous()

    def to(self, device):
        return Exl3Weight(self.trellis.to(device), self.suh.to(device), self.svh.to(device), self.bits, self.kind)

    def nbytes(self):
        return self.trellis.numel() * 2 + self.suh.numel() * 2 + self.svh.numel() * 2


def random_exl3(n: int, k: int, bits: int = 4, experts: int = 0, std: float = 0.02, seed: int = 0,
                device="cpu", kind: str = "mul1") -> Exl3Weight:
    """Random-init EXL3 weight whose decoded entries have standard deviation ~`std`: codebook values
    are ~N(0,1) and the two Hadamard transforms are orthonormal, so |suh|*|svh| = std."""
    assert n % 128 == 0 and k % 128 == 0, "EXL3 needs 128-aligned shapes (Hadamard blocks)"
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    lead = (experts,) if experts else ()
    trellis = torch.randint(-32768, 32768, lead + (k // 16, n // 16, 16 * bits), dtype=torch.int16,
                            device=device, generator=g)
    s = math.sqrt(std)
    suh = ((torch.randint(0, 2, lead + (k,), device=device, generator=g) * 2 - 1).float() * s).half()
    svh = ((torch.randint(0, 2, lead + (n,), device=device, generator=g) * 2 - 1).float() * s).half()
    return Exl3Weight(trellis, suh, svh, bits, kind)


# ----------------------------------------------------------------------------- MXFP4 / FP8
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
                            -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


def e8m0_to_float(e: torch.Tensor) -> torch.Tensor:
    """E8M0 byte -> 2^(e-127) (255 = NaN is never generated)."""
    return torch.pow(2.0, e.float() - 127.0)


def quant_mxfp4(w: torch.Tensor):
    """[..., K] fp32 -> (packed nibbles uint8 [..., K/2] low nibble first, scales uint8 [..., K/32]).
    Scale = 2^ceil(log2(amax/6)) per 32 (UE8M0, reference/ds41/kernel.py:76-93), round-to-nearest
    on the E2M1 grid (ties to the even code)."""
    K = w.shape[-1]
    blk = w.float().reshape(*w.shape[:-1], K // 32, 32)
    amax = blk.abs().amax(-1).clamp_min(6.0 * 2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    sc = torch.pow(2.0, e)
    x = blk / sc.unsqueeze(-1)
    grid = E2M1_VALUES[:8]
    mag = x.abs().clamp(max=6.0)
    d = (mag.unsqueeze(-1) - grid).abs()
    # ties -> even code (codes with mantissa bit 0): prefer even index on equal distance
    d = d + torch.tensor([0, 1, 0, 1, 0, 1, 0, 1]) * 1e-7
    code = d.argmin(-1)
    code = code + (x < 0).long() * 8
    code = code.reshape(*w.shape[:-1], K)
    packed = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)
    return packed, (e + 127).to(torch.uint8)


def dequant_mxfp4(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    lo = (packed & 0xF).long()
    hi = (packed >> 4).long()
    code = torch.stack((lo, hi), -1).flatten(-2)
    v = E2M1_VALUES.to(packed.device)[code]
    K = v.shape[-1]
    return (v.view(*v.shape[:-1], K // 32, 32) * e8m0_to_float(scales).unsqueeze(-1)).reshape(*v.shape)


class Mxfp4Weight(QuantWeight):
    """[N,K] (or [E,N,K]) E2M1 nibbles + E8M0 scale per 32 along K."""

    def __init__(self, packed, scales):
        self.packed, self.scales = packed, scales
        self.experts = packed.dim() == 3
        self.n, self.k = packed.shape[-2], packed.shape[-1] * 2

    def dequant(self):
        return dequant_mxfp4(self.packed.cpu(), self.scales.cpu())

    def dequant_expert(self, e):
        return dequant_mxfp4(self.packed[e].cpu(), self.scales[e].cpu())

    def to(self, device):
        return Mxfp4Weight(self.packed.to(device), self.scales.to(device))

    def nbytes(self):
        return self.packed.numel() + self.scales.numel()


def random_mxfp4(n, k, experts=0, std=0.02, seed=0, device="cpu") -> Mxfp4Weight:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    lead = (experts,) if experts else ()
    packed = torch.randint(0, 256, lead + (n, k // 2), dtype=torch.uint8, device=device, generator=g)
    # E2M1 uniform codes have rms ~2.9; pick the exponent so that the decoded std is ~`std`
    e = int(round(math.log2(std / 2.9))) + 127
    scales = torch.randint(e - 1, e + 1, lead + (n, k // 32), dtype=torch.uint8, device=device, generator=g)
    return Mxfp4Weight(packed, scales)


def quant_fp8_block(w: torch.Tensor, bn: int = 128, bk: int = 128, pow2: bool = False):
    """[N,K] fp32 -> (e4m3 [N,K], fp32 scales [N/bn, K/bk]); amax clamp 1e-4
    (reference/ds41/kernel.py:59-73)."""
    N, K = w.shape
    blk = w.float().view(N // bn, bn, K // bk, bk)
    amax = blk.abs().amax((1, 3)).clamp_min(1e-4)
    sc = amax / 448.0
    if pow2:
        sc = torch.pow(2.0, torch.ceil(torch.log2(sc)))
    q = (blk / sc.view(N // bn, 1, K // bk, 1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(N, K), sc


class Fp8BlockWeight(QuantWeight):
    """e4m3 [N,K] with fp32 scale per (bn x bk) block (128x128 dense weights; 1x128 activations)."""

    def __init__(self, q, scales, bn=128, bk=128):
        self.q, self.scales, self.bn, self.bk = q, scales, bn, bk
        self.experts = q.dim() == 3
        self.n, self.k = q.shape[-2], q.shape[-1]

    def _deq(self, q, s):
        N, K = q.shape
        return (q.float().view(N // self.bn, self.bn, K // self.bk, self.bk)
                * s.view(N // self.bn, 1, K // self.bk, 1)).view(N, K)

    def dequant(self):
        return self._deq(self.q.cpu(), self.scales.cpu())

    def dequant_expert(self, e):
        return self._deq(self.q[e].cpu(), self.scales[e].cpu())

    def to(self, device):
        return Fp8BlockWeight(self.q.to(device), self.scales.to(device), self.bn, self.bk)

    def nbytes(self):
        return self.q.numel() + self.scales.numel() * 4


def random_fp8_block(n, k, experts=0, std=0.02, seed=0, device="cpu") -> Fp8BlockWeight:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    lead = (experts,) if experts else ()
    w = torch.randn(lead + (n, k), device=device, generator=g)
    q = (w * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
    sc = torch.full(lead + (n // 128, k // 128), std / 100, device=device) \
        * (1 + 0.1 * torch.rand(lead + (n // 128, k // 128), device=device, generator=g))
    return Fp8BlockWeight(q, sc)


def act_quant_fp8(x: torch.Tensor, block: int = 128, pow2: bool = False):
    """Activation quant e4m3 per 1 x `block` (reference/ds41/kernel.py:59-73)."""
    R, K = x.shape
    blk = x.float().view(R, K // block, block)
    amax = blk.abs().amax(-1).clamp_min(1e-4)
    sc = amax / 448.0
    if pow2:
        sc = torch.pow(2.0, torch.ceil(torch.log2(sc)))
    return (blk / sc.unsqueeze(-1)).to(torch.float8_e4m3fn).view(R, K), sc


# ----------------------------------------------------------------------------------------------- MXFP8
def quant_mxfp8(w: torch.Tensor):
    """[..., K] fp32 -> (e4m3 [..., K], E8M0 scale bytes [..., K/32]); scale = 2^ceil(log2(amax/448)) per 32
    (reference/ds41/kernel.py:76-93)."""
    K = w.shape[-1]
    blk = w.float().reshape(*w.shape[:-1], K // 32, 32)
    amax = blk.abs().amax(-1).clamp_min(448.0 * 2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q = (blk / torch.pow(2.0, e).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).reshape(w.shape)
    return q, (e + 127).to(torch.uint8)


def dequant_mxfp8(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    K = q.shape[-1]
    return (q.float().reshape(*q.shape[:-1], K // 32, 32) * e8m0_to_float(scales).unsqueeze(-1)).reshape(q.shape)


class Mxfp8Weight(QuantWeight):
    """e4m3 [N,K] + E8M0 scale per 32 along K: the operand format of the block-scaled tensor-core GEMM."""
    experts = False

    def __init__(self, q, scales):
        self.q, self.scales = q, scales
        self.n, self.k = q.shape

    @staticmethod
    def encode(w: torch.Tensor) -> "Mxfp8Weight":
        return Mxfp8Weight(*quant_mxfp8(w))

    def dequant(self):
        return dequant_mxfp8(self.q.cpu(), self.scales.cpu())

    def to(self, device):
        return Mxfp8Weight(self.q.to(device), self.scales.to(device))

    def nbytes(self):
        return self.q.numel() + self.scales.numel()


def random_mxfp8(n, k, std=0.02, seed=0, device="cpu") -> Mxfp8Weight:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    q = (torch.randn(n, k, device=device, generator=g) * 100).clamp(-448, 448).to(torch.float8_e4m3fn)
    e = int(round(math.log2(std / 100))) + 127
    scales = torch.randint(e - 1, e + 1, (n, k // 32), dtype=torch.uint8, device=device, generator=g)
    return Mxfp8Weight(q, scales)


# ----------------------------------------------------------------------------- slicing (tensor-parallel shards)
# A shard of a quantised matrix is cut out of the packed tensors without decoding.  Output rows are taken in whole
# 128-row blocks (the EXL3 output Hadamard and the FP8 block scales mix 128 rows; the MX formats scale along K only,
# but every shard rule cuts at multiples of the head size, so one rule serves all), input columns in whole 128-column
# blocks, experts by index range.  Dense tensors take the same three cuts with plain indexing.
def _blocks_of(idx: torch.Tensor, block: int) -> torch.Tensor:
    if idx.numel() % block:
        raise ValueError(f"output rows of a quantised matrix must be selected in whole aligned blocks of {block}")
    idx = idx.reshape(-1, block)
    first = idx[:, 0]
    if (first % block).any() or not torch.equal(idx, first.unsqueeze(1) + torch.arange(block)):
        raise ValueError(f"output rows of a quantised matrix must be selected in whole aligned blocks of {block}")
    return first // block


def take_out(w, idx: torch.Tensor):
    """Rows `idx` (output features) of a [.., N, K] weight."""
    idx = idx.cpu()
    if isinstance(w, torch.Tensor):
        return w.index_select(-2, idx.to(w.device)).contiguous()
    if isinstance(w, Exl3Weight):
        tiles = (_blocks_of(idx, 128).unsqueeze(1) * 8 + torch.arange(8)).flatten().to(w.trellis.device)
        return Exl3Weight(w.trellis.index_select(-2, tiles).contiguous(), w.suh,
                          w.svh.index_select(-1, idx.to(w.svh.device)).contiguous(), w.bits, w.kind)
    if isinstance(w, Mxfp4Weight):
        i = idx.to(w.packed.device)
        return Mxfp4Weight(w.packed.index_select(-2, i).contiguous(), w.scales.index_select(-2, i).contiguous())
    if isinstance(w, Mxfp8Weight):
        i = idx.to(w.q.device)
        return Mxfp8Weight(w.q.index_select(-2, i).contiguous(), w.scales.index_select(-2, i).contiguous())
    if isinstance(w, Fp8BlockWeight):
        blk = _blocks_of(idx, w.bn).to(w.q.device)
        return Fp8BlockWeight(w.q.index_select(-2, idx.to(w.q.device)).contiguous(),
                              w.scales.index_select(-2, blk).contiguous(), w.bn, w.bk)
    raise TypeError(type(w))


def take_in(w, lo: int, hi: int):
    """Columns [lo, hi) (input features) of a [.., N, K] weight; lo and hi multiples of 128 for quantised formats."""
    if isinstance(w, torch.Tensor):
        return w[..., lo:hi].contiguous()
    if lo % 128 or hi % 128:
        raise ValueError("input columns of a quantised matrix are cut at multiples of 128")
    if isinstance(w, Exl3Weight):
        return Exl3Weight(w.trellis[..., lo // 16: hi // 16, :, :].contiguous(), w.suh[..., lo:hi].contiguous(), w.svh,
                          w.bits, w.kind)
    if isinstance(w, Mxfp4Weight):
        return Mxfp4Weight(w.packed[..., lo // 2: hi // 2].contiguous(), w.scales[..., lo // 32: hi // 32].contiguous())
    if isinstance(w, Mxfp8Weight):
        return Mxfp8Weight(w.q[..., lo:hi].contiguous(), w.scales[..., lo // 32: hi // 32].contiguous())
    if isinstance(w, Fp8BlockWeight):
        return Fp8BlockWeight(w.q[..., lo:hi].contiguous(), w.scales[..., lo // w.bk: hi // w.bk].contiguous(), w.bn, w.bk)
    raise TypeError(type(w))


def take_experts(w, lo: int, hi: int):
    """Experts [lo, hi) of a stacked [E, N, K] weight."""
    if isinstance(w, torch.Tensor):
        return w[lo:hi].contiguous()
    if isinstance(w, Exl3Weight):
        return Exl3Weight(w.trellis[lo:hi].contiguous(), w.suh[lo:hi].contiguous(), w.svh[lo:hi].contiguous(), w.bits, w.kind)
    if isinstance(w, Mxfp4Weight):
        return Mxfp4Weight(w.packed[lo:hi].contiguous(), w.scales[lo:hi].contiguous())
    if isinstance(w, Fp8BlockWeight):
        return Fp8BlockWeight(w.q[lo:hi].contiguous(), w.scales[lo:hi].contiguous(), w.bn, w.bk)
    raise TypeError(type(w))


def weight_tensors(w) -> dict:
    """The packed tensors of a weight by field name (what a checkpoint stores)."""
    if isinstance(w, torch.Tensor):
        return {"weight": w}
    if isinstance(w, Exl3Weight):
        return {"trellis": w.trellis, "suh": w.suh, "svh": w.svh}
    if isinstance(w, Mxfp4Weight):
        return {"packed": w.packed, "scales": w.scales}
    if isinstance(w, Mxfp8Weight):
        return {"q8": w.q, "scales8": w.scales}
    if isinstance(w, Fp8BlockWeight):
        return {"q": w.q, "block_scales": w.scales}
    raise TypeError(type(w))


def weight_from_tensors(t: dict, meta: dict):
    """Inverse of `weight_tensors`; `meta` carries the format attributes that are not tensors."""
    if "weight" in t:
        return t["weight"]
    if "trellis" in t:
        return Exl3Weight(t["trellis"], t["suh"], t["svh"], t["trellis"].shape[-1] // 16, meta.get("kind", "mul1"))
    if "packed" in t:
        return Mxfp4Weight(t["packed"], t["scales"])
    if "q8" in t:
        return Mxfp8Weight(t["q8"], t["scales8"])
    if "q" in t:
        return Fp8BlockWeight(t["q"], t["block_scales"], int(meta.get("bn", 128)), int(meta.get("bk", 128)))
    raise ValueError(sorted(t))
