"""Vision towers: a ViT encoder (patch embedding, pre-norm blocks with 2-D rotary or learned positions, optional
window-free full attention) followed by a spatial-merge aligner that maps patch groups to rows of the language
model's hidden size.  One class covers the three towers of the reference by configuration (depth, width, patch,
merge, rope on/off); weights may be dense or any `QuantWeight` (the Qwen tower ships as 6-bit EXL3).  Everything runs
on PyTorch ops: the towers are prefill-only and GEMM-bound, the reference runs them on libtorch as well
(engine-rs/src/vision.rs:24-166, qwen/vision.rs:30-298, ds41/vision.rs:19-148).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops


@dataclass
class VisionConfig:
    depth: int = 24
    width: int = 1024
    heads: int = 16
    mlp: int = 4096
    patch: int = 14
    merge: int = 2                 # merge x merge patches -> one language-model row
    out_hidden: int = 4096
    rope2d: bool = True            # rotary over (row, column) of the patch; False: learned position table
    max_side: int = 64             # patches per side of the position table (learned positions)
    norm_eps: float = 1e-6

    def rows_for(self, height: int, width: int) -> int:
        return (height // self.patch // self.merge) * (width // self.patch // self.merge)


def init_vision_weights(c: VisionConfig, seed: int = 0, std: float = 0.02) -> dict:
    g = torch.Generator().manual_seed(seed)

    def mat(*s):
        return torch.randn(*s, generator=g) * std
    W = {"patch": mat(c.width, 3 * c.patch * c.patch), "patch_b": torch.zeros(c.width), "norm_f": torch.ones(c.width),
         "merge_fc1": mat(c.mlp, c.width * c.merge * c.merge), "merge_fc2": mat(c.out_hidden, c.mlp), "blocks": []}
    if not c.rope2d:
        W["pos"] = mat(c.max_side * c.max_side, c.width)
    for _ in range(c.depth):
        W["blocks"].append({"n1": torch.ones(c.width), "n2": torch.ones(c.width), "qkv": mat(3 * c.width, c.width),
                            "qkv_b": torch.zeros(3 * c.width), "o": mat(c.width, c.width), "fc1": mat(c.mlp, c.width),
                            "fc2": mat(c.width, c.mlp)})
    return W


def patchify(canvas: torch.Tensor, patch: int) -> torch.Tensor:
    """uint8 [H, W, 3] -> float [gh*gw, 3*patch*patch] in [-1, 1], row-major over the patch grid."""
    H, Wd, _ = canvas.shape
    gh, gw = H // patch, Wd // patch
    x = canvas[: gh * patch, : gw * patch].float() / 127.5 - 1.0
    x = x.view(gh, patch, gw, patch, 3).permute(0, 2, 4, 1, 3).reshape(gh * gw, 3 * patch * patch)
    return x


def rope_2d(x: torch.Tensor, gh: int, gw: int, theta: float = 1e4) -> torch.Tensor:
    """x [T, heads, D]: the first half of D rotates with the patch row, the second half with the column
    (multi-axis rotary positions of the Qwen tower)."""
    T, Hh, D = x.shape
    q = D // 4
    inv = theta ** (-torch.arange(q, dtype=torch.float32, device=x.device) / q)
    rows = torch.arange(gh, device=x.device).repeat_interleave(gw).float()
    cols = torch.arange(gw, device=x.device).repeat(gh).float()
    out = []
    for pos, part in ((rows, x[..., : 2 * q]), (cols, x[..., 2 * q: 4 * q])):
        ang = pos.unsqueeze(1) * inv.unsqueeze(0)
        cos, sin = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
        a, b = part[..., :q], part[..., q:]
        out.append(torch.cat((a * cos - b * sin, b * cos + a * sin), -1))
    return torch.cat(out + [x[..., 4 * q:]], -1)


class VisionTower:
    def __init__(self, cfg: VisionConfig, W: dict, device="cpu", dtype=torch.float32):
        self.c, self.device, self.dtype = cfg, device, dtype
        from ..models.weights import to_device
        self.W = to_device(W, device, dtype) if str(device) != "cpu" else W

    def _lin(self, x, w, b=None):
        # plain library GEMMs, as the reference's towers (vision.rs: libtorch ops): patch and merge widths (3 * 14 * 14 =
        # 588, ...) do not meet the alignment rules of the language model's kernels, and a tower runs once per frame
        y = F.linear(x.to(self.dtype), w.to(self.dtype))
        return y if b is None else y + b.to(y.dtype)

    @torch.no_grad()
    def encode(self, canvas: torch.Tensor) -> torch.Tensor:
        """uint8 [H, W, 3] canvas -> [rows_for(H, W), out_hidden]."""
        c, W = self.c, self.W
        gh, gw = canvas.shape[0] // c.patch, canvas.shape[1] // c.patch
        x = self._lin(patchify(canvas.to(self.device), c.patch), W["patch"], W["patch_b"])
        if not c.rope2d:
            idx = (torch.arange(gh, device=x.device).unsqueeze(1) * c.max_side + torch.arange(gw, device=x.device)).flatten()
            x = x + W["pos"][idx].to(x.dtype)
        T, D = x.shape[0], c.width // c.heads
        for b in W["blocks"]:
            h = F.layer_norm(x.float(), (c.width,), b["n1"].float(), None, c.norm_eps).to(x.dtype)
            qkv = self._lin(h, b["qkv"], b["qkv_b"]).view(T, 3, c.heads, D)
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
            if c.rope2d:
                q, k = rope_2d(q.float(), gh, gw).to(x.dtype), rope_2d(k.float(), gh, gw).to(x.dtype)
            a = F.scaled_dot_product_attention(q.transpose(0, 1).float(), k.transpose(0, 1).float(), v.transpose(0, 1).float())
            x = x + self._lin(a.transpose(0, 1).reshape(T, c.width), b["o"])
            h = F.layer_norm(x.float(), (c.width,), b["n2"].float(), None, c.norm_eps).to(x.dtype)
            x = x + self._lin(F.gelu(self._lin(h, b["fc1"]).float(), approximate="tanh"), b["fc2"])
        x = F.layer_norm(x.float(), (c.width,), W["norm_f"].float(), None, c.norm_eps)
        # aligner: merge x merge neighbouring patches -> one row of the language model
        m = c.merge
        x = x.view(gh // m, m, gw // m, m, c.width).permute(0, 2, 1, 3, 4).reshape((gh // m) * (gw // m), m * m * c.width)
        return self._lin(F.gelu(self._lin(x, W["merge_fc1"]).float()), W["merge_fc2"]).float()
