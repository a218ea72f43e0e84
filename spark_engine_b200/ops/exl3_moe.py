"""Prefill-size MoE over EXL3 experts: dequant to the tcgen05 grouped GEMM.

Rows arrive in expert order.  Default: per projection an input Hadamard with the row's expert sign/scale
vector (fp16), then the fused grouped kernel (`exl3_mgemm.cu`) that decodes each expert's packed trellis once
per <= 64 rows straight into MMA fragments and applies the output Hadamard in its epilogue.  With very many rows
per expert: all experts' trellises reconstructed to fp16 K-major matrices in one launch, grouped tcgen05
GEMM over the <=128-row tile list, output Hadamard with the expert's output vector.  The reference
runs this with mma.sync grouped kernels that decode B tiles in the mainloop
(engine-rs/shim/moe_exl3.cuh:521-1233).
"""
from __future__ import annotations

import os

import torch

from . import cuda as cu


EXL3_MOE_FUSED = os.environ.get("SPARK_EXL3_MOE_FUSED", "1") == "1"
SMALL_ITEM_ROWS_PER_EXPERT = int(os.environ.get("SPARK_MG_SMALL", "24"))   # average rows per expert up to which 32-row items win
FUSED_MAX_ROWS_PER_EXPERT = int(os.environ.get("SPARK_MG_FUSED_MAX", "48"))   # average rows per expert beyond which the
                                     # one-off reconstruction + tcgen05 grouped GEMM beats decoding once per 64 rows


def exl3_grouped_experts(a, wgu, wd, ids, perm, tiles, ntile, max_tiles, c):
    dev = a.device
    E = wgu.trellis.shape[0]
    H, F2 = wgu.k, wgu.n
    F = F2 // 2
    # rows past this rank's pairs are filler (perm 0): their expert id may be -1 (non-local) -> clamp, they are
    # never part of a tile and never combined
    row_expert = ids.view(-1)[perm.long()].clamp_min(0).to(torch.int32).contiguous()
    xh = cu.exl3_had_rows(a, wgu.suh, post=False, row_expert=row_expert, expert_stride=H)
    if EXL3_MOE_FUSED and wgu.bits == 4 and a.shape[0] <= FUSED_MAX_ROWS_PER_EXPERT * E:
        # packed trellises straight into the MMA: decode once per <= 64 rows of an expert, output Hadamard fused
        rpi = 32 if a.shape[0] <= SMALL_ITEM_ROWS_PER_EXPERT * E else 64
        gu = cu.exl3_mgemm(xh, wgu, tiles, ntile, max_tiles, rows_per_item=rpi)
        act = cu.swiglu(gu, c.swiglu_limit)
        xh2 = cu.exl3_had_rows(act, wd.suh, post=False, row_expert=row_expert, expert_stride=F)
        return cu.exl3_mgemm(xh2, wd, tiles, ntile, max_tiles, out_f32=True, rows_per_item=rpi)
    wt = cu.exl3_reconstruct(wgu, cu.scratch("exl3_recon_gu", E * F2 * H, torch.float16, dev)[: E * F2 * H].view(E, F2, H))
    acc = cu.grouped_gemm(xh, wt.view(E * F2, H), tiles, ntile, max_tiles, E, F2, F2, 0, fmt=0)
    gu = cu.exl3_had_rows(acc, wgu.svh, post=True, row_expert=row_expert, expert_stride=F2)
    act = cu.swiglu(gu, c.swiglu_limit)
    xh2 = cu.exl3_had_rows(act, wd.suh, post=False, row_expert=row_expert, expert_stride=F)
    wt2 = cu.exl3_reconstruct(wd, cu.scratch("exl3_recon_d", E * H * F, torch.float16, dev)[: E * H * F].view(E, H, F))
    acc2 = cu.grouped_gemm(xh2, wt2.view(E * H, F), tiles, ntile, max_tiles, E, H, H, 0, fmt=0)
    return cu.exl3_had_rows(acc2, wd.svh, post=True, row_expert=row_expert, expert_stride=H)
