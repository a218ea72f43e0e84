"""Block-sparse selection for the sparse-attention layers: indexer scores + exact top-k (ties -> lowest index)."""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

from . import cuda as cu

vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
_bound = False


def _dll():
    global _bound
    dll = cu.lib()._dll
    if not _bound:
        dll.spark_idx_score.argtypes = [vp, i32, i32, i32, vp, vp, vp, i32, vp, f32, vp, i32, i32, vp]
        dll.spark_idx_score.restype = i32
        dll.spark_idx_score_mma.argtypes = [vp, i32, i32, vp, vp, vp, i32, i32, i32, vp, f32, vp, i32, vp]
        dll.spark_idx_score_mma.restype = i32
        dll.spark_topk_select.argtypes = [vp, i32, vp, i32, i32, i32, vp, i32, vp, vp, i32]
        dll.spark_topk_select.restype = i32
        dll.spark_topk_select_mc.argtypes = [vp, i32, vp, i32, i32, i32, vp, i32, vp, vp, i32, i32, vp]
        dll.spark_topk_select_mc.restype = i32
        _bound = True
    return dll


SCORE_MMA = os.environ.get("SPARK_IDX_SCORE_MMA", "1") == "1"
SCORE_MMA_MIN_ROWS = 64


def select_tokens(qi, pool, row_kv, pos32, block, topk, max_ctx, head_w=None, scale=None, window=0, segs=None):
    """qi [R,H,Dm] fp32 indexer queries; pool [*, Dm] fp32 pooled keys (block b of a sequence at row_kv/block + b).
    `window` > 0 keeps the last `window` positions visible as well.  `segs` = (segment table int32 [nseg, 4], nseg,
    longest segment) when the rows are whole segments at consecutive positions: prefill-size batches are then scored
    on tensor cores.  Returns (sel [R, topk*block + block + window] int32 token indices, sel_n [R])."""
    R, H, Dm = qi.shape
    dev = qi.device
    nb_max = max(1, max_ctx // block)
    score = cu.scratch("idx_score", R * nb_max, torch.float32, dev)
    cu.add_launches(2)
    sc = float(scale if scale is not None else 1.0 / math.sqrt(Dm))
    if (SCORE_MMA and segs is not None and R >= SCORE_MMA_MIN_ROWS and 1 <= H <= 64 and H & (H - 1) == 0
            and Dm % 8 == 0 and 8 <= Dm <= 128):
        seg, nseg, max_rows = segs
        rc = _dll().spark_idx_score_mma(cu.P(qi), H, Dm, cu.P(pool), cu.P(row_kv), cu.P(seg), nseg, max_rows, block,
                                        cu.P(head_w), sc, cu.P(score), nb_max, cu.stream())
        cu.check(rc, "spark_idx_score_mma")
    else:
        rc = _dll().spark_idx_score(cu.P(qi), R, H, Dm, cu.P(pool), cu.P(row_kv), cu.P(pos32), block, cu.P(head_w), sc,
                                    cu.P(score), nb_max, nb_max, cu.stream())
        cu.check(rc, "spark_idx_score")
    sel, sel_n = topk_select(score, nb_max, pos32, block, topk, window)
    return sel, sel_n


MC_MIN_CANDIDATES = int(os.environ.get("SPARK_TOPK_MC_MIN", "32768"))


def topk_select(score, nb_max, pos32, block, topk, window=0, ctas=None):
    """Exact top-k blocks per row (ties -> lowest index), expanded to token indices + the always-visible tail.  Rows
    of >= MC_MIN_CANDIDATES candidates with few rows in the batch use the multi-CTA select (`ctas` CTAs per row, 4096
    candidates each, at most 64); the result is identical."""
    R = pos32.shape[0]
    dev = score.device
    sel_ld = topk * block + block + window
    sel = torch.empty(R, sel_ld, dtype=torch.int32, device=dev)
    sel_n = torch.empty(R, dtype=torch.int32, device=dev)
    if ctas is None:
        ctas = min(64, (nb_max + 4095) // 4096) if (nb_max >= MC_MIN_CANDIDATES and R <= 64) else 1
    if ctas > 1:
        work = cu.scratch("topk_mc_work", R * (3 * 2048 + 3 * ctas), torch.int32, dev)
        cu.add_launches(4)                       # 5 launches instead of 1
        rc = _dll().spark_topk_select_mc(cu.P(score), nb_max, cu.P(pos32), R, block, topk, cu.P(sel), sel_ld, cu.P(sel_n),
                                         cu.stream(), window, ctas, cu.P(work))
        cu.check(rc, "spark_topk_select_mc")
        return sel, sel_n
    rc = _dll().spark_topk_select(cu.P(score), nb_max, cu.P(pos32), R, block, topk, cu.P(sel), sel_ld, cu.P(sel_n),
                                  cu.stream(), window)
    cu.check(rc, "spark_topk_select")
    return sel, sel_n


def select_blocks(mixer, qi, plan, d):
    c = mixer.c
    segs = None if plan.is_tree else (d["seg"], len(plan.segs), max(s.n for s in plan.segs))
    return select_tokens(qi, mixer.ik_pool, d["row_kv"], d["pos32"], c.block, c.sparse_topk_blocks, d["max_ctx"], segs=segs)
