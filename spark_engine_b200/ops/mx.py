"""Device ops for the micro-scaled weight formats (FP8 128x128-block dense weights, MXFP4 experts).

Decode / verify rows (<= 16) and MoE (expert,row) pairs stream the packed weights through the tensor-core
GEMV of `csrc/kernels/mx.cu`; prefill-size batches convert the weights to bf16 once per call and run the
tcgen05 GEMM (dense) or the grouped tcgen05 GEMM over the ragged expert tile list.  Activation
quantisers (FP8 1x128, MXFP8 1x32) are exposed for the block-scaled paths and the FP8 KV / latent stores.
Reference: engine-rs/shim/ds41_mx.cu (fp8_gemv_mx, up_mx/down_mx, up_gemm/down_gemm, act_quant),
fp8.cu / fp8ws.cu, engine-rs/src/ds41/load.rs:116-160.
"""
from __future__ import annotations

import ctypes
import os

import torch

from ..quant.formats import Fp8BlockWeight, Mxfp4Weight, Mxfp8Weight, QuantWeight
from ..quant.recode import Fp8RowWeight, Q4Weight, Q8Weight
from . import cuda as cu

_vp, _i32, _i64, _f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_SIGS = {
    "spark_mx_gemv": [_vp, _i32, _vp, _vp, _i32, _i64, _i64, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _i32, _f32, _i32,
                      _vp],
    "spark_mx_dequant": [_vp, _vp, _i32, _vp, _i64, _i32, _i32, _vp],
    "spark_act_quant": [_vp, _i32, _i32, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp],
    "spark_gemm_mxfp8": [_vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp],
    "spark_mx_sf_to_blocks": [_vp, _vp, _i32, _i32, _vp],
    "spark_mx_mgemm": [_vp, _i32, _vp, _vp, _i64, _i64, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _i32, _f32, _vp],
    "spark_mx4_items": [_i32, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _vp],
    "spark_mx4_prep": [_i32, _vp, _vp, _vp, _vp, _i32, _i32, _vp, _i32, _vp, _vp, _vp, _vp],
    "spark_mx_sf_tile_blocks": [_vp, _vp, _vp, _i32, _i32, _vp, _vp],
    "spark_moe_mxfp4": [_vp, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _i32, _i32, _i32, _vp, _vp],
    "spark_coded_gemv": [_vp, _i32, _vp, _vp, _i32, _vp, _i32, _i32, _i32, _i32, _i32, _vp],
}
_bound = False


def _lib():
    global _bound
    dll = cu.lib()
    if not _bound:
        for name, sig in _SIGS.items():
            fn = getattr(dll._dll, name)
            fn.argtypes, fn.restype = sig, _i32
        _bound = True
    return dll


def _parts(w: QuantWeight):
    """(packed bytes, scales, fmt, bytes per expert, scale elements per expert)"""
    if isinstance(w, Fp8BlockWeight):
        assert w.bn == 128 and w.bk == 128, "the device path serves 128x128 block scales"
        q = w.q.view(torch.uint8)
        return q, w.scales, 0, w.n * w.k, (w.n // 128) * (w.k // 128)
    if isinstance(w, Mxfp4Weight):
        return w.packed, w.scales, 1, w.n * w.k // 2, w.n * (w.k // 32)
    if isinstance(w, Mxfp8Weight):
        return w.q.view(torch.uint8), w.scales, 2, w.n * w.k, w.n * (w.k // 32)
    raise TypeError(type(w))


def gemv(x, w: QuantWeight, items=1, rows_per_item=None, pair_expert=None, pair_row=None, act=0, limit=0.0,
         out_f32=False):
    x = cu._as_bf16(x).contiguous()
    q, sc, fmt, wes, ses = _parts(w)
    if fmt == 1 and not getattr(w, "_scale_range_ok", False) and not torch.cuda.is_current_stream_capturing():
        # the decode kernel folds 2^14 into the fp16 block scale: scales up to 2 (E8M0 byte 128) are exact
        if int(sc.max()) > 128:
            raise ValueError("MXFP4 block scale above 2: outside the range of the decode kernel")
        w._scale_range_ok = True
    rows_per_item = rows_per_item if rows_per_item is not None else x.shape[0]
    y = torch.empty(items * rows_per_item, w.n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    rc = _lib().spark_mx_gemv(cu.P(x), x.stride(0), cu.P(q), cu.P(sc), fmt, wes, ses, cu.P(y), w.n, items, rows_per_item,
                              w.n, w.k, cu.P(pair_expert), cu.P(pair_row), act, float(limit), int(out_f32), cu.stream())
    cu.check(rc, "spark_mx_gemv")
    return y


def dequant_bf16(w: QuantWeight, out=None):
    """All rows (all experts) of `w` as bf16 [.., N, K] on the device."""
    q, sc, fmt, _, _ = _parts(w)
    E = q.shape[0] if w.experts else 1
    rows = E * w.n
    if out is None:
        out = torch.empty(rows * w.k, dtype=torch.bfloat16, device=q.device)
    rc = _lib().spark_mx_dequant(cu.P(q), cu.P(sc), fmt, cu.P(out), rows, w.n, w.k, cu.stream())
    cu.check(rc, "spark_mx_dequant")
    return out[: rows * w.k].view(*((E,) if w.experts else ()), w.n, w.k)


def act_quant(x, block=128, pow2=False, act=0, limit=0.0):
    """x [R, K] (or [R, 2K] = [gate | up] with act=1) bf16/fp32 -> (e4m3 [R, K], scales): fp32 [R, K/128] for
    block 128, E8M0 bytes [R, K/32] for block 32."""
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype in (torch.bfloat16, torch.float32)
    R = x.shape[0]
    K = x.shape[1] // (2 if act else 1)
    q = torch.empty(R, K, dtype=torch.uint8, device=x.device)
    sc = torch.empty(R, K // block, dtype=torch.float32 if block == 128 else torch.uint8, device=x.device)
    rc = _lib().spark_act_quant(cu.P(x), x.stride(0), int(x.dtype == torch.float32), cu.P(q), cu.P(sc), R, K, block,
                                int(pow2), act, float(limit), cu.stream())
    cu.check(rc, "spark_act_quant")
    return q.view(torch.float8_e4m3fn), sc


def coded_gemv(x, w, out_f32=False):
    """<= 16 rows through the int8 / int4 / FP8-per-row re-coded copy of a dense weight."""
    x = cu._as_bf16(x).contiguous()
    q4, f8 = isinstance(w, Q4Weight), isinstance(w, Fp8RowWeight)
    assert f8 or ((w.group == 64) if q4 else (w.group == 128))
    y = torch.empty(x.shape[0], w.n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    rc = _lib().spark_coded_gemv(cu.P(x), x.stride(0), cu.P(w.q), cu.P(w.sm if q4 else w.scales), 4 if f8 else (3 if q4 else 2),
                                 cu.P(y), w.n, x.shape[0], w.n, w.k, int(out_f32), cu.stream())
    cu.check(rc, "spark_coded_gemv")
    return y


def _resident_bf16(w: QuantWeight, device) -> torch.Tensor:
    """bf16 expansion of a re-coded weight, made once (prefill-size batches; codings without a device kernel yet)."""
    t = getattr(w, "_bf16", None)
    if t is None or t.device != device:
        t = w.dequant().to(torch.bfloat16).to(device)
        w._bf16 = t
    return t


def sf_blocks(sf: torch.Tensor) -> torch.Tensor:
    """E8M0 scale bytes [rows, K/32] -> the tensor core's block layout [ceil(rows/128), K/128, 512]."""
    rows, kb = sf.shape
    out = torch.empty((rows + 127) // 128, kb // 4, 512, dtype=torch.uint8, device=sf.device)
    rc = _lib().spark_mx_sf_to_blocks(cu.P(sf.contiguous()), cu.P(out), rows, kb, cu.stream())
    cu.check(rc, "spark_mx_sf_to_blocks")
    return out


def gemm_mxfp8(a_q, a_sf, w: Mxfp8Weight, out_f32=False):
    """C = (a_q . a_sf) (w.q . w.scales)^T on the block-scaled tcgen05 path.  a_q e4m3 [M,K], a_sf u8 [M, K/32]."""
    M, K = a_q.shape
    assert K == w.k and K % 128 == 0
    wb = getattr(w, "_sf_blocks", None)
    if wb is None or wb.device != a_q.device:
        wb = w._sf_blocks = sf_blocks(w.scales)
    ab = sf_blocks(a_sf)
    c = torch.empty(M, w.n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a_q.device)
    rc = _lib().spark_gemm_mxfp8(cu.P(a_q), cu.P(w.q), cu.P(ab), cu.P(wb), cu.P(c), M, w.n, K, a_q.stride(0), w.q.stride(0),
                                 w.n, int(out_f32), cu.P(cu.status_word(a_q.device)), cu.stream())
    cu.check(rc, "spark_gemm_mxfp8")
    return c


MX_MOE_TC = os.environ.get("SPARK_MX_MOE_TC", "1") == "1"


def moe_mxfp4_tc(x, w: Mxfp4Weight, out_rows, max_items, tiles=None, ntile=None, pair_expert=None, pair_row=None,
                 act=0, limit=0.0, out_f32=False):
    """Grouped expert GEMM on the block-scaled tcgen05 path: MXFP8 activations (quantised here, SwiGLU of a
    [gate | up] input first when act=1) x packed MXFP4 experts, the nibbles expanded by TMA on the way to shared
    memory.  Work items come from the expert-sorted tile list (prefill) or from (token, expert) pairs (decode)."""
    dev = x.device
    E, N, K = w.packed.shape[0], w.n, w.k
    a_q, a_sf = act_quant(x, block=32, act=act, limit=limit)
    items = torch.empty(max_items, 4, dtype=torch.int32, device=dev)
    n_items = torch.empty(1, dtype=torch.int32, device=dev)
    mode = 0 if tiles is not None else 1
    sfa = torch.empty(max_items, K // 128, 512, dtype=torch.uint8, device=dev)
    rc = _lib().spark_mx4_prep(mode, cu.P(tiles), cu.P(ntile), cu.P(pair_expert), cu.P(pair_row),
                               0 if mode == 0 else max_items, max_items, cu.P(a_sf), K // 32, cu.P(items), cu.P(n_items),
                               cu.P(sfa), cu.stream())
    cu.check(rc, "spark_mx4_prep")
    wb = getattr(w, "_sf_blocks", None)
    if wb is None or wb.device != dev:
        wb = w._sf_blocks = sf_blocks(w.scales.reshape(E * N, K // 32))
    c = torch.empty(out_rows, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
    rc = _lib().spark_moe_mxfp4(cu.P(a_q), a_q.stride(0), a_q.shape[0], cu.P(w.packed), cu.P(sfa), cu.P(wb), cu.P(items),
                                cu.P(n_items), max_items, E, N, K, cu.P(c), N, int(out_f32), int(mode == 1),
                                cu.P(cu.status_word(dev)), cu.stream())
    cu.check(rc, "spark_moe_mxfp4")
    return c


def quant_linear(x, w: QuantWeight):
    x = cu._as_bf16(x).contiguous()
    if isinstance(w, Mxfp8Weight) and x.shape[0] <= 16:
        return gemv(x, w)                 # decode rows: bf16 activations, weights decoded in the GEMV
    if isinstance(w, Mxfp8Weight):
        # activations are quantised to MXFP8 (1 x 32 E8M0 scales) and both operands go to the tensor core as they are
        a_q, a_sf = act_quant(x, block=32)
        return gemm_mxfp8(a_q, a_sf, w)
    if isinstance(w, (Fp8BlockWeight, Mxfp4Weight)):
        if x.shape[0] <= 16:
            return gemv(x, w)
        wt = dequant_bf16(w, cu.scratch("mx_deq", w.n * w.k, torch.bfloat16, x.device))
        return cu.gemm_bf16(x, wt)
    if isinstance(w, (Q8Weight, Q4Weight, Fp8RowWeight)) and x.shape[0] <= 16 and w.n % 16 == 0 and w.k % 128 == 0:
        return coded_gemv(x, w)
    return cu.dense_linear(x, _resident_bf16(w, x.device))


MX_DECODE_TC = os.environ.get("SPARK_MX_DECODE_TC", "1") == "1"


def expert_gemv(x, w, pairs, pair_expert, pair_row, act, limit, out_f32):
    if MX_DECODE_TC and isinstance(w, Mxfp4Weight) and w.n % 128 == 0 and w.k % 128 == 0:
        # decode pairs on the block-scaled tensor-core path (activations quantised to MXFP8)
        return moe_mxfp4_tc(cu._as_bf16(x).contiguous(), w, pairs, pairs, pair_expert=pair_expert, pair_row=pair_row,
                            act=act, limit=limit, out_f32=out_f32)
    return gemv(x, w, items=pairs, rows_per_item=1, pair_expert=pair_expert, pair_row=pair_row, act=act, limit=limit,
                out_f32=out_f32)


MX_MOE_FUSED = os.environ.get("SPARK_MX_MOE_FUSED", "1") == "1"


def mx_mgemm(x, w: Mxfp4Weight, tiles, ntile, max_tiles, act=0, limit=0.0, out_f32=False):
    """Rows in expert order x packed MXFP4 experts -> [P, N] (fused decode, <= 64 rows per work item)."""
    Pn = x.shape[0]
    y = torch.empty(Pn, w.n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    rc = _lib().spark_mx_mgemm(cu.P(x), x.stride(0), cu.P(w.packed), cu.P(w.scales), w.n * w.k // 2, w.n * (w.k // 32),
                               cu.P(tiles), cu.P(ntile), max_tiles, cu.P(y), w.n, int(out_f32), w.n, w.k, act, float(limit),
                               cu.stream())
    cu.check(rc, "spark_mx_mgemm")
    return y


def grouped_experts(a, wgu, wd, ids, perm, tiles, ntile, max_tiles, c):
    """Rows in expert order through gate/up (+SwiGLU) and down; returns fp32 [P, H]."""
    E, F2, H = wgu.packed.shape[0] if isinstance(wgu, Mxfp4Weight) else wgu.q.shape[0], wgu.n, wgu.k
    dev = a.device
    if MX_MOE_TC and isinstance(wgu, Mxfp4Weight) and F2 % 256 == 0 and H % 128 == 0:
        # block-scaled tensor-core path: MXFP8 activations x packed MXFP4 experts, no decoded copy of the weights
        Pn = a.shape[0]
        gu = moe_mxfp4_tc(cu._as_bf16(a).contiguous(), wgu, Pn, max_tiles, tiles=tiles, ntile=ntile)
        return moe_mxfp4_tc(gu, wd, Pn, max_tiles, tiles=tiles, ntile=ntile, act=1, limit=c.swiglu_limit, out_f32=True)
    if MX_MOE_FUSED and isinstance(wgu, Mxfp4Weight) and F2 % 128 == 0 and H % 128 == 0 and a.shape[0] <= 512 * E:
        # packed experts straight into the MMA: the weights cross HBM once, SwiGLU is applied while the down
        # projection stages its input
        gu = mx_mgemm(cu._as_bf16(a).contiguous(), wgu, tiles, ntile, max_tiles)
        return mx_mgemm(gu, wd, tiles, ntile, max_tiles, act=1, limit=c.swiglu_limit, out_f32=True)
    wt = dequant_bf16(wgu, cu.scratch("mx_deq_gu", E * F2 * H, torch.bfloat16, dev))
    act = cu.grouped_gemm(a, wt.view(E * F2, H), tiles, ntile, max_tiles, E, F2, F2 // 2, 1, c.swiglu_limit)
    wt2 = dequant_bf16(wd, cu.scratch("mx_deq_d", E * H * (F2 // 2), torch.bfloat16, dev))
    return cu.grouped_gemm(act, wt2.view(E * H, F2 // 2), tiles, ntile, max_tiles, E, H, H, 0)
