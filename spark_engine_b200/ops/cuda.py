"""ctypes bindings of libspark_kernels.so and the CUDA implementations of the ops.

The kernels take raw pointers, shapes and a stream (C ABI); this module owns the glue: output
allocation, persistent scratch (so captured CUDA graphs replay against fixed addresses), the device
status word that bounded waits report to, and dispatch between GEMV-class (<= 16 rows) and
GEMM-class (tcgen05) kernels.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import Optional

import torch

from ..quant.formats import Exl3Weight, Fp8BlockWeight, Mxfp4Weight, QuantWeight

_LIB = None
_here = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SPARK_KERNEL_LIB") or os.path.join(os.path.dirname(_here), "_lib", "libspark_kernels.so")

vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_longlong, C.c_float

_SIGS = {
    "spark_gemm_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp],
    "spark_gemm_bf16_swiglu": [vp, vp, vp, i32, i32, i32, i32, i32, i32, f32, vp, vp],
    "spark_gemm_grouped_bf16": [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, i32, f32, i32, vp, vp],
    "spark_gemv_bf16": [vp, i32, vp, i64, i32, vp, i32, i32, i32, i32, i32, vp, vp, i32, f32, i32, vp],
    "spark_gemv_bf16_items": [vp, i32, i64, vp, i64, i32, vp, i32, i64, i32, i32, i32, i32, vp, i32, vp],
    "spark_add_rmsnorm": [vp, i32, vp, vp, vp, i32, i32, f32, i32, vp],
    "spark_rmsnorm_bf16": [vp, vp, vp, i32, i32, f32, i32, vp],
    "spark_embed": [vp, vp, vp, i32, i32, vp, i32, vp],
    "spark_decode_advance": [vp, vp, i32, vp],
    "spark_moe_router_topk": [vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, vp, f32, i32, i32, i32, i32, i32, i32,
                              i32, vp, vp, vp, vp, vp, vp],
    "spark_moe_combine_norm": [vp, vp, vp, i32, i32, i32, vp, vp, f32, i32, vp, vp, vp, vp],
    "spark_swiglu": [vp, vp, i32, i32, f32, vp],
    "spark_argmax": [vp, i32, i32, vp, vp, vp, vp, vp],
    "spark_gumbel_perturb": [vp, i32, i32, i32, vp, vp, vp, i32, vp],
    "spark_token_prob_part": [vp, i32, i32, i32, vp, i32, i32, vp, i32, vp, vp],
    "spark_token_prob_final": [vp, i32, i32, vp, vp, i32, vp],
    "spark_mhc_site": [vp, i32, i32, i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i32, f32, i32, vp, vp],
    "spark_hc_gated_site": [vp, i32, i32, i32, i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, f32, vp, vp],
    "spark_ngram_gate": [vp, vp, vp, vp, vp, i32, i32, f32, vp],
    "spark_draft_topk": [vp, i32, i32, i32, vp, vp, vp],
    "spark_draft_path": [vp, vp, vp, vp, i32, i32, i32, vp, vp, vp, vp, vp],
    "spark_add": [vp, i32, vp, C.c_long, vp],
    "spark_f32_to_bf16": [vp, vp, C.c_long, vp],
    "spark_gather_rows_bf16": [vp, vp, vp, i32, i32, vp],
    "spark_gdn_seq": [vp, i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, f32, i32, vp, vp, i32, i32],
    "spark_mla_prep": [vp, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                       vp, vp, vp, i32],
    "spark_mla_qrope": [vp, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp],
    "spark_mla_attn": [vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, f32, vp, vp, vp, vp, vp, i32],
    "spark_kda_chunk_prefill": [vp, i32, vp, vp, i32, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, vp, vp, vp, vp, i32,
                                i32, i32, vp],
    "spark_kda_seq": [vp, i32, vp, vp, i32, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32, i32, vp, vp, i32, i32],
    "spark_attn_prefill": [vp, vp, vp, vp, vp, i32, i32, vp, i32, i32, vp, i32, i32, i32, f32, vp],
    "spark_attn_prefill_masked": [vp, vp, vp, vp, vp, i32, i32, vp, i32, i32, vp, i32, i32, i32, f32, vp, vp, i32, i32, vp,
                                  i32, vp],
    "spark_exl3_mgemm": [vp, i32, vp, vp, i64, i64, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32, i32, vp],
    "spark_gdn_chunk_prefill": [vp, i32, vp, i32, vp, vp, vp, vp, vp, vp, vp, i32, vp, i32, vp, vp, vp, vp, i32, i32, i32,
                                i32, f32, vp],
    "spark_attn_prep": [vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, f32, vp, vp, vp, vp, vp, vp, vp,
                        vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp],
    "spark_attn_decode": [vp, vp, vp, vp, vp, i32, vp, vp, vp, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, i32,
                          f32, vp, vp, vp, vp, vp, i32],
    "spark_moe_route": [vp, i32, i32, i32, i32, i32, vp, f32, i32, vp, vp, vp, vp, vp, i32, i32],
    "spark_moe_sort": [vp, i32, i32, vp, vp, vp, vp, vp, vp, vp],
    "spark_moe_combine": [vp, vp, i32, vp, vp, i32, i32, vp, vp, i32, vp, vp, vp],
    "spark_exl3_gemv": [vp, i32, vp, vp, vp, i64, i64, i64, vp, i32, i32, vp, vp, i32, i32, i32, i32, i32, i32,
                        f32, i32, vp, vp, i32],
    "spark_exl3_reconstruct": [vp, vp, i32, i32, i32, vp, i32],
    "spark_exl3_reconstruct_bits": [vp, vp, i32, i32, i32, vp, i32, i32],
    "spark_exl3_had_rows": [vp, i32, vp, vp, i32, i32, i32, i32, vp, vp, i64],
}


# kernels launched by one call of each entry point (for the launch counter)
_KERNELS_PER_CALL = {"spark_attn_decode": 2, "spark_moe_sort": 3, "spark_argmax": 2, "spark_hc_gated_site": 2}
_launches = 0


class _Counting:
    """Proxy over the shared library that counts kernel launches made through it."""

    def __init__(self, dll):
        self._dll = dll
        self._fns = {}

    def __getattr__(self, name):
        fn = self._fns.get(name)
        if fn is None:
            raw = getattr(self._dll, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*a, _raw=raw, _n=n):
                global _launches
                _launches += _n
                return _raw(*a)
            self._fns[name] = fn
        return fn


def launch_count() -> int:
    return _launches


def add_launches(n: int):
    global _launches
    _launches += n


def reset_launch_count():
    global _launches
    _launches = 0


from ..utils import debug as dbg

def lib():
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python -m spark_engine_b200.build` (the CUDA kernels are required "
                "on a GPU; there is no silent eager fallback)")
        dll = C.CDLL(LIB_PATH)
        from ..utils import precision
        precision.ensure()                  # library GEMMs that remain on the path: fp32 accumulation, TF32 only by flag
        _LIB = _Counting(dll)
        for name, sig in _SIGS.items():
            fn = getattr(dll, name, None)
            if fn is not None:
                fn.argtypes = sig
                fn.restype = i32 if name not in ("spark_add_rmsnorm", "spark_rmsnorm_bf16", "spark_embed", "spark_swiglu",
                                                 "spark_argmax", "spark_add", "spark_f32_to_bf16",
                                                 "spark_gather_rows_bf16") else None
    return _LIB


def P(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def stream():
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str):
    if rc:
        raise RuntimeError(f"{what} failed with code {rc}")


# ----------------------------------------------------------------------------- persistent buffers
_status = {}
_scratch = {}
_retired = []


def status_word(device) -> torch.Tensor:
    """int32[4] device status: kernels whose bounded waits run out write {code, detail...} here."""
    d = torch.device(device)
    key = d.index if d.index is not None else torch.cuda.current_device()     # "cuda" and "cuda:0" are one word
    if key not in _status:
        _status[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _status[key]


def read_status(device) -> tuple:
    st = status_word(device).tolist()
    return tuple(st)


def reset_status(device):
    status_word(device).zero_()


def clear_status(device):
    status_word(device).zero_()


def scratch(name: str, numel: int, dtype, device, zero: bool = False) -> torch.Tensor:
    """Persistent scratch keyed by name (grows, never shrinks): fixed addresses for graph replay."""
    key = (name, dtype, str(device))
    t = _scratch.get(key)
    if t is None or t.numel() < numel:
        if t is not None:
            _retired.append(t)      # captured graphs may still point at the old buffer: keep it alive
        t = (torch.zeros if zero else torch.empty)(max(numel, 1), dtype=dtype, device=device)
        _scratch[key] = t
    if dbg.POISON and not zero:
        dbg.poison(t[:max(numel, 1)])
    return t


def scratch_bytes() -> int:
    return sum(t.numel() * t.element_size() for t in _scratch.values())


# ----------------------------------------------------------------------------- decode rounds
DECODE_ROWS_MAX = 16
FUSED_DECODE = os.environ.get("SPARK_FUSED_DECODE", "1") == "1"
SHARED_AS_PAIR = os.environ.get("SPARK_SHARED_PAIR", "0") == "1"
FUSED_COMBINE = os.environ.get("SPARK_FUSED_COMBINE", "1") == "1"


class PendingMoe:
    """Expert outputs of a decode round that have not been combined yet: y fp32 [R * slots, H] in pair order.  The
    slot-order combine runs fused with the residual update and the next RMSNorm (`add_rmsnorm`), or on its own
    (`tensor()`)."""

    def __init__(self, y, wts, ids, slots, R, H, shared=None, sg=None):
        self.y, self.wts, self.ids, self.slots, self.R, self.H, self.shared, self.sg = y, wts, ids, slots, R, H, shared, sg

    def tensor(self) -> torch.Tensor:
        out = torch.empty(self.R, self.H, dtype=torch.bfloat16, device=self.y.device)
        rc = lib().spark_moe_combine(None, P(self.y), 1, None, P(self.wts), self.R, self.slots, P(self.shared), P(self.sg),
                                     self.H, P(out), stream(), P(self.ids))
        check(rc, "spark_moe_combine")
        return out


# ----------------------------------------------------------------------------- dense linear
def _as_bf16(x):
    return x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out_f32: bool = False, fmt: int = 1) -> torch.Tensor:
    """C[M,N] = A[M,K] B[N,K]^T on tcgen05.  fmt 1 = bf16 operands, 0 = fp16 operands."""
    M, K = a.shape
    N = b.shape[0]
    assert a.stride(1) == 1 and b.stride(1) == 1 and K % 8 == 0
    c = torch.empty(M, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=a.device)
    rc = lib().spark_gemm_bf16(P(a), P(b), P(c), M, N, K, a.stride(0), b.stride(0), N, int(out_f32), fmt,
                               P(status_word(a.device)), stream())
    check(rc, "spark_gemm_bf16")
    return c


def gemv_bf16(x, w, items=1, rows_per_item=None, pair_expert=None, pair_row=None, act=0, limit=0.0, out_f32=False,
              expert_stride=0, n=None, k=None, out=None, ldx=None):
    rows_per_item = rows_per_item if rows_per_item is not None else x.shape[0]
    n = n if n is not None else w.shape[-2]
    k = k if k is not None else w.shape[-1]
    if out is None:
        y = torch.empty(items * rows_per_item, n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
        ldy = n
    else:
        y, ldy = out, out.stride(0)
        out_f32 = out.dtype == torch.float32
    if dbg.CHECK:
        dbg.check_index("gemv_bf16 pair_expert", pair_expert, 0, w.shape[0] if w.dim() == 3 else 1, allow=-1, count=items)
        dbg.check_index("gemv_bf16 pair_row", pair_row, 0, x.shape[0], count=items)
    rc = lib().spark_gemv_bf16(P(x), ldx if ldx is not None else x.stride(0), P(w), expert_stride, w.stride(-2), P(y), ldy,
                               items, rows_per_item, n, k, P(pair_expert), P(pair_row), act, float(limit), int(out_f32),
                               stream())
    check(rc, "spark_gemv_bf16")
    return y


def gemv_bf16_items(x, ldx, x_item_stride, w, expert_stride, ldw, y, ldy, y_item_stride, items, rows_per_item, n, k,
                    pair_expert):
    """Per-item GEMV over strided slices: item i multiplies rows x[i * x_item_stride + r * ldx] (r < rows_per_item) by
    matrix pair_expert[i] of `w` and writes y[i * y_item_stride + r * ldy].  Strides in elements."""
    if dbg.CHECK:
        dbg.check_index("gemv_bf16_items pair_expert", pair_expert, 0, w.shape[0], count=items)
    rc = lib().spark_gemv_bf16_items(P(x), ldx, x_item_stride, P(w), expert_stride, ldw, P(y), ldy, y_item_stride, items,
                                     rows_per_item, n, k, P(pair_expert), int(y.dtype == torch.float32), stream())
    check(rc, "spark_gemv_bf16_items")
    return y


def dense_linear(x: torch.Tensor, w: torch.Tensor, out_f32: bool = False) -> torch.Tensor:
    if w.dtype != torch.bfloat16:
        raise TypeError("dense weights must be bf16 on the device")
    x = _as_bf16(x)
    R = x.shape[0]
    if R <= 16:
        return gemv_bf16(x.contiguous(), w, out_f32=out_f32)
    return gemm_bf16(x.contiguous(), w, out_f32)


# ----------------------------------------------------------------------------- EXL3
def _pick_slices(K: int, items: int = 1) -> int:
    """K-slices per 128-column strip = CTAs of one cluster (<= 8): aim at 256-deep slices so that one
    batch of loads per warp covers the whole slice.  SPARK_EXL3_S / SPARK_EXL3_S_PAIRS force the count for
    single-matrix / per-pair launches."""
    blocks = K // 128
    forced = int(os.environ.get("SPARK_EXL3_S_PAIRS" if items > 1 else "SPARK_EXL3_S", "0"))
    if forced and blocks % forced == 0:
        return forced
    best = 1
    for s in range(1, 9):
        if blocks % s == 0 and K // s >= 128:
            best = s
            if K // s <= 256:
                break
    return best


def exl3_gemv(x, w: Exl3Weight, items=1, rows_per_item=None, pair_expert=None, pair_row=None, act=0, limit=0.0,
              out_f32=False, pairs_early: bool = False):
    """`pairs_early`: the pair tables were written at least two launches back, so the kernel may read them and issue
    its weight loads before it waits for its predecessor (programmatic dependent launch)."""
    assert w.bits == 4, "the GEMV kernel handles 4 bpw"
    rows_per_item = rows_per_item if rows_per_item is not None else x.shape[0]
    K, N = w.k, w.n
    if dbg.CHECK:
        dbg.check_index("exl3_gemv pair_expert", pair_expert, 0, w.trellis.shape[0] if w.experts else 1, allow=-1, count=items)
        dbg.check_index("exl3_gemv pair_row", pair_row, 0, x.shape[0], count=items)
    S = _pick_slices(K, items)
    dev = x.device
    y = torch.empty(items * rows_per_item, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=dev)
    tw = (K // 16) * (N // 16) * 32
    es = (tw, K, N) if w.experts else (0, 0, 0)
    rc = lib().spark_exl3_gemv(P(x), x.stride(0), P(w.trellis), P(w.suh), P(w.svh), es[0], es[1], es[2], P(y), N,
                               int(out_f32), P(pair_expert), P(pair_row), items, rows_per_item, K, N, S,
                               act, float(limit), 0 if w.kind == "mul1" else 1, stream(), None, int(pairs_early))
    check(rc, "spark_exl3_gemv")
    return y


def exl3_reconstruct(w: Exl3Weight, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inner codebook weights as fp16 [.., N, K] (K-major B operand)."""
    E = w.trellis.shape[0] if w.experts else 1
    if out is None:
        out = torch.empty((E, w.n, w.k) if w.experts else (w.n, w.k), dtype=torch.float16, device=w.trellis.device)
    if w.bits != 4:
        rc = lib().spark_exl3_reconstruct_bits(P(w.trellis), P(out), w.k, w.n, 0 if w.kind == "mul1" else 1, stream(), E, w.bits)
        check(rc, "spark_exl3_reconstruct_bits")
        return out
    rc = lib().spark_exl3_reconstruct(P(w.trellis), P(out), w.k, w.n, 0 if w.kind == "mul1" else 1, stream(), E)
    check(rc, "spark_exl3_reconstruct")
    return out


def exl3_had_rows(x, scale, post: bool, row_expert=None, expert_stride=0):
    R, Cn = x.shape
    y = torch.empty(R, Cn, dtype=torch.bfloat16 if post else torch.float16, device=x.device)
    rc = lib().spark_exl3_had_rows(P(x), x.stride(0), P(scale), P(y), Cn, R, Cn, int(post), P(row_expert), stream(),
                                   expert_stride)
    check(rc, "spark_exl3_had_rows")
    return y


def exl3_fold(w: Exl3Weight) -> torch.Tensor:
    """The dense bf16 weight [N, K] of an EXL3 tensor, made on the device: inner codebook values (any bit width), then
    the input-side Hadamard + sign/scale along K and the output-side ones along N folded in, so that y = x @ W^T needs no
    Hadamard passes at run time.  For tensors that are cheaper to keep dense than to decode on every call (a sub-vocabulary
    head, a drafter's head).  Reference: engine-rs/shim/qwen_exl3.cuh:661 `fold_kernel`."""
    assert not w.experts
    wt = exl3_reconstruct(w).float()                                          # inner^T [N, K]
    a = exl3_had_rows(wt, w.suh, post=True)                                   # rows n: had128 along K, x suh[k]
    b = exl3_had_rows(a.t().float().contiguous(), w.svh, post=True)           # rows k: had128 along N, x svh[n]
    return b.t().contiguous()


def _pick_mg_slices(K: int, target: int) -> int:
    """K-slices (cluster size) of the grouped EXL3 GEMM: the smallest of 1/2/4/8 that brings the slice to <= target."""
    blocks = K // 128
    best = 1
    for s in (1, 2, 4, 8):
        if blocks % s == 0:
            best = s
            if K // s <= target:
                break
    return best


def exl3_mgemm(xh, w: Exl3Weight, tiles, ntile, max_tiles, out_f32=False, rows_per_item=64):
    """Rows in expert order (fp16, input Hadamard applied) x expert trellises -> [P, N]; output Hadamard fused."""
    Pn, K = xh.shape
    y = torch.empty(Pn, w.n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=xh.device)
    t = w.trellis
    # slice depth: two (64-row items) or three (32-row items) CTAs per SM must fit their rows + reduction buffers
    target = int(os.environ.get("SPARK_MG_KS", "512" if rows_per_item == 32 else "256"))
    rc = lib().spark_exl3_mgemm(P(xh), xh.stride(0), P(t), P(w.svh), (K // 16) * (w.n // 16) * 32, w.n, P(tiles),
                                P(ntile), max_tiles, P(y), w.n, int(out_f32), K, w.n, _pick_mg_slices(K, target),
                                0 if w.kind == "mul1" else 1, rows_per_item, stream())
    check(rc, "spark_exl3_mgemm")
    return y


EXL3_RESIDENT_MAX_BYTES = int(os.environ.get("SPARK_EXL3_RESIDENT_MB", "4096")) << 20
_exl3_resident_bytes = 0


def _exl3_resident(w: Exl3Weight) -> Optional[torch.Tensor]:
    """fp16 inner weights of a tensor whose bit width has no GEMV kernel (everything but 4 bpw), decoded once and kept
    for decode rows, within a byte budget (a 6 bpw head of 152K x 2048 is 622 MB)."""
    global _exl3_resident_bytes
    t = getattr(w, "_inner_fp16", None)
    if t is None:
        need = w.n * w.k * 2
        if _exl3_resident_bytes + need > EXL3_RESIDENT_MAX_BYTES:
            return None
        t = exl3_reconstruct(w)
        w._inner_fp16 = t
        _exl3_resident_bytes += need
    return t


def exl3_linear(x, w: Exl3Weight):
    x = _as_bf16(x).contiguous()
    if x.shape[0] <= 16 and w.bits == 4:
        return exl3_gemv(x, w)
    xh = exl3_had_rows(x, w.suh, post=False)
    wt = _exl3_resident(w) if (x.shape[0] <= 16 and not w.experts) else None
    if wt is None:
        wt = exl3_reconstruct(w, scratch("exl3_recon", w.n * w.k, torch.float16, x.device)[: w.n * w.k].view(w.n, w.k))
    acc = gemm_bf16(xh, wt, out_f32=True, fmt=0)
    return exl3_had_rows(acc, w.svh, post=True)


def quant_linear(x, w: QuantWeight):
    if isinstance(w, Exl3Weight):
        return exl3_linear(x, w)
    from . import mx
    return mx.quant_linear(x, w)


# ----------------------------------------------------------------------------- elementwise
def _delta_tensor(delta):
    """Plain tensor of a deferred block output (a row-parallel product or an uncombined MoE)."""
    if delta is None or isinstance(delta, torch.Tensor):
        return delta
    if isinstance(delta, PendingMoe):
        return delta.tensor()
    return linear_any(delta.x, delta.w)            # ops.Partial


def add_rmsnorm(delta, res, w, eps, one_plus=False):
    R, H = res.shape
    assert res.dtype == torch.float32 and res.is_contiguous()
    out = torch.empty(R, H, dtype=torch.bfloat16, device=res.device)
    if isinstance(delta, PendingMoe) and H % 128 == 0 and H <= 8192 and FUSED_COMBINE:
        # decode round: slot-order combine + residual add + RMSNorm in one launch
        rc = lib().spark_moe_combine_norm(P(delta.y), P(delta.wts), P(delta.ids), R, delta.slots, H, P(res), P(w), float(eps),
                                          int(one_plus), P(out), P(delta.shared), P(delta.sg), stream())
        check(rc, "spark_moe_combine_norm")
        return out, res
    delta = _delta_tensor(delta)
    if delta is not None:
        delta = delta.contiguous()
    lib().spark_add_rmsnorm(P(delta), int(delta is not None and delta.dtype == torch.float32), P(res), P(w), P(out), R, H,
                            float(eps), int(one_plus), stream())
    return out, res


def rmsnorm(x, w, eps, one_plus=False):
    R, H = x.shape
    out = torch.empty(R, H, dtype=torch.bfloat16, device=x.device)
    x = x.contiguous()
    if x.dtype == torch.float32:
        lib().spark_add_rmsnorm(None, 0, P(x), P(w), P(out), R, H, float(eps), int(one_plus), stream())
    else:
        lib().spark_rmsnorm_bf16(P(x), P(w), P(out), R, H, float(eps), int(one_plus), stream())
    return out


def embed(table, ids32):
    R, H = ids32.shape[0], table.shape[1]
    dbg.check_index("embed token ids", ids32, 0, table.shape[0])
    out = torch.empty(R, H, dtype=torch.float32, device=table.device)
    lib().spark_embed(P(table), P(ids32), P(out), R, H, stream(), table.shape[0], P(status_word(table.device)))
    return out


def swiglu(gu, limit=0.0):
    R, F2 = gu.shape
    out = torch.empty(R, F2 // 2, dtype=torch.bfloat16, device=gu.device)
    lib().spark_swiglu(P(gu.contiguous()), P(out), R, F2 // 2, float(limit), stream())
    return out


def residual_add(res, delta):
    lib().spark_add(P(delta.contiguous()), int(delta.dtype == torch.float32), P(res), res.numel(), stream())
    return res


def argmax(logits):
    R, V = logits.shape
    ids = torch.empty(R, dtype=torch.int32, device=logits.device)
    pv = scratch("argmax_v", R * 64, torch.float32, logits.device)
    pi = scratch("argmax_i", R * 64, torch.int32, logits.device)
    lib().spark_argmax(P(logits.contiguous()), R, V, P(ids), None, P(pv), P(pi), stream())
    return ids


def gumbel_perturb(logits, temps, seeds, positions, offset):
    """In place on fp32 logits [R, V]: rows with temperature > 0 become logits / T + Gumbel noise of the global ids."""
    R, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    check(lib().spark_gumbel_perturb(P(logits), R, V, logits.stride(0), P(temps), P(seeds), P(positions), int(offset), stream()),
          "gumbel_perturb")
    return logits


def token_prob(logits, ids32, tp=None):
    """softmax(logits)[ids] per row -> fp32 [R]; `logits` is this rank's vocabulary slice under `tp` (the per-rank
    (max, sum) pairs and the owner's logit go through the rank-ordered all-reduce, so every rank gets the same bits)."""
    R, V = logits.shape
    rank, world = (tp.rank, tp.world) if tp is not None else (0, 1)
    assert world <= 8 and logits.dtype == torch.float32 and logits.stride(1) == 1
    ms = torch.zeros(R, 16, dtype=torch.float32, device=logits.device)
    lt = torch.empty(R, dtype=torch.float32, device=logits.device)
    check(lib().spark_token_prob_part(P(logits), R, V, logits.stride(0), P(ids32), rank * V, rank, P(ms), 16, P(lt), stream()),
          "token_prob_part")
    lt1 = lt
    if world > 1:
        ms = tp.allreduce(ms).clone()          # the packet channel's output buffer is reused by the next call
        lt1 = tp.allreduce(lt.view(R, 1))[:, 0].contiguous()
    out = torch.empty(R, dtype=torch.float32, device=logits.device)
    check(lib().spark_token_prob_final(P(ms), ms.stride(0), world, P(lt1), P(out), R, stream()), "token_prob_final")
    return out


# ----------------------------------------------------------------------------- hyper-connections
def _hc_scratch(T, D, gated, dev):
    dll = lib()._dll
    fn = dll.spark_hc_partial_floats
    fn.restype, fn.argtypes = i32, [i32, i32, i32]
    return (scratch("hc_partial", fn(T, D, int(gated)), torch.float32, dev),
            scratch("hc_counter", max(T, 1024), torch.int32, dev, zero=True))


def _hc_weights(w):
    """bf16 copies of the matrices, fp32 vectors (cached on the dict)."""
    c = w.get("_dev")
    if c is None:
        c = {k: (v.to(torch.bfloat16).contiguous() if (torch.is_tensor(v) and v.dim() == 2 and k != "norm") else
                 (v.float().contiguous() if torch.is_tensor(v) else v)) for k, v in w.items() if k != "_dev"}
        w["_dev"] = c
    return c


def mhc_site(X, pend, w, iters, eps, mode=1, norm=None):
    """One launch: apply the previous block's update `pend` = (x, post, comb) to the streams X [T,S,D] (out of place: the
    updated streams are returned), then (mode 1) the next block's mixed row with its post / comb, or (mode 2) the
    stream mean and its RMSNorm (`norm`).  Returns (X', h bf16 [T,D], post, comb) or (X', h, mean fp32)."""
    T, S, D = X.shape
    assert X.dtype == torch.float32 and X.is_contiguous()
    dev = X.device
    x, post_in, comb_in = pend if pend is not None else (None, None, None)
    Xn = X
    if x is not None:
        x = x.contiguous()
        assert x.dtype in (torch.float32, torch.bfloat16)
        Xn = torch.empty_like(X)
    h = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    partial, counter = _hc_scratch(T, D, False, dev)
    xf = int(x is not None and x.dtype == torch.float32)
    if mode == 1:
        c = _hc_weights(w)
        post = torch.empty(T, S, dtype=torch.float32, device=dev)
        comb = torch.empty(T, S, S, dtype=torch.float32, device=dev)
        rc = lib().spark_mhc_site(P(X), T, S, D, P(x), xf, P(post_in), P(comb_in), P(c["fn"]), P(c["scale"]), P(c["base"]),
                                  P(c["norm"]), P(h), None, P(post), P(comb), P(partial), P(counter), int(iters), float(eps), 1,
                                  stream(), P(Xn) if x is not None else None)
        check(rc, "spark_mhc_site")
        return Xn, h, post, comb
    mean = torch.empty(T, D, dtype=torch.float32, device=dev)
    rc = lib().spark_mhc_site(P(X), T, S, D, P(x), xf, P(post_in), P(comb_in), None, None, None, P(norm.float().contiguous()),
                              P(h), P(mean), None, None, P(partial), P(counter), int(iters), float(eps), 2, stream(),
                              P(Xn) if x is not None else None)
    check(rc, "spark_mhc_site")
    return Xn, h, mean


def hc_gated_site(X, pend, w, eps):
    """Two launches: apply `pend` = (x, post) to the streams (out of place), logits of the gate (and the next post), then
    the mixed row.  Returns (X', h bf16, h fp32, post or None)."""
    T, S, D = X.shape
    assert X.dtype == torch.float32 and X.is_contiguous()
    dev = X.device
    c = _hc_weights(w)
    x, post_in = pend if pend is not None else (None, None)
    Xn = X
    if x is not None:
        x = x.contiguous()
        Xn = torch.empty_like(X)
    r = c["down"].shape[0]
    h = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    hf = torch.empty(T, D, dtype=torch.float32, device=dev)
    tvec = torch.empty(T, r + S, dtype=torch.float32, device=dev)
    post = torch.empty(T, S, dtype=torch.float32, device=dev) if "inject" in c else None
    partial, counter = _hc_scratch(T, D, True, dev)
    rc = lib().spark_hc_gated_site(P(X), T, S, D, r, P(x), int(x is not None and x.dtype == torch.float32), P(post_in),
                                   P(c["norm"]), P(c["down"]), P(c.get("inject")), P(c["up"]), P(tvec), P(post), P(h), P(hf),
                                   P(partial), P(counter), float(eps), stream(), P(Xn) if x is not None else None)
    check(rc, "spark_hc_gated_site")
    return Xn, h, hf, post


def ngram_gate(X, key, val, nk, nq, eps):
    """X (fp32, in place) += sigmoid(sign(d) sqrt|d|) * val with d the scaled dot of the normalised key and hidden rows."""
    R, H = X.shape
    check(lib().spark_ngram_gate(P(X), P(key.contiguous()), P(val.contiguous()), P(nk), P(nq), R, H, float(eps), stream()),
          "spark_ngram_gate")
    return X


def draft_topk(logits, K):
    """[J, V] fp32 logits -> (ids int32 [J, K], log-probabilities [J, K]) sorted descending, ties -> lowest id."""
    J, V = logits.shape
    ids = torch.empty(J, K, dtype=torch.int32, device=logits.device)
    unary = torch.empty(J, K, dtype=torch.float32, device=logits.device)
    check(lib().spark_draft_topk(P(logits), J, V, K, P(ids), P(unary), stream()), "spark_draft_topk")
    return ids, unary


def draft_path(unary, ids, eu, ev):
    """Edge scores <eu[j, a], ev[j+1, b]> and the greedy path through (unary + edge): (edges, path, tokens, conf)."""
    J, K = unary.shape
    r = eu.shape[-1]
    dev = unary.device
    edges = torch.empty(max(J - 1, 0), K, K, dtype=torch.float32, device=dev)
    path = torch.empty(J, dtype=torch.int32, device=dev)
    tok = torch.empty(J, dtype=torch.int32, device=dev)
    conf = torch.empty(J, dtype=torch.float32, device=dev)
    check(lib().spark_draft_path(P(unary), P(ids), P(eu), P(ev), J, K, r, P(edges), P(path), P(tok), P(conf), stream()),
          "spark_draft_path")
    return edges, path, tok, conf


def gather_rows(src, idx32):
    R, H = idx32.shape[0], src.shape[1]
    dbg.check_index("gather_rows indices", idx32, 0, src.shape[0])
    out = torch.empty(R, H, dtype=torch.bfloat16, device=src.device)
    lib().spark_gather_rows_bf16(P(src), P(idx32), P(out), R, H, stream())
    return out


# ----------------------------------------------------------------------------- MoE
ROUTER_KIND = {"softmax": 0, "sigmoid_bias": 1, "sqrt_softplus": 2}


def moe_route(h, w, c, e_lo=0, e_hi=None):
    R = h.shape[0]
    dev = h.device
    logits = dense_linear(h, w["gate"], out_f32=True)
    wts = torch.empty(R, c.top_k, dtype=torch.float32, device=dev)
    ids = torch.empty(R, c.top_k, dtype=torch.int32, device=dev)
    prow = torch.empty(R, c.top_k, dtype=torch.int32, device=dev)
    sg = torch.empty(R, dtype=torch.float32, device=dev) if c.shared_gate else None
    rc = lib().spark_moe_route(P(logits), logits.stride(0), R, c.n_experts, c.top_k, ROUTER_KIND[c.router],
                               P(w.get("bias")), float(c.route_scale), int(c.shared_gate), P(wts), P(ids), P(prow), P(sg),
                               stream(), e_lo, c.n_experts if e_hi is None else e_hi)
    check(rc, "spark_moe_route")
    return wts, ids, prow, sg


def _expert_gemv(x, w, pairs, pair_expert, pair_row, act, limit, out_f32, pairs_early=False):
    if isinstance(w, Exl3Weight):
        return exl3_gemv(x, w, items=pairs, rows_per_item=1, pair_expert=pair_expert, pair_row=pair_row, act=act,
                         limit=limit, out_f32=out_f32, pairs_early=pairs_early)
    if isinstance(w, QuantWeight):
        from . import mx
        return mx.expert_gemv(x, w, pairs, pair_expert, pair_row, act, limit, out_f32)
    E, N, K = w.shape
    return gemv_bf16(x, w, items=pairs, rows_per_item=1, pair_expert=pair_expert, pair_row=pair_row, act=act,
                     limit=limit, out_f32=out_f32, expert_stride=N * K, n=N, k=K)


def moe_sort(ids, E):
    Pn = ids.numel()
    dev = ids.device
    dbg.check_index("moe_sort expert ids", ids, 0, E, allow=-1)
    perm = torch.zeros(Pn, dtype=torch.int32, device=dev)      # entries past the local pairs stay valid indices
    inv = torch.empty(Pn, dtype=torch.int32, device=dev)
    offs = torch.empty(E + 1, dtype=torch.int32, device=dev)
    max_tiles = (Pn + 127) // 128 + E
    tiles = torch.empty(max_tiles, 4, dtype=torch.int32, device=dev)
    ntile = torch.empty(1, dtype=torch.int32, device=dev)
    hist = scratch("moe_hist", ((Pn + 255) // 256) * E, torch.int32, dev)
    rc = lib().spark_moe_sort(P(ids), Pn, E, P(perm), P(inv), P(offs), P(tiles), P(ntile), P(hist), stream())
    check(rc, "spark_moe_sort")
    return perm, inv, offs, tiles, ntile, max_tiles


def grouped_gemm(a, b, tiles, ntile, max_tiles, n_experts, rows_per_expert, N, mode, limit=0.0, fmt=1):
    """a [P, K] rows in expert order; b [E*rows_per_expert, K]; mode 0 -> fp32 [P, N]; 1 -> swiglu bf16 [P, N]."""
    Pn, K = a.shape
    out = torch.empty(Pn, N, dtype=torch.bfloat16 if mode == 1 else torch.float32, device=a.device)
    rc = lib().spark_gemm_grouped_bf16(P(a), P(b), P(out), Pn, N, K, a.stride(0), K, N, n_experts, rows_per_expert,
                                       P(tiles), P(ntile), max_tiles, mode, float(limit), fmt, P(status_word(a.device)),
                                       stream())
    check(rc, "spark_gemm_grouped_bf16")
    return out


DECODE_PAIRS_MAX = 256


SIDE_STREAMS = os.environ.get("SPARK_SIDE_STREAMS", "1") == "1"
_side = {}


def _side_stream(device) -> torch.cuda.Stream:
    key = torch.device(device).index
    if key not in _side:
        _side[key] = torch.cuda.Stream(device=device)
    return _side[key]


def _shared_expert_decode(h, w, c):
    """The shared expert's two GEMVs for decode rows (when it is not a pair of the stack)."""
    sgu = w["s_gu"]
    if isinstance(sgu, Exl3Weight):
        if sgu.bits != 4 or w["s_down"].bits != 4:       # bit widths without a GEMV kernel: resident fp16 inner weights
            return exl3_linear(swiglu(exl3_linear(h, sgu), c.swiglu_limit), w["s_down"])
        return exl3_gemv(exl3_gemv(h, sgu), w["s_down"], act=1, limit=c.swiglu_limit)
    if isinstance(sgu, QuantWeight):
        return quant_linear(swiglu(quant_linear(h, sgu), c.swiglu_limit), w["s_down"])
    return gemv_bf16(gemv_bf16(h, sgu), w["s_down"], act=1, limit=c.swiglu_limit, k=w["s_down"].shape[1])


def _moe_decode(h, w, c, defer: bool):
    """Decode rows (<= 16): ONE router launch (GEMV + top-k + pair tables), gate/up GEMV and SwiGLU + down GEMV
    over the (row, expert) pairs, then the slot-order combine (deferred into the residual update when `defer`).
    The shared expert is one more pair when it lives in the expert stack (`w["shared_in_stack"]`)."""
    h = _as_bf16(h).contiguous()
    R, H = h.shape
    dev = h.device
    ep = w.get("ep")
    e_lo, e_hi = ep if ep else (0, c.n_experts)
    rank, world = w.get("tp_rank", (0, 1))
    # the shared expert as one more pair of the stack: always under tensor parallelism (row r's pair belongs to rank
    # r % world); on one GPU it runs as two GEMVs on a side stream next to the router instead (SPARK_SHARED_PAIR=1
    # forces the pair form)
    stacked = bool(w.get("shared_in_stack")) and (world > 1 or SHARED_AS_PAIR or "s_gu" not in w)
    slots = c.top_k + (1 if stacked else 0)
    gate = w["gate"]
    NE = c.n_experts + (1 if c.shared_gate else 0)
    ld = (NE + 7) // 8 * 8
    logits = scratch("router_logits", DECODE_ROWS_MAX * ld, torch.float32, dev)
    counter = scratch("router_counter", 4, torch.int32, dev, zero=True)
    wts = torch.empty(R, slots, dtype=torch.float32, device=dev)
    ids = torch.empty(R, slots, dtype=torch.int32, device=dev)
    prow = torch.empty(R, slots, dtype=torch.int32, device=dev)
    shared_sep = "s_gu" in w and not stacked
    sg = torch.empty(R, dtype=torch.float32, device=dev) if (c.shared_gate and shared_sep) else None
    rc = lib().spark_moe_router_topk(P(h), h.stride(0), P(gate), gate.stride(0), P(logits), ld,
                                     R, H, c.n_experts, c.top_k, ROUTER_KIND[c.router], P(w.get("bias")), float(c.route_scale),
                                     int(c.shared_gate), slots, e_hi - e_lo, e_lo, e_hi, rank, world, P(wts), P(ids), P(prow),
                                     P(sg), P(counter), stream())
    check(rc, "spark_moe_router_topk")
    shared = None
    side = None
    if shared_sep:
        hm = h
        main = torch.cuda.current_stream()
        side = _side_stream(dev) if SIDE_STREAMS else None
        if side is not None:
            side.wait_stream(main)
        with torch.cuda.stream(side if side is not None else main):
            shared = _shared_expert_decode(hm, w, c)
    Pn = R * slots
    pe, pr = ids.view(-1), prow.view(-1)
    gu = _expert_gemv(h, w["w_gu"], Pn, pe, pr, 0, 0.0, False)                      # [P, 2F] bf16
    y = _expert_gemv(gu, w["w_down"], Pn, pe, None, 1, c.swiglu_limit, True, pairs_early=True)   # [P, H] fp32
    if side is not None:
        torch.cuda.current_stream().wait_stream(side)
    pm = PendingMoe(y, wts, ids, slots, R, H, shared, sg)
    return pm if defer else pm.tensor()


def moe(h, w, c, defer: bool = False):
    """Routed + shared experts; returns the bf16 block output [R, H] (or, with `defer`, the uncombined expert
    outputs of a decode round).  Under expert parallelism (`w["ep"]` = (first local expert, end)) only the local
    experts' pairs are computed and the result is this rank's partial sum; the shared expert is added by the rank
    that holds it."""
    if h.shape[0] * c.top_k <= DECODE_PAIRS_MAX and h.shape[0] <= DECODE_ROWS_MAX and FUSED_DECODE:
        return _moe_decode(h, w, c, defer)
    h = _as_bf16(h).contiguous()
    R, H = h.shape
    dev = h.device
    ep = w.get("ep")
    wts, ids, prow, sg = moe_route(h, w, c, *(ep if ep else (0, None)))
    Pn = R * c.top_k
    wgu, wd = w["w_gu"], w["w_down"]
    shared = None
    side = None
    if "s_gu" in w:
        if R <= 16:
            # decode rows: the shared expert's two GEMVs do not depend on the router, so they run on a side stream
            # next to the routed experts (a fork/join that a captured graph keeps as parallel branches)
            sgu = w["s_gu"]
            main = torch.cuda.current_stream()
            side = _side_stream(dev) if SIDE_STREAMS else None
            if side is not None:
                side.wait_stream(main)
            with torch.cuda.stream(side if side is not None else main):
                if isinstance(sgu, Exl3Weight):
                    if sgu.bits != 4 or w["s_down"].bits != 4:
                        shared = exl3_linear(swiglu(exl3_linear(h, sgu), c.swiglu_limit), w["s_down"])
                    else:
                        gu_s = exl3_gemv(h, sgu)
                        shared = exl3_gemv(gu_s, w["s_down"], act=1, limit=c.swiglu_limit)
                elif isinstance(sgu, QuantWeight):
                    shared = quant_linear(swiglu(quant_linear(h, sgu), c.swiglu_limit), w["s_down"])
                else:
                    gu_s = gemv_bf16(h, sgu)
                    shared = gemv_bf16(gu_s, w["s_down"], act=1, limit=c.swiglu_limit, k=w["s_down"].shape[1])
        elif w.get("shared_in_stack") and w.get("tp_rank", (0, 1))[1] > 1:
            # every rank holds the shared expert: rank r computes it for rows r, r + world, ... (the all-reduce of
            # the block output puts the rows together)
            rk, wd_ = w["tp_rank"]
            rows = torch.arange(rk, R, wd_, device=dev)
            shared = torch.zeros(R, H, dtype=torch.bfloat16, device=dev)
            if rows.numel():
                shared[rows] = linear_any(swiglu(linear_any(h[rows].contiguous(), w["s_gu"]), c.swiglu_limit), w["s_down"])
        else:
            shared = linear_any(swiglu(linear_any(h, w["s_gu"]), c.swiglu_limit), w["s_down"])
    out = torch.empty(R, H, dtype=torch.bfloat16, device=dev)
    if Pn <= DECODE_PAIRS_MAX:
        pe, pr = ids.view(-1), prow.view(-1)
        gu = _expert_gemv(h, wgu, Pn, pe, pr, 0, 0.0, False)                       # [P, 2F] bf16
        y = _expert_gemv(gu, wd, Pn, pe, None, 1, c.swiglu_limit, True)            # [P, H] fp32
        inv = None
    else:
        perm, inv, offs, tiles, ntile, max_tiles = moe_sort(ids.view(-1), (ep[1] - ep[0]) if ep else c.n_experts)
        src = torch.div(perm, c.top_k, rounding_mode="floor").to(torch.int32)
        a = gather_rows(h, src)
        if isinstance(wgu, Exl3Weight):
            from .exl3_moe import exl3_grouped_experts
            y = exl3_grouped_experts(a, wgu, wd, ids, perm, tiles, ntile, max_tiles, c)
        elif isinstance(wgu, QuantWeight):
            from . import mx
            y = mx.grouped_experts(a, wgu, wd, ids, perm, tiles, ntile, max_tiles, c)
        else:
            E, F2, K = wgu.shape
            act = grouped_gemm(a, wgu.view(E * F2, K), tiles, ntile, max_tiles, E, F2, F2 // 2, 1, c.swiglu_limit)
            y = grouped_gemm(act, wd.view(E * H, F2 // 2), tiles, ntile, max_tiles, E, H, H, 0)
    if side is not None:
        torch.cuda.current_stream().wait_stream(side)          # join: the combine reads the shared expert's output
    rc = lib().spark_moe_combine(None, P(y), int(y.dtype == torch.float32), P(inv), P(wts), R, c.top_k, P(shared), P(sg), H,
                                 P(out), stream(), P(ids) if ep else None)
    check(rc, "spark_moe_combine")
    return out


def linear_any(x, w):
    return quant_linear(x, w) if isinstance(w, QuantWeight) else dense_linear(x, w)


# ----------------------------------------------------------------------------- mixers
def _plan_dev(plan, device):
    if not plan.dev:
        from ..models.plan import plan_device_arrays
        plan.dev = plan_device_arrays(plan, device)
    return plan.dev


def _check_cache_rows(what, d, tree, cache_rows):
    """SPARK_CHECK: every row's cache slot (sequence base + position, or + node slot for tree rows) is inside the cache."""
    slot = d["row_kv"] + ((d["row_pos0"] + d["row_j"]) if tree else d["pos32"]).long()
    dbg.check_index(what + " cache slot", slot, 0, cache_rows)


def _check_slots(what, plan, n_slots):
    bad = [s.slot for s in plan.segs if not 0 <= s.slot < n_slots]
    if bad:
        raise dbg.IndexTableError(f"{what}: sequence slots {bad} outside [0, {n_slots})")


GDN_CHUNKED = os.environ.get("SPARK_GDN_CHUNKED", "1") == "1"
GDN_CHUNK_MIN_ROWS = 64
_KERNELS_PER_CALL["spark_gdn_chunk_prefill"] = 3


def _gdn_chunk_prefill(mixer, proj, ab, plan, d, out):
    """Committed segments of >= 64 rows: chunked (WY-form) gated delta rule on tensor cores, three launches."""
    c, w, dev = mixer.c, mixer.w, proj.device
    if "gdn_chunks" not in d:
        chunks, first = [], []
        for i, sg in enumerate(plan.segs):
            first.append(len(chunks))
            chunks += [(i, k) for k in range((sg.n + 63) // 64)]
        d["gdn_chunks"] = torch.tensor(chunks, dtype=torch.int32).to(dev)
        d["gdn_chunk0"] = torch.tensor(first, dtype=torch.int32).to(dev)
    chunks, first = d["gdn_chunks"], d["gdn_chunk0"]
    nch = chunks.shape[0]
    dll = lib()
    fn = dll._dll.spark_gdn_chunk_ws_floats
    fn.restype, fn.argtypes = C.c_longlong, [i32, i32]
    ws = scratch("gdn_chunk_ws", fn(nch, c.n_v_heads), torch.float32, dev)
    o_raw = scratch("gdn_chunk_o", proj.shape[0] * c.n_v_heads * c.head_dim, torch.float32, dev)
    rc = dll.spark_gdn_chunk_prefill(P(proj), proj.stride(0), P(ab), ab.stride(0), P(w["conv"]), P(w["A_log"]),
                                     P(w["dt_bias"]), P(w["norm"]), P(mixer.S), P(mixer.tail), P(d["seg"]), len(plan.segs),
                                     P(chunks), nch, P(first), P(ws), P(o_raw), P(out), out.stride(0), c.n_k_heads,
                                     c.n_v_heads, c.head_dim, float(mixer.cfg.norm_eps), stream())
    check(rc, "spark_gdn_chunk_prefill")
    return out


def _tree_walks(plan, dev, accepted=None):
    """Virtual segments for linear-attention kernels on a verification tree: one root-to-node walk per node (verify) or
    the accepted walk per sequence (commit).  Returns (seg [n,4], walk lengths [n], rows [n, ld], n, ld)."""
    key = "tree_walks" if accepted is None else None
    d = plan.dev
    if key and key in d:
        return d[key]
    segs, lens, rows = [], [], []
    for i, sg in enumerate(plan.segs):
        par = sg.parents if sg.parents is not None else [j - 1 for j in range(sg.n)]
        if accepted is not None:
            walks = [list(accepted[i])] if accepted[i] else []
        else:
            walks = []
            for j in range(sg.n):
                w, k = [], j
                while k >= 0:
                    w.append(k)
                    k = par[k]
                walks.append(w[::-1])
        for w in walks:
            segs.append([sg.slot, sg.r0, 0, sg.pos0])
            lens.append(len(w))
            rows.append([sg.r0 + k for k in w])
    ld = max([len(r) for r in rows] + [1])
    for s_, l in zip(segs, lens):
        s_[2] = ld
    tab = torch.tensor([r + [0] * (ld - len(r)) for r in rows] or [[0]], dtype=torch.int32).to(dev)
    out = (torch.tensor(segs or [[0, 0, 0, 0]], dtype=torch.int32).to(dev), torch.tensor(lens or [0], dtype=torch.int32).to(dev),
           tab, len(segs), ld)
    if key:
        d[key] = out
    return out


def gdn_mixer(mixer, proj, ab, plan, commit, n_rows=None, accepted=None):
    c = mixer.c
    d = _plan_dev(plan, proj.device)
    R = proj.shape[0]
    out = torch.empty(R, c.n_v_heads * c.head_dim, dtype=torch.bfloat16, device=proj.device)
    w = mixer.w
    if dbg.CHECK:
        _check_slots("gdn_mixer", plan, mixer.S.shape[0])
    if plan.is_tree:
        # every node forks its parent's state: one walk from the committed state per node (verify), or the accepted
        # walk per sequence (commit); a tree round never commits directly
        assert not commit or accepted is not None
        seg, lens, tab, nw, ld = _tree_walks(plan, proj.device, accepted)
        dbg.check_index("gdn_mixer walk table", tab, 0, R, allow=-1)
        rc = lib().spark_gdn_seq(P(proj), proj.stride(0), P(ab), ab.stride(0), P(w["conv"]), P(w["A_log"]), P(w["dt_bias"]),
                                 P(w["norm"]), P(mixer.S), P(mixer.tail), P(seg), P(lens), nw, P(out), out.stride(0),
                                 c.n_k_heads, c.n_v_heads, c.head_dim, float(mixer.cfg.norm_eps), int(commit), stream(),
                                 P(tab), ld, int(ld > 1))
        check(rc, "spark_gdn_seq")
        return out
    if (commit and n_rows is None and c.head_dim == 128 and GDN_CHUNKED
            and min(s.n for s in plan.segs) >= GDN_CHUNK_MIN_ROWS):
        return _gdn_chunk_prefill(mixer, proj, ab, plan, d, out)
    rc = lib().spark_gdn_seq(P(proj), proj.stride(0), P(ab), ab.stride(0), P(w["conv"]), P(w["A_log"]), P(w["dt_bias"]),
                             P(w["norm"]), P(mixer.S), P(mixer.tail), P(d["seg"]), P(n_rows), len(plan.segs), P(out),
                             out.stride(0), c.n_k_heads, c.n_v_heads, c.head_dim, float(mixer.cfg.norm_eps), int(commit),
                             stream(), None, 0, int(max(sg.n for sg in plan.segs) > 1))
    check(rc, "spark_gdn_seq")
    return out


def gdn_commit(mixer, proj, ab, plan, accepted) -> bool:
    if plan.is_tree:
        gdn_mixer(mixer, proj, ab, plan, True, accepted=accepted)
        return True
    n_rows = torch.tensor([len(a) for a in accepted], dtype=torch.int32, device=proj.device)
    gdn_mixer(mixer, proj, ab, plan, True, n_rows)
    return True


KDA_CHUNKED = os.environ.get("SPARK_KDA_CHUNKED", "1") == "1"
_KERNELS_PER_CALL["spark_kda_chunk_prefill"] = 3


def kda_mixer(mixer, pre, lr, plan, commit, n_rows=None, accepted=None):
    """KDA layer core on the device: the low-rank gate expansions run on the GEMV/GEMM kernels, conv + norms +
    per-channel-decay delta rule + gated RMS output in one launch (sequential over the rows of a segment; on a
    verification tree one root-to-node walk per node, see `_tree_walks`)."""
    c, w = mixer.c, mixer.w
    dev = pre.device
    d = _plan_dev(plan, dev)
    r, n = c.gate_rank, c.n_heads * c.head_dim
    if not hasattr(mixer, "_gate_w"):
        mixer._gate_w = (w["f_b"].to(torch.bfloat16).contiguous(), w["g_b"].to(torch.bfloat16).contiguous())
    pre = _as_bf16(pre)
    lr = _as_bf16(lr)
    if pre.shape[0] <= 16 and lr.stride(0) % 8 == 0 and r % 8 == 0 and lr.data_ptr() % 16 == 0:
        # decode rows: the GEMV reads the two low-rank halves in place (row stride of `lr`; 16-byte aligned rows)
        g1 = gemv_bf16(lr[:, :r], mixer._gate_w[0], out_f32=True, ldx=lr.stride(0))
        g2 = gemv_bf16(lr[:, r: 2 * r], mixer._gate_w[1], out_f32=True, ldx=lr.stride(0))
    else:
        g1 = dense_linear(lr[:, :r].contiguous(), mixer._gate_w[0], out_f32=True)
        g2 = dense_linear(lr[:, r: 2 * r].contiguous(), mixer._gate_w[1], out_f32=True)
    R = pre.shape[0]
    out = torch.empty(R, n, dtype=torch.bfloat16, device=dev)
    if dbg.CHECK:
        _check_slots("kda_mixer", plan, mixer.S.shape[0])
    if plan.is_tree:
        assert not commit or accepted is not None
        seg, lens, tab, nw, ld = _tree_walks(plan, dev, accepted)
        dbg.check_index("kda_mixer walk table", tab, 0, R, allow=-1)
        rc = lib().spark_kda_seq(P(pre), pre.stride(0), P(g1), P(g2), n, P(lr), lr.stride(0), 2 * r, P(w["conv"]), P(w["A_log"]),
                                 P(w["dt_bias"]), P(w["o_norm"]), P(mixer.S), P(mixer.tail), P(seg), P(lens), nw, P(out), n,
                                 c.n_heads, c.head_dim, int(commit), stream(), P(tab), ld, int(ld > 1))
        check(rc, "spark_kda_seq")
        return out
    if (commit and n_rows is None and c.head_dim == 128 and KDA_CHUNKED
            and min(s.n for s in plan.segs) >= GDN_CHUNK_MIN_ROWS):
        # committed segments of >= 64 rows: chunked form on tensor cores (16-row chunks, per-channel decay)
        if "kda_chunks" not in d:
            chunks, first = [], []
            for i, sg in enumerate(plan.segs):
                first.append(len(chunks))
                chunks += [(i, k) for k in range((sg.n + 15) // 16)]
            d["kda_chunks"] = torch.tensor(chunks, dtype=torch.int32).to(dev)
            d["kda_chunk0"] = torch.tensor(first, dtype=torch.int32).to(dev)
        chunks, first = d["kda_chunks"], d["kda_chunk0"]
        nch = chunks.shape[0]
        dll = lib()
        fn = dll._dll.spark_kda_chunk_ws_floats
        fn.restype, fn.argtypes = C.c_longlong, [i32, i32]
        ws = scratch("kda_chunk_ws", fn(nch, c.n_heads), torch.float32, dev)
        o_raw = scratch("kda_chunk_o", R * n, torch.float32, dev)
        rc = dll.spark_kda_chunk_prefill(P(pre), pre.stride(0), P(g1), P(g2), n, P(lr), lr.stride(0), 2 * r, P(w["conv"]),
                                         P(w["A_log"]), P(w["dt_bias"]), P(w["o_norm"]), P(mixer.S), P(mixer.tail), P(d["seg"]),
                                         len(plan.segs), P(chunks), nch, P(first), P(ws), P(o_raw), P(out), n, c.n_heads,
                                         c.head_dim, stream())
        check(rc, "spark_kda_chunk_prefill")
        return out
    rc = lib().spark_kda_seq(P(pre), pre.stride(0), P(g1), P(g2), n, P(lr), lr.stride(0), 2 * r, P(w["conv"]), P(w["A_log"]),
                             P(w["dt_bias"]), P(w["o_norm"]), P(mixer.S), P(mixer.tail), P(d["seg"]), P(n_rows),
                             len(plan.segs), P(out), n, c.n_heads, c.head_dim, int(commit), stream(), None, 0,
                             int(max(sg.n for sg in plan.segs) > 1))
    check(rc, "spark_kda_seq")
    return out


def kda_commit(mixer, pre, lr, plan, accepted) -> bool:
    if plan.is_tree:
        kda_mixer(mixer, pre, lr, plan, True, accepted=accepted)
        return True
    n_rows = torch.tensor([len(a) for a in accepted], dtype=torch.int32, device=pre.device)
    kda_mixer(mixer, pre, lr, plan, True, n_rows)
    return True


MLA_TS = 64
MLA_KERNELS = os.environ.get("SPARK_MLA_KERNELS", "1") == "1"
_KERNELS_PER_CALL["spark_mla_attn"] = 2


def mla_fp8_shape_ok(kv_lora: int, rope: int) -> bool:
    """Latent shapes the packed FP8 rows of the kernels cover (<= 4 scale tiles, 16 codes per lane of one warp)."""
    nt = kv_lora // 128 if kv_lora >= 128 else 1
    return kv_lora <= 512 and kv_lora % 16 == 0 and kv_lora % nt == 0 and (kv_lora // nt) % 16 == 0 \
        and rope % 8 == 0 and rope <= 256


def mla_mixer(mixer, h, plan, seqs):
    """Latent attention on the device: returns the per-head outputs [R, H*D] (before the output projection), or None.
    Rows of a verification tree read the committed context densely plus their ancestors' in-flight slots (bit-masks
    in the decode kernel); a tree on a context long enough to need the pool selection runs the generic path."""
    if not MLA_KERNELS:
        return None
    c, w, cfg = mixer.c, mixer.w, mixer.cfg
    if mixer.fp8 and not mla_fp8_shape_ok(c.kv_lora, c.rope_dim):
        return None
    dev = h.device
    d = _plan_dev(plan, dev)
    R = h.shape[0]
    if "row_kv" not in d:
        d["row_kv"] = torch.tensor([seqs[s.slot].kv_base for s in plan.segs for _ in range(s.n)], dtype=torch.int64).to(dev)
        d["max_ctx"] = max(s.pos0 + s.n for s in plan.segs)
        for s in plan.segs:
            assert s.pos0 + s.n <= seqs[s.slot].kv_cap, "sequence capacity exceeded"
    tree = plan.is_tree
    if tree:
        if d["max_ctx"] // c.pool > c.topk_pools:
            return None
        if "anc" not in d:
            d["anc"] = tree_ancestor_masks(plan, dev)
    H, D, L, Rr = c.n_heads, c.head_dim, c.kv_lora, c.rope_dim
    KW = L + Rr
    if not hasattr(mixer, "_dev"):
        half = max(Rr // 2, 1)
        inv = (c.rope_theta ** (-torch.arange(half, dtype=torch.float64) * 2 / max(Rr, 1))).to(dev)
        mixer._dev = {"inv": inv, "w_ukT": mixer.w_uk.transpose(1, 2).contiguous().to(torch.bfloat16),
                      "w_uv": mixer.w_uv.contiguous().to(torch.bfloat16),
                      "ape": w["ape"].float().contiguous()}
    md = mixer._dev
    if dbg.CHECK:
        _check_cache_rows("mla_mixer", d, tree, mixer.lat.shape[0])
    a = _as_bf16(linear_any(h, w["a"])).contiguous()
    cq = torch.empty(R, c.q_lora, dtype=torch.bfloat16, device=dev)
    hw = torch.empty(R, c.idx_heads, dtype=torch.float32, device=dev)
    rc = lib().spark_mla_prep(P(a), a.stride(0), R, c.q_lora, L, Rr, c.idx_dim, c.idx_heads, c.pool, float(cfg.norm_eps),
                              P(w["q_a_norm"]), P(w["kv_a_norm"]), P(w["k_ln_w"]), P(w["k_ln_b"]), P(md["ape"]), P(md["inv"]),
                              P(d["pos32"]), P(d["row_kv"]), P(d["row_j"]), P(cq), P(mixer.lat), P(mixer.ik), P(mixer.ig),
                              P(mixer.pool), P(hw), stream(), P(d["row_pos0"]) if tree else None,
                              int(mixer.fp8))
    check(rc, "spark_mla_prep")
    qb = _as_bf16(linear_any(cq, w["q_b"]))
    nq = H * (D + Rr)
    q_full = torch.empty(R, H, KW, dtype=torch.bfloat16, device=dev)
    decode = R * H <= 4096 and R <= 16
    if decode:
        key = ("mla_heads", H)
        if key not in md:
            md[key] = torch.arange(H, dtype=torch.int32, device=dev)
        heads = md[key]
        qn = qb[:, :nq].contiguous()
        # absorb W_uk: one item per head over all rows (the head's [L, D] matrix is streamed once for the round)
        gemv_bf16_items(qn, H * (D + Rr), D + Rr, md["w_ukT"], L * D, D, q_full, H * KW, KW, H, R, L, D, heads)
    else:
        q_full[..., :L] = torch.einsum("thd,hld->thl", qb[:, :nq].view(R, H, D + Rr)[..., :D], md["w_ukT"])
    if Rr:
        rc = lib().spark_mla_qrope(P(qb), qb.stride(0), R, H, D, Rr, L, P(md["inv"]), P(d["pos32"]), P(q_full), stream())
        check(rc, "spark_mla_qrope")
    sel = sel_n = None
    sel_ld = 0
    max_ctx = d["max_ctx"]
    if max_ctx // c.pool > c.topk_pools:
        from . import sparse as sp
        qi = qb[:, nq:].float().view(R, c.idx_heads, c.idx_dim).contiguous()
        sel, sel_n = sp.select_tokens(qi, mixer.pool, d["row_kv"], d["pos32"], c.pool, c.topk_pools, max_ctx, head_w=hw,
                                      scale=c.idx_dim ** -0.5, window=c.window,
                                      segs=None if tree else (d["seg"], len(plan.segs), max(s.n for s in plan.segs)))
        sel_ld = sel.shape[1]
        max_ctx = sel_ld
    nsplit = (max_ctx + MLA_TS - 1) // MLA_TS
    part_o = scratch("mla_part_o", R * H * nsplit * L, torch.float32, dev)
    part_ml = scratch("mla_part_ml", R * H * nsplit * 2, torch.float32, dev)
    out_lat = torch.empty(R, H, L, dtype=torch.bfloat16, device=dev)
    rc = lib().spark_mla_attn(P(q_full), P(mixer.lat), P(d["pos32"]), P(d["row_kv"]), P(sel), P(sel_n), sel_ld, P(part_o),
                              P(part_ml), nsplit, P(w.get("sink")) if c.sink else None, R, H, L, Rr,
                              1.0 / math.sqrt(D + Rr), P(out_lat), stream(), P(d["row_pos0"]) if tree else None,
                              P(d["row_j"]) if tree else None, P(d["anc"]) if tree else None, int(mixer.fp8))
    check(rc, "spark_mla_attn")
    if decode:
        out = torch.empty(R, H * D, dtype=torch.bfloat16, device=dev)
        return gemv_bf16_items(out_lat, H * L, L, md["w_uv"], D * L, L, out, H * D, D, H, R, D, L, md[("mla_heads", H)])
    return torch.einsum("thl,hdl->thd", out_lat, md["w_uv"]).reshape(R, H * D)


ATT_TS = 64


ATTN_PREFILL_KERNEL = os.environ.get("SPARK_ATTN_PREFILL", "1") == "1"
ATTN_PREFILL_MIN_ROWS = 32
# block-sparse prefill rows take the masked dense tiles while a segment's average causal context is at most this
# (measured: 16K-token prompts 21.4k tok/s at 6144, 21.6k at 12288 and above; 64K-token prompts 17.6k at 6144, 17.2k at
# 32768, 13.0k with every chunk on the masked tiles)
ATTN_MASKED_MAX_KEYS = int(os.environ.get("SPARK_ATTN_MASKED_MAX_KEYS", "12288"))


def tree_ancestor_masks(plan, device) -> torch.Tensor:
    """Per row, the bitmask of segment-local rows it may attend to (itself and its ancestors; chains: all earlier
    rows of the segment)."""
    import numpy as np
    m = np.zeros(plan.rows, dtype=np.uint32)
    for sg in plan.segs:
        assert sg.n <= 32, "a verification tree holds at most 32 nodes per sequence"
        for j in range(sg.n):
            if sg.parents is None:
                m[sg.r0 + j] = (1 << (j + 1)) - 1
            else:
                par = sg.parents[j]
                m[sg.r0 + j] = (1 << j) | (int(m[sg.r0 + par]) if par >= 0 else 0)
    return torch.from_numpy(m.view(np.int32)).to(device)


def attn_mixer(mixer, qkv, plan, seqs):
    c = mixer.c
    dev = qkv.device
    d = _plan_dev(plan, dev)
    R = qkv.shape[0]
    if "row_kv" not in d:
        kvb = torch.tensor([seqs[s.slot].kv_base for s in plan.segs for _ in range(s.n)], dtype=torch.int64)
        d["row_kv"] = kvb.to(dev)
        d["max_ctx"] = max(s.pos0 + s.n for s in plan.segs)
        for s in plan.segs:
            assert s.pos0 + s.n <= seqs[s.slot].kv_cap, "sequence capacity exceeded"
    sparse = c.sparse_topk_blocks > 0
    tree = plan.is_tree
    if tree:
        # ancestor-masked rows run on the tensor-core decode kernel; a tree that also needs the block-sparse selection
        # (context beyond the selection budget) or an unsupported head shape takes the generic path
        if (c.head_dim not in (64, 128, 256) or c.n_q_heads // c.n_kv_heads > 16
                or (sparse and d["max_ctx"] > c.sparse_topk_blocks * c.block)):
            return None
        if "anc" not in d:
            d["anc"] = tree_ancestor_masks(plan, dev)
    w = mixer.w
    if dbg.CHECK:
        _check_cache_rows("attn_mixer", d, tree, mixer.k.shape[0])
    qbuf = torch.empty(R, c.n_q_heads, c.head_dim, dtype=torch.bfloat16, device=dev)
    qi = torch.empty(R, c.idx_heads, c.idx_dim, dtype=torch.float32, device=dev) if sparse else None
    rc = lib().spark_attn_prep(P(qkv), qkv.stride(0), R, c.n_q_heads, c.n_kv_heads, c.head_dim, c.rope_dim, int(c.gated),
                               int(c.qk_norm), c.idx_heads if sparse else 0, c.idx_dim if sparse else 0, c.block,
                               int(mixer.fp8), float(mixer.cfg.norm_eps), P(w.get("q_norm")), P(w.get("k_norm")),
                               P(w.get("iq_norm")), P(w.get("ik_norm")), P(mixer.inv), P(d["pos32"]), P(d["row_kv"]),
                               P(d["row_j"]), P(qbuf), P(mixer.k), P(mixer.v), P(getattr(mixer, "ks", None)),
                               P(getattr(mixer, "vs", None)), P(qi), P(getattr(mixer, "ik_raw", None)),
                               P(getattr(mixer, "ik_pool", None)), stream(), P(d["row_pos0"]) if tree else None)
    check(rc, "spark_attn_prep")
    sel = sel_n = None
    sel_ld = 0
    max_ctx = d["max_ctx"]
    if sparse and max_ctx > c.sparse_topk_blocks * c.block:
        from . import sparse as sp
        sel, sel_n = sp.select_blocks(mixer, qi, plan, d)
        sel_ld = sel.shape[1]
        max_ctx = sel_ld
    if (sel is None and not tree and not mixer.fp8 and ATTN_PREFILL_KERNEL and c.head_dim in (64, 128, 256)
            and min(s.n for s in plan.segs) >= ATTN_PREFILL_MIN_ROWS):
        # whole segments, dense context: flash-style tensor-core kernel (one CTA per 64 rows of a head)
        out = torch.empty(R, c.n_q_heads * c.head_dim, dtype=torch.bfloat16, device=dev)
        rc = lib().spark_attn_prefill(P(qbuf), P(mixer.k), P(mixer.v), P(d["row_kv"]), P(d["seg"]), len(plan.segs),
                                      max(s.n for s in plan.segs), P(qkv), qkv.stride(0), int(c.gated), P(out),
                                      c.n_q_heads, c.n_kv_heads, c.head_dim, 1.0 / math.sqrt(c.head_dim), stream())
        check(rc, "spark_attn_prefill")
        return out
    if (sel is not None and not tree and not mixer.fp8 and ATTN_PREFILL_KERNEL and c.block == 4
            and c.head_dim in (64, 128, 256) and min(s.n for s in plan.segs) >= ATTN_PREFILL_MIN_ROWS
            and max(s.pos0 + s.n // 2 for s in plan.segs) <= ATTN_MASKED_MAX_KEYS):
        # block-sparse rows on a context of a few thousand tokens: the dense tiles with the unselected blocks masked
        # (64 rows share every key tile) beat one gathering CTA per row, which is bound by L2 bandwidth
        mw = (d["max_ctx"] + 127) // 128
        bmask = scratch("attn_block_mask", R * mw, torch.int32, dev)
        out = torch.empty(R, c.n_q_heads * c.head_dim, dtype=torch.bfloat16, device=dev)
        add_launches(1)
        rc = lib().spark_attn_prefill_masked(P(qbuf), P(mixer.k), P(mixer.v), P(d["row_kv"]), P(d["seg"]), len(plan.segs),
                                             max(s.n for s in plan.segs), P(qkv), qkv.stride(0), int(c.gated), P(out),
                                             c.n_q_heads, c.n_kv_heads, c.head_dim, 1.0 / math.sqrt(c.head_dim), P(sel),
                                             P(sel_n), sel_ld, R, P(bmask), mw, stream())
        check(rc, "spark_attn_prefill_masked")
        return out
    nsplit, chunks = (max_ctx + ATT_TS - 1) // ATT_TS, 1
    if R >= 64 and c.head_dim in (64, 128, 256) and c.n_q_heads // c.n_kv_heads <= 16:
        # prefill-size batches have rows enough to fill the GPU: one CTA walks a row's whole context with a running
        # softmax, so no per-split partials are written and merged (2.2 GB of them for a 4096-row chunk at 2K tokens each)
        nsplit, chunks = 1, nsplit
    part_o = scratch("attn_part_o", R * c.n_q_heads * nsplit * c.head_dim, torch.float32, dev)
    part_ml = scratch("attn_part_ml", R * c.n_q_heads * nsplit * 2, torch.float32, dev)
    out = torch.empty(R, c.n_q_heads * c.head_dim, dtype=torch.bfloat16, device=dev)
    rc = lib().spark_attn_decode(P(qbuf), P(mixer.k), P(mixer.v), P(getattr(mixer, "ks", None)),
                                 P(getattr(mixer, "vs", None)), int(mixer.fp8), P(d["pos32"]), P(d["row_kv"]), P(sel),
                                 P(sel_n), sel_ld, P(part_o), P(part_ml), nsplit, P(qkv), qkv.stride(0), int(c.gated), R,
                                 c.n_q_heads, c.n_kv_heads, c.head_dim, 1.0 / math.sqrt(c.head_dim), P(out), stream(),
                                 P(d["row_pos0"]) if tree else None, P(d["row_j"]) if tree else None,
                                 P(d["anc"]) if tree else None, chunks)
    check(rc, "spark_attn_decode")
    return out
