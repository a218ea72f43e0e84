"""Global numerics of the library GEMMs that remain on the path (ATen / cuBLAS batched products of latent attention,
the vision towers, the oracles): fp32 accumulation without reduced-precision split-K reductions, TF32 only by flag.
Reference: engine-rs/src/tp.rs:231-237 and shim/shim.cpp:426-438 (`set_fp32_accum`)."""
from __future__ import annotations

import os

import torch

_done = False


def set_fp32_accum(tf32: bool | None = None) -> dict:
    """Idempotent.  `tf32` None reads SPARK_TF32 (default off).  Returns the flags in force."""
    global _done
    if tf32 is None:
        tf32 = os.environ.get("SPARK_TF32", "0") == "1"
    mm = torch.backends.cuda.matmul
    mm.allow_bf16_reduced_precision_reduction = False
    mm.allow_fp16_reduced_precision_reduction = False
    mm.allow_tf32 = bool(tf32)
    torch.backends.cudnn.allow_tf32 = bool(tf32)
    _done = True
    return {"bf16_reduced_precision_reduction": False, "fp16_reduced_precision_reduction": False, "tf32": bool(tf32)}


def ensure() -> None:
    if not _done:
        set_fp32_accum()
