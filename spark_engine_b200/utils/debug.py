"""Debug modes that make index and initialisation bugs show up as Python errors instead of device faults.

`SPARK_CHECK=1`   every index table a kernel gathers through (expert of a pair, row of a pair, token ids, cache slots,
                  root-to-node walks, n-gram rows) is reduced to (min, max) on its device and compared with the extent
                  it indexes BEFORE the launch: a bad table raises `IndexTableError`, nothing is launched, no GPU
                  faults.  One small reduction + a host read per table, so it is a debug mode; captured graphs are
                  validated by the eager warm-up that precedes every capture (checks are skipped while capturing).
`SPARK_POISON=1`  scratch buffers are refilled with NaN (floats) or 0x7f bytes (integers) every time a wrapper asks for
                  them, so a kernel that reads scratch it did not write in the same call produces NaN / wild values
                  that the numerics tests catch (the role of an initcheck run; no sanitizer needed).

The reference has no sanitizer or checked build (engine-rs/build.rs:80-93); it relies on run-twice equality and
graph == eager checks (spec_probe.rs:316-366), which the tests here keep as well.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

CHECK = os.environ.get("SPARK_CHECK", "0") == "1"
POISON = os.environ.get("SPARK_POISON", "0") == "1"

stats = {"checked": 0, "poisoned": 0}


class IndexTableError(RuntimeError):
    pass


def _capturing(t: torch.Tensor) -> bool:
    return t.is_cuda and torch.cuda.is_current_stream_capturing()


def check_index(what: str, table: Optional[torch.Tensor], lo: int, hi: int, allow: Optional[int] = None,
                count: Optional[int] = None) -> None:
    """Raise unless every entry of `table` (the first `count` when given) lies in [lo, hi) or equals `allow`."""
    if not CHECK or table is None or table.numel() == 0 or _capturing(table):
        return
    v = table.detach().reshape(-1)
    if count is not None:
        v = v[:count]
    if allow is not None:
        v = v[v != allow]
    if v.numel() == 0:
        return
    stats["checked"] += 1
    mn, mx = int(v.min()), int(v.max())
    if mn < lo or mx >= hi:
        raise IndexTableError(f"{what}: entries span [{mn}, {mx}], valid range is [{lo}, {hi})"
                              + (f" or {allow}" if allow is not None else ""))


def poison(t: torch.Tensor) -> torch.Tensor:
    """Fill a scratch tensor with a pattern no kernel should consume (NaN / 0x7f7f...)."""
    if not POISON or t.numel() == 0 or _capturing(t):
        return t
    stats["poisoned"] += 1
    if t.dtype.is_floating_point and t.element_size() > 1:
        t.fill_(float("nan"))
    else:
        t.view(torch.uint8).fill_(0x7F)
    return t
