"""Model-independent multimodal prompt plumbing.

Front end: every image (video: frames stacked) is resized / padded onto the model's canvas (uint8, HWC) and written
to a file under /dev/shm; each placeholder run of the prompt is expanded into *salted* ids in [MM_BASE, MM_TOP):
never a vocabulary id and distinct per media content, so exact-prefix reuse (plain id comparison) tells different media
apart while the same media hits the cache again.
Engine: the segments a prefill chunk touches are encoded straight from the canvas file (rank 0) and the chunk's rows are
written into the embedding rows of those positions before the vocabulary-parallel embed sum (a salted id is outside
every rank's vocabulary slice, so the other ranks contribute zeros there).
Reference: engine-rs/src/mm_canvas.rs:1-132, serve/mm.py (salted ids, canvases), weights.rs:536-569 (row injection).
"""
from __future__ import annotations

import hashlib
import os
from dataclasses import dataclass, field
from typing import Callable, List, Sequence, Tuple

import numpy as np
import torch

MM_BASE = 1 << 20
MM_TOP = 1 << 24


def is_salted(t: int) -> bool:
    return MM_BASE <= t < MM_TOP


def salted_ids(content: bytes, n: int, frame: int = 0) -> List[int]:
    """n placeholder ids for one segment: a content hash spread over [MM_BASE, MM_TOP), position-dependent so that a
    truncated or shifted run never aliases another one."""
    h = hashlib.sha256(content + frame.to_bytes(4, "little")).digest()
    seed = int.from_bytes(h[:8], "little")
    span = MM_TOP - MM_BASE
    return [MM_BASE + (seed + 0x9E3779B97F4A7C15 * (i + 1)) % span for i in range(n)]


def fit_to_canvas(img: np.ndarray, height: int, width: int) -> np.ndarray:
    """uint8 HWC image -> canvas of (height, width): nearest-neighbour resize keeping the aspect ratio, zero padding."""
    assert img.dtype == np.uint8 and img.ndim == 3 and img.shape[2] == 3
    h, w = img.shape[:2]
    sc = min(height / h, width / w)
    nh, nw = max(1, int(round(h * sc))), max(1, int(round(w * sc)))
    yi = np.minimum((np.arange(nh) / sc).astype(np.int64), h - 1)
    xi = np.minimum((np.arange(nw) / sc).astype(np.int64), w - 1)
    out = np.zeros((height, width, 3), np.uint8)
    out[:nh, :nw] = img[yi][:, xi]
    return out


def write_canvas(frames: Sequence[np.ndarray], height: int, width: int, directory: str = "/dev/shm", tag: str = "") -> dict:
    """Stack the fitted frames into one file; returns the request's mm item (without segments)."""
    data = np.stack([fit_to_canvas(f, height, width) for f in frames])
    digest = hashlib.sha256(data.tobytes()).hexdigest()[:24]
    path = os.path.join(directory, f"spark-mm-{tag}{digest}.u8")
    if not os.path.exists(path):
        tmp = path + f".{os.getpid()}.tmp"
        data.tofile(tmp)
        os.replace(tmp, path)
    return {"path": path, "frames": len(frames), "height": height, "width": width, "segments": []}


def expand_placeholders(ids: List[int], placeholder: int, items: List[dict], seg_len: Callable[[dict], int]) -> List[int]:
    """Replace the k-th occurrence of `placeholder` by the salted run of the k-th (item, frame) and record the
    segments [position, length, frame] in the items."""
    flat = [(it, f) for it in items for f in range(it["frames"])]
    out: List[int] = []
    k = 0
    for t in ids:
        if t != placeholder:
            out.append(t)
            continue
        if k >= len(flat):
            raise ValueError("more placeholders than media segments")
        it, f = flat[k]
        n = seg_len(it)
        with open(it["path"], "rb") as fh:
            fh.seek(f * it["height"] * it["width"] * 3)
            content = fh.read(it["height"] * it["width"] * 3)
        it["segments"].append([len(out), n, f])
        out += salted_ids(content, n, f)
        k += 1
    if k != len(flat):
        raise ValueError("fewer placeholders than media segments")
    return out


@dataclass
class MmItem:
    path: str
    frames: int
    height: int
    width: int
    segments: List[Tuple[int, int, int]] = field(default_factory=list)    # (prompt position, count, frame)


def parse_items(v, seg_len: Callable[[MmItem], int]) -> List[MmItem]:
    """Validate the request's "mm" array against the canvas files and the model's geometry."""
    out = []
    for it in v or []:
        item = MmItem(it["path"], int(it["frames"]), int(it["height"]), int(it["width"]))
        if item.frames < 1 or item.height < 1 or item.width < 1:
            raise ValueError(f"mm item has a bad canvas {item.frames}x{item.height}x{item.width}")
        n = seg_len(item)
        size = os.path.getsize(item.path)
        want = item.frames * item.height * item.width * 3
        if size != want:
            raise ValueError(f"mm canvas {item.path} has {size} bytes, expected {want}")
        for pos, cnt, frame in it["segments"]:
            if pos < 0 or cnt != n or not 0 <= frame < item.frames:
                raise ValueError(f"mm segment ({pos},{cnt},{frame}) does not fit the canvas")
            item.segments.append((int(pos), int(cnt), int(frame)))
        out.append(item)
    return out


def validate(ids: Sequence[int], vocab: int, items: List[MmItem]):
    """Every id is a vocabulary id or a salted placeholder, and the placeholder positions are exactly the segments."""
    mark = [False] * len(ids)
    for it in items:
        for pos, n, _ in it.segments:
            if pos + n > len(ids):
                raise ValueError("mm segment past the end of the prompt")
            for p in range(pos, pos + n):
                if mark[p] or not is_salted(ids[p]):
                    raise ValueError(f"mm segment at {pos} does not cover salted placeholders only")
                mark[p] = True
    for p, t in enumerate(ids):
        if is_salted(t) != mark[p]:
            raise ValueError(f"position {p}: placeholder without media (or media without placeholder)")
        if not mark[p] and not 0 <= t < vocab:
            raise ValueError(f"position {p}: id {t} is outside the vocabulary")


def load_frame(item: MmItem, frame: int) -> torch.Tensor:
    """One canvas frame as uint8 [H, W, 3] (memory-mapped read of the slice)."""
    n = item.height * item.width * 3
    a = np.fromfile(item.path, dtype=np.uint8, count=n, offset=frame * n)
    return torch.from_numpy(a).view(item.height, item.width, 3)


def chunk_rows(items: List[MmItem], chunk_start: int, chunk_len: int, encode: Callable[[MmItem, int], torch.Tensor]):
    """Rows of the media segments that intersect prompt positions [chunk_start, chunk_start + chunk_len):
    list of (row index inside the chunk, tensor [n, hidden]).  A segment that straddles two chunks is encoded for both
    (the encoder is deterministic) and each chunk takes its part."""
    out = []
    for it in items:
        for pos, n, frame in it.segments:
            lo, hi = max(pos, chunk_start), min(pos + n, chunk_start + chunk_len)
            if lo >= hi:
                continue
            rows = encode(it, frame)
            assert rows.shape[0] == n, "encoder returned a different number of rows than the segment holds"
            out.append((lo - chunk_start, rows[lo - pos: hi - pos]))
    return out


def inject_rows(embed_rows: torch.Tensor, ids: torch.Tensor, injected) -> torch.Tensor:
    """Write the encoded rows over the (zero) embedding rows of the salted positions of a chunk."""
    for r0, rows in injected:
        assert bool(((ids[r0: r0 + rows.shape[0]] >= MM_BASE) & (ids[r0: r0 + rows.shape[0]] < MM_TOP)).all())
        embed_rows[r0: r0 + rows.shape[0]] = rows.to(embed_rows.dtype).to(embed_rows.device)
    return embed_rows
