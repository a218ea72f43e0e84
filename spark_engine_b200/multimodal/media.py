"""Media pre-processing for the front end: fetch, decode, resize, frames, and the chat-content walk.

A chat message's content may be a list of parts; `image_url` parts (data URLs, local files, and http(s) URLs when
fetching is allowed) and `video_url` parts (animated images: frames sampled evenly) are decoded with PIL to uint8 RGB,
resized with antialiasing onto the model's canvas (aspect ratio kept, zero padding) and written to canvas files; the
text keeps one placeholder per frame, which `canvas.expand_placeholders` turns into salted ids.  Nothing here touches
a GPU: the engine encodes the canvases while it prefills the chunks that contain them.
Reference: serve/mm.py (fetch / decode / canvases in the front end), engine-rs/src/mm_canvas.rs:1-132.
"""
from __future__ import annotations

import base64
import io
import os
import urllib.request
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import canvas as C

MAX_MEDIA_BYTES = 32 << 20
MAX_PIXELS = 64 << 20


def _read_source(src, allow_fetch: bool, timeout: float = 10.0) -> bytes:
    if isinstance(src, (bytes, bytearray)):
        data = bytes(src)
    elif not isinstance(src, str):
        raise ValueError("media source must be a URL, a path or bytes")
    elif src.startswith("data:"):
        head, _, payload = src.partition(",")
        if not payload:
            raise ValueError("empty data URL")
        data = base64.b64decode(payload, validate=False) if ";base64" in head else urllib.request.unquote_to_bytes(payload)
    elif src.startswith(("http://", "https://")):
        if not allow_fetch:
            raise ValueError("fetching media over the network is switched off on this server (send a data URL)")
        with urllib.request.urlopen(src, timeout=timeout) as r:          # noqa: S310 (scheme checked above)
            data = r.read(MAX_MEDIA_BYTES + 1)
    else:
        path = src[len("file://"):] if src.startswith("file://") else src
        if not os.path.isfile(path):
            raise ValueError(f"media file {path!r} does not exist")
        if os.path.getsize(path) > MAX_MEDIA_BYTES:
            raise ValueError("media file is too large")
        with open(path, "rb") as f:
            data = f.read()
    if len(data) > MAX_MEDIA_BYTES:
        raise ValueError(f"media exceeds {MAX_MEDIA_BYTES >> 20} MiB")
    return data


def decode_frames(src, allow_fetch: bool = False, max_frames: int = 1) -> List[np.ndarray]:
    """uint8 RGB frames [H, W, 3] of an image (one frame) or an animated image (`max_frames` sampled evenly)."""
    from PIL import Image, ImageSequence
    data = _read_source(src, allow_fetch)
    try:
        im = Image.open(io.BytesIO(data))
        if im.width * im.height > MAX_PIXELS:
            raise ValueError("image has too many pixels")
        n = getattr(im, "n_frames", 1)
        if n <= 1 or max_frames <= 1:
            return [np.asarray(im.convert("RGB"), dtype=np.uint8).copy()]
        pick = sorted({min(n - 1, int(round(i * (n - 1) / max(max_frames - 1, 1)))) for i in range(min(max_frames, n))})
        frames = []
        for i, fr in enumerate(ImageSequence.Iterator(im)):
            if i in pick:
                frames.append(np.asarray(fr.convert("RGB"), dtype=np.uint8).copy())
        return frames
    except ValueError:
        raise
    except Exception as e:      # noqa: BLE001 (PIL raises many types for damaged files)
        raise ValueError(f"cannot decode media: {e}") from e


def fit_smooth(img: np.ndarray, height: int, width: int) -> np.ndarray:
    """uint8 HWC image -> canvas (height, width): antialiased resize keeping the aspect ratio, zero padding."""
    from PIL import Image
    assert img.dtype == np.uint8 and img.ndim == 3 and img.shape[2] == 3
    h, w = img.shape[:2]
    sc = min(height / h, width / w)
    nh, nw = max(1, min(height, int(round(h * sc)))), max(1, min(width, int(round(w * sc))))
    small = Image.fromarray(img).resize((nw, nh), Image.BILINEAR, reducing_gap=2.0 if sc < 0.5 else None)
    out = np.zeros((height, width, 3), np.uint8)
    out[:nh, :nw] = np.asarray(small, dtype=np.uint8)
    return out


def split_chat_content(messages: Sequence[dict], placeholder: str) -> Tuple[List[dict], List[Tuple[str, object]]]:
    """Messages with list contents flattened to text in which every media part is `placeholder`, and the media sources
    in order: [("image" | "video", source)]."""
    out, media = [], []
    for m in messages:
        c = m.get("content")
        if not isinstance(c, list):
            out.append(m)
            continue
        text = []
        for p in c:
            if not isinstance(p, dict):
                continue
            kind = p.get("type", "text")
            if kind == "text":
                text.append(p.get("text", ""))
            elif kind in ("image_url", "image", "input_image", "video_url", "video"):
                v = p.get("image_url") or p.get("video_url") or p.get("image") or p.get("video") or p.get("url")
                src = v.get("url") if isinstance(v, dict) else v
                if src is None:
                    raise ValueError(f"{kind} part without a source")
                media.append(("video" if "video" in kind else "image", src))
                text.append(placeholder)
            else:
                raise ValueError(f"unsupported content part {kind!r}")
        out.append(dict(m, content="".join(text)))
    return out, media


def build_items(media: Sequence[Tuple[str, object]], height: int, width: int, directory: str = "/dev/shm",
                allow_fetch: bool = False, video_frames: int = 4) -> List[dict]:
    """One canvas file per media part (frames stacked); returns the request's "mm" items without segments."""
    items = []
    for kind, src in media:
        frames = decode_frames(src, allow_fetch, video_frames if kind == "video" else 1)
        fitted = [fit_smooth(f, height, width) for f in frames]
        items.append(C.write_canvas(fitted, height, width, directory))
    return items


def expand_prompt(ids: List[int], image_token_id: int, items: List[dict], seg_len) -> List[int]:
    """`ids` holds one placeholder id per media part; an item of several frames takes that many runs."""
    flat: List[int] = []
    k = 0
    for t in ids:
        if t == image_token_id:
            if k >= len(items):
                raise ValueError("more media placeholders than media parts")
            flat += [image_token_id] * items[k]["frames"]
            k += 1
        else:
            flat.append(t)
    if k != len(items):
        raise ValueError("fewer media placeholders than media parts")
    return C.expand_placeholders(flat, image_token_id, items, seg_len)
