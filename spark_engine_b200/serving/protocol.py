"""Engine <-> front-end line protocol: newline-delimited JSON over a Unix socket.

Requests : {"id", "prompt_ids", "max_new", "stop_token_ids", "temperature", "seed"[, "mm"]}
           {"cancel": id}   {"id", "stats": true}   {"shutdown": true}
Replies  : {"id", "queued": true}   {"id", "delta": [ids]}   {"id", "error": "..."}
           {"id", "done": true, "token_ids", "queue_ms", "prefill_ms", "decode_ms", "prefix_hit_tokens", "rounds",
            "accepted_drafts", "drafted_tokens", "finish_reason"}
           {"id", "stats": {...}}
Same fields as the reference (engine-rs/src/spec_probe.rs:2039-2048,2611-2706; qwen/serve.rs:1-10; ds41/serve.rs:1-19).
"""
from __future__ import annotations

import json
from typing import Any, Dict, List


def encode(msg: Dict[str, Any]) -> bytes:
    return (json.dumps(msg, separators=(",", ":")) + "\n").encode()


class LineBuffer:
    def __init__(self):
        self.buf = b""

    def feed(self, data: bytes) -> List[Dict[str, Any]]:
        self.buf += data
        out = []
        while b"\n" in self.buf:
            line, self.buf = self.buf.split(b"\n", 1)
            line = line.strip()
            if not line:
                continue
            try:
                out.append(json.loads(line))
            except json.JSONDecodeError:
                out.append({"error": "bad json"})
        return out


def validate_request(msg: Dict[str, Any], vocab: int, max_ctx: int) -> str:
    """Empty string if the request is well-formed, else the reason."""
    ids = msg.get("prompt_ids")
    if not isinstance(ids, list) or not ids:
        return "prompt_ids must be a non-empty list"
    # salted media placeholders (outside every vocabulary) are legal only with an "mm" array, which the engine checks
    # position by position against its canvases
    lo, hi = (1 << 20, 1 << 24) if msg.get("mm") else (0, 0)
    if any((not isinstance(t, int)) or t < 0 or (t >= vocab and not lo <= t < hi) for t in ids):
        return "prompt_ids out of range"
    mn = msg.get("max_new", 256)
    if not isinstance(mn, int) or mn <= 0:
        return "max_new must be a positive integer"
    if len(ids) + mn > max_ctx:
        return f"prompt ({len(ids)}) + max_new ({mn}) exceeds the context budget ({max_ctx})"
    return ""
