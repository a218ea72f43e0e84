"""Prefix reuse: in-memory checkpoint library (LRU, host memory) and the NVMe prefix cache.

A checkpoint is `Model.snapshot(slot)` at a token boundary: KV rows up to the boundary, linear-attention states and
conv tails, indexer pools.  The library keeps snapshots on the host keyed by their token prefix; the NVMe tier
serialises a snapshot into one flat buffer and hands it to the C++ `Pcache` (O_DIRECT writer thread, chunk
checksums, tmp + fdatasync + rename, LRU byte budget, identity directory).
Reference: engine-rs/src/spec_probe.rs:1420-1576 (ckpt_save/restore/clone, library LRU), pcache_core.rs:249-765.
"""
from __future__ import annotations

import io
import os
from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

import torch

from ..runtime import rt


def _flatten(snap: dict) -> Tuple[bytes, list]:
    buf = io.BytesIO()
    torch.save(snap, buf)
    return buf.getvalue()


class CheckpointLibrary:
    """Host-memory LRU of sequence checkpoints keyed by their token prefix."""

    def __init__(self, max_entries: int = 16):
        self.max = max_entries
        self.items: "OrderedDict[tuple, dict]" = OrderedDict()

    def save(self, tokens: Sequence[int], snap: dict):
        key = tuple(tokens)
        self.items[key] = {k: v for k, v in snap.items()}
        self.items.move_to_end(key)
        while len(self.items) > self.max:
            self.items.popitem(last=False)

    def longest_prefix(self, prompt: Sequence[int]) -> Optional[Tuple[tuple, dict]]:
        best = None
        p = tuple(prompt)
        for key, snap in self.items.items():
            if len(key) < len(p) and p[: len(key)] == key and (best is None or len(key) > len(best[0])):
                best = (key, snap)
        if best is not None:
            self.items.move_to_end(best[0])
        return best


class DiskPrefixCache:
    def __init__(self, root: str, identity_parts: List[str], byte_budget: int, granule: int = 256, direct_io: bool = True):
        R = rt()
        self.granule = granule
        self.pc = R.Pcache(root, R.Pcache.identity_dir(identity_parts), byte_budget, direct_io)

    def save(self, tokens: Sequence[int], snap: dict, wait: bool = True) -> bool:
        n = len(tokens) // self.granule * self.granule
        if n == 0 or snap["length"] != n:
            return False
        raw = _flatten(snap)
        key = rt().Pcache.prefix_key(list(tokens[:n]))
        return self.pc.save(key, n, raw)

    def lookup(self, prompt: Sequence[int]) -> Tuple[int, str]:
        """(tokens covered, key) of the longest cached prefix that leaves at least one prompt token to prefill."""
        t, key = self.pc.longest_prefix(list(prompt[: len(prompt) - 1]), self.granule)
        return t, key

    def load(self, key: str, max_bytes: int = 1 << 32) -> Optional[dict]:
        ent = next((e for e in self.pc.entries() if e.key == key), None)
        if ent is None:
            return None
        buf = bytearray(ent.bytes)
        n = self.pc.load(key, buf)
        if n < 0:
            return None
        return torch.load(io.BytesIO(bytes(buf[:n])), weights_only=False)

    def agree(self, group=None):
        """Keep only entries every rank holds (intersection), like the reference's `agree` all-reduce."""
        import torch.distributed as dist
        if not dist.is_initialized() or dist.get_world_size(group) == 1:
            return
        mine = sorted(e.key for e in self.pc.entries())
        all_keys = [None] * dist.get_world_size(group)
        dist.all_gather_object(all_keys, mine, group=group)
        common = set(all_keys[0]).intersection(*map(set, all_keys[1:]))
        self.pc.keep_only(sorted(common))

    def stats(self) -> dict:
        d = dict(self.pc.stats())
        d["bytes"] = self.pc.bytes_used()
        return d
