"""KV pool manager: leases token regions of the per-GPU KV pool to sequence slots (C++ `KvPool`), evicts idle
stores LRU, and keeps the model runner's per-slot regions in sync.  Reference: engine-rs/src/kv_pool.rs:53-241."""
from __future__ import annotations

from typing import Dict, Optional

from ..runtime import rt


class KvBacking:
    """Device memory behind the model's KV tensors as growable virtual ranges: every per-token tensor (keys, values,
    scales, indexer keys, pooled keys, latent rows) reserves address space for the whole token budget and maps physical
    chunks only up to the highest token any lease reaches.  Addresses never move, so captured graphs and leases stay
    valid while the backing grows or shrinks.  Rows past the backed size are unmapped: nothing may touch them, which the
    lease bookkeeping guarantees (`KvManager` backs a region before it hands it out).
    Reference: engine-rs/src/kv_pool.rs:53-241 (VMM backend), shim/vmm.cpp."""

    def __init__(self, device, fake: bool = False, min_tokens: int = 256):
        import torch
        self.dev = torch.device(device)
        self.fake = fake or self.dev.type != "cuda"
        self.index = self.dev.index if self.dev.index is not None else 0
        self.min_tokens = min_tokens
        self.bufs = []                 # (GrowableDeviceBuffer, tensor over the whole range, row bytes, rows_of(tokens))
        self.tokens = 0

    def alloc(self, rows_total: int, row_shape, dtype, rows_of):
        """A zero tensor [rows_total, *row_shape] whose first rows_of(tokens) rows are backed once `ensure(tokens)` ran."""
        import math
        import torch
        from ..utils.devmem import GrowableDeviceBuffer
        row_bytes = int(math.prod(row_shape) if row_shape else 1) * torch.empty((), dtype=dtype).element_size()
        buf = GrowableDeviceBuffer(self.index, max(rows_total * row_bytes, 1), fake=self.fake)
        buf.resize(max(rows_of(self.min_tokens) * row_bytes, 1))          # the base address must be mapped before torch sees it
        t = buf.view_unchecked(rows_total * row_bytes).view(dtype).view(rows_total, *row_shape)
        t[: buf.size // row_bytes].zero_()
        self.bufs.append((buf, t, row_bytes, rows_of))
        return t

    def ensure(self, tokens: int):
        """Back every tensor up to `tokens` tokens (newly mapped rows are zeroed)."""
        if tokens <= self.tokens:
            return
        for buf, t, row_bytes, rows_of in self.bufs:
            need = min(rows_of(tokens), t.shape[0]) * row_bytes
            old = buf.size
            if need > old:
                buf.resize(need)
                t[old // row_bytes: min(buf.size // row_bytes, t.shape[0])].zero_()
        self.tokens = tokens

    def shrink(self, tokens: int):
        """Unmap what lies past `tokens` tokens (never below the initial mapping)."""
        tokens = max(tokens, self.min_tokens)
        if tokens >= self.tokens:
            return
        if not self.fake:
            import torch
            torch.cuda.synchronize(self.dev)      # no kernel in flight may still address the rows that are about to go
        for buf, t, row_bytes, rows_of in self.bufs:
            buf.resize(max(min(rows_of(tokens), t.shape[0]) * row_bytes, 1))
        self.tokens = tokens

    def backed_bytes(self) -> int:
        return sum(b.size for b, _, _, _ in self.bufs)


class KvManager:
    def __init__(self, model, granule: int = 256):
        self.model = model
        self.pool = rt().KvPool(model.kv_tokens, granule)
        self.lease: Dict[int, int] = {}           # slot -> lease id
        self.backing = getattr(model, "kv_backing", None)

    def _back(self):
        """Grow / shrink the physical backing to the highest token any live lease can reach."""
        if self.backing is None:
            return
        top = 0
        for lid in self.lease.values():
            l = self.pool.get(lid)
            top = max(top, l.base + l.cap)
        if top > self.backing.tokens:
            self.backing.ensure(top)
        elif top < self.backing.tokens:
            self.backing.shrink(top)

    def assign(self, slot: int, tokens: int) -> bool:
        """Give `slot` room for `tokens` rows (evicting idle stores if needed).  False = does not fit."""
        self.release(slot)
        lid = self.pool.acquire(tokens)
        while lid < 0:
            v = self.pool.lru_victim()
            if v < 0:
                return False
            owner = next((s for s, l in self.lease.items() if l == v), None)
            self.pool.release(v)
            if owner is not None:
                del self.lease[owner]
                self.model.reset_slot(owner)
            lid = self.pool.acquire(tokens)
        l = self.pool.get(lid)
        self.lease[slot] = lid
        self.pool.pin(lid, True)
        self._back()                                  # the rows exist before anything may address them
        self.model.set_kv_region(slot, l.base, l.cap)
        return True

    def grow(self, slot: int, tokens: int) -> bool:
        lid = self.lease[slot]
        if not self.pool.grow(lid, tokens):
            return False
        l = self.pool.get(lid)
        self._back()
        self.model.set_kv_region(slot, l.base, l.cap)
        return True

    def idle(self, slot: int):
        """The sequence finished: keep its rows for prefix reuse but allow eviction."""
        if slot in self.lease:
            self.pool.pin(self.lease[slot], False)
            self.pool.set_used(self.lease[slot], self.model.seqs[slot].length)
            self.pool.touch(self.lease[slot])

    def release(self, slot: int):
        lid = self.lease.pop(slot, None)
        if lid is not None:
            self.pool.release(lid)
            self._back()

    def stats(self) -> dict:
        d = {"kv_budget": self.pool.total(), "kv_allocated": self.pool.allocated_tokens(),
             "kv_active": self.pool.active_tokens(), "kv_free_run": self.pool.largest_free_run()}
        if self.backing is not None:
            d["kv_backed_tokens"], d["kv_backed_bytes"] = self.backing.tokens, self.backing.backed_bytes()
        return d
