"""KV pool manager: leases token regions of the per-GPU KV pool to sequence slots (C++ `KvPool`), evicts idle
stores LRU, and keeps the model runner's per-slot regions in sync.  Reference: engine-rs/src/kv_pool.rs:53-241."""
from __future__ import annotations

from typing import Dict, Optional

from ..runtime import rt


class KvManager:
    def __init__(self, model, granule: int = 256):
        self.model = model
        self.pool = rt().KvPool(model.kv_tokens, granule)
        self.lease: Dict[int, int] = {}           # slot -> lease id

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
        self.model.set_kv_region(slot, l.base, l.cap)
        return True

    def grow(self, slot: int, tokens: int) -> bool:
        lid = self.lease[slot]
        if not self.pool.grow(lid, tokens):
            return False
        l = self.pool.get(lid)
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

    def stats(self) -> dict:
        return {"kv_budget": self.pool.total(), "kv_allocated": self.pool.allocated_tokens(),
                "kv_active": self.pool.active_tokens(), "kv_free_run": self.pool.largest_free_run()}
