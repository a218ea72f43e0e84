"""Host-resident n-gram tables with asynchronous row gathers.

The hashed n-gram tables of the DS-style and Qwen-style models are far larger than what the device should hold
(2 x 98 GB and 39 GB in the reference), so they stay on the host: in pinned memory when they fit, else memory-mapped
from NVMe.  A request for rows is served by gather threads that copy the rows into a slot of a pinned ring and start
the host-to-device copy on a side stream; the model asks for layer L+1's rows while layer L computes and only waits
on an event when it consumes them.  Reference: engine-rs/src/ds41/engram.rs:123-509 (mmap / pread / O_DIRECT gathers,
prefetch one chunk ahead), engine-rs/shim/qwen_ple.cu.
"""
from __future__ import annotations

import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Optional

import numpy as np
import torch


class EngramTable:
    def __init__(self, table, device="cpu", ring_slots: int = 4, max_rows: int = 1 << 16, threads: int = 4):
        """`table`: a CPU tensor [rows, dim] or a path to a raw little-endian file (then `dtype`/`dim` come from
        `from_file`)."""
        self.table = table
        self.rows, self.dim = table.shape
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        pin = self.cuda
        self.ring = [torch.empty(max_rows, self.dim, dtype=table.dtype, pin_memory=pin) for _ in range(ring_slots)]
        self.dev = [torch.empty(max_rows, self.dim, dtype=table.dtype, device=self.device) for _ in range(ring_slots)] \
            if self.cuda else None
        self.max_rows = max_rows
        self.pool = ThreadPoolExecutor(max_workers=threads)
        self.threads = threads
        self.stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._next = 0
        self._lock = threading.Lock()
        self._busy = [None] * ring_slots           # event (cuda) guarding reuse of a slot
        self.stats = {"requests": 0, "rows": 0}

    @staticmethod
    def from_file(path: str, rows: int, dim: int, dtype=torch.bfloat16, **kw) -> "EngramTable":
        npdt = {torch.bfloat16: np.uint16, torch.float16: np.float16, torch.float32: np.float32, torch.uint8: np.uint8}[dtype]
        mm = np.memmap(path, dtype=npdt, mode="r", shape=(rows, dim))
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")          # the mapping is read-only on purpose; rows are only read
            t = torch.from_numpy(mm)
        return EngramTable(t.view(dtype) if dtype == torch.bfloat16 else t, **kw)

    def _gather(self, ids: torch.Tensor, dst: torch.Tensor):
        n = ids.numel()
        per = (n + self.threads - 1) // self.threads
        futs = []
        for i in range(0, n, per):
            futs.append(self.pool.submit(lambda a, b: torch.index_select(self.table, 0, ids[a:b], out=dst[a:b]), i, min(n, i + per)))
        for f in futs:
            f.result()

    def prefetch(self, row_ids: torch.Tensor) -> Future:
        """Start gathering rows (any shape of int64 ids, on the host).  The future resolves to (tensor [n, dim] on the
        device, event or None); the tensor stays valid until `ring_slots - 1` later requests."""
        ids = row_ids.reshape(-1).to("cpu", torch.long)
        n = ids.numel()
        if n > self.max_rows:
            raise ValueError(f"{n} rows exceed the ring slot of {self.max_rows} rows")
        with self._lock:
            slot = self._next
            self._next = (self._next + 1) % len(self.ring)
            self.stats["requests"] += 1
            self.stats["rows"] += n
        fut: Future = Future()

        def work():
            try:
                if self._busy[slot] is not None:
                    self._busy[slot].synchronize()
                host = self.ring[slot][:n]
                self._gather(ids, host)
                if not self.cuda:
                    fut.set_result((host, None))
                    return
                with torch.cuda.stream(self.stream):
                    self.dev[slot][:n].copy_(host, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.stream)
                self._busy[slot] = ev
                fut.set_result((self.dev[slot][:n], ev))
            except Exception as e:          # surfaced when the consumer asks for the rows
                fut.set_exception(e)
        threading.Thread(target=work, daemon=True).start()
        return fut

    @staticmethod
    def take(fut: Future) -> torch.Tensor:
        """Rows of a prefetch, ordered behind the consumer's current stream."""
        t, ev = fut.result()
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        return t

    def close(self):
        self.pool.shutdown(wait=True)
