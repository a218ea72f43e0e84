"""Failure detection on the host side, and a host model of the peer-memory protocol for fault-injection tests.

* `FakeArena` / `fake_allreduce`: the slot + sequence-number protocol of the device collectives (push my rows into
  every peer's slot, raise my flag on every peer with a release store, wait for every peer's flag with a time budget,
  sum the slots in rank order) executed by threads on ordinary memory.  A test can drop, delay or duplicate a flag write
  or never start a rank; the wait then runs out and returns the same status tuple the kernels write
  ({ST_TIMEOUT_PEER_FLAG, peer, expected sequence, last sequence seen}) instead of hanging.  Nothing here touches a GPU:
  faults are injected on the host only.
* `Heartbeat`: leader beats, followers check a deadline (control plane liveness, engine-rs/src/spec_probe.rs:2319-2366).
* `StepWatchdog`: a thread that calls `on_expire` (default: abort the *process*, never the device) when a step has been
  running past its deadline (engine-rs/shim/shim.cpp:714 NCCL watchdog; serve/start-glm.sh:23-29 liveness).
"""
from __future__ import annotations

import os
import threading
import time
from typing import Callable, List, Optional

import torch

ST_OK, ST_TIMEOUT_PEER_FLAG = 0, 5


class FakeArena:
    """World-size slots and flags per rank, plus injectable faults on flag writes: fault(src, dst, seq) may return
    "drop", "dup", or a delay in seconds."""

    def __init__(self, world: int, rows: int, n: int, fault: Optional[Callable[[int, int, int], object]] = None):
        self.world, self.rows, self.n = world, rows, n
        self.slots = [torch.zeros(2, world, rows, n) for _ in range(world)]       # [parity][src]
        self.flags = [[0] * world for _ in range(world)]                          # flags[dst][src] = last sequence
        self.lock = threading.Lock()
        self.fault = fault

    def write_flag(self, src: int, dst: int, seq: int):
        act = self.fault(src, dst, seq) if self.fault else None
        if act == "drop":
            return
        if isinstance(act, (int, float)) and act > 0:
            time.sleep(act)
        with self.lock:
            self.flags[dst][src] = max(self.flags[dst][src], seq)                 # release store; duplicates are harmless
        if act == "dup":
            with self.lock:
                self.flags[dst][src] = max(self.flags[dst][src], seq)

    def wait_flag(self, me: int, src: int, seq: int, budget_s: float):
        t0 = time.monotonic()
        seen = 0
        while True:
            with self.lock:
                seen = self.flags[me][src]
            if seen >= seq:
                return (ST_OK, 0, 0, 0)
            if time.monotonic() - t0 > budget_s:
                return (ST_TIMEOUT_PEER_FLAG, src, seq, seen)
            time.sleep(0.0005)


def fake_allreduce(arena: FakeArena, rank: int, x: torch.Tensor, seq: int, budget_s: float = 1.0):
    """One-shot all-reduce of x [rows, n] as rank `rank`: returns (status tuple, rank-ordered sum or None)."""
    par = seq & 1
    for p in range(arena.world):
        arena.slots[p][par, rank, : x.shape[0]] = x
    for p in range(arena.world):
        arena.write_flag(rank, p, seq)
    for p in range(arena.world):
        st = arena.wait_flag(rank, p, seq, budget_s)
        if st[0] != ST_OK:
            return st, None
    acc = torch.zeros_like(x)
    for p in range(arena.world):                                                  # fixed rank order
        acc = acc + arena.slots[rank][par, p, : x.shape[0]]
    return (ST_OK, 0, 0, 0), acc


class Heartbeat:
    """Leader: `beat()` at least every `period`; followers: `alive()` is False once no beat arrived for `deadline`."""

    def __init__(self, deadline_s: float = 2.0, clock: Callable[[], float] = time.monotonic):
        self.deadline, self.clock = deadline_s, clock
        self.last = clock()
        self.count = 0

    def beat(self):
        self.last = self.clock()
        self.count += 1

    def alive(self) -> bool:
        return self.clock() - self.last <= self.deadline


class StepWatchdog:
    """`with wd.step("decode round"):` arms a deadline; a background thread calls `on_expire(name, elapsed)` once if the
    step is still running after it.  Default action: write a message and abort the process (the device is left alone)."""

    def __init__(self, deadline_s: float, on_expire: Optional[Callable[[str, float], None]] = None, poll_s: float = 0.01):
        self.deadline, self.poll = deadline_s, poll_s
        self.on_expire = on_expire or self._abort
        self._cur = None
        self._lock = threading.Lock()
        self._stop = False
        self.fired: List[str] = []
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    @staticmethod
    def _abort(name: str, elapsed: float):
        os.write(2, f"[watchdog] step '{name}' exceeded its deadline ({elapsed:.1f} s): aborting the process\n".encode())
        os._exit(86)

    def _run(self):
        while not self._stop:
            with self._lock:
                cur = self._cur
            if cur is not None and not cur[2] and time.monotonic() - cur[1] > self.deadline:
                cur[2] = True
                self.fired.append(cur[0])
                self.on_expire(cur[0], time.monotonic() - cur[1])
            time.sleep(self.poll)

    def step(self, name: str):
        wd = self

        class _Ctx:
            def __enter__(self_inner):
                with wd._lock:
                    wd._cur = [name, time.monotonic(), False]

            def __exit__(self_inner, *exc):
                with wd._lock:
                    wd._cur = None
                return False
        return _Ctx()

    def close(self):
        self._stop = True
        self._thread.join(1.0)
