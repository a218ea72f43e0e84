"""Lock-step replication of the serving loop over the ranks of one box.

Rank 0 (the leader) owns the socket and the decisions; every other rank (a follower) runs the same `EngineServer`
on its own shard and replays the leader's inputs in the same order: request submissions (the full JSON, with the
leader's arrival time), cancellations, and "run one scheduler step" marks.  The schedulers are deterministic, the
collectives give bit-identical logits on every rank and sampling is keyed by (seed, position), so all ranks take the
same decisions without ever exchanging them.  The transport is the shared-memory op log of the native runtime
(`csrc/runtime/oplog.cpp`); long requests span several records.

Failure detection stays on the host: before a step that needs every rank's collectives the leader waits (bounded)
until all followers have read the step mark, and raises `FollowerLost` otherwise -- nothing is launched towards a
rank that has stopped; a follower that sees neither an op nor a heartbeat before its deadline raises `LeaderLost`.
Reference: engine-rs/src/spec_probe.rs:1515,1741-1758,2355-2383 (replicated op log, follower loop, doorbell),
ds41/serve.rs:266-300 (one JSON step per round on a control channel).
"""
from __future__ import annotations

import json
import time
from typing import Optional

from ..runtime import rt

OP_MSG_PART, OP_MSG_END, OP_STEP, OP_SHUTDOWN, OP_HEARTBEAT = 1, 2, 3, 4, 5
_CHUNK = 1016 * 4                         # payload bytes per record (1018 ints; one holds the byte count)


class FollowerLost(RuntimeError):
    pass


class LeaderLost(RuntimeError):
    pass


def _pack(b: bytes):
    pad = (-len(b)) % 4
    ints = [len(b)]
    bb = b + b"\0" * pad
    ints += [int.from_bytes(bb[i: i + 4], "little", signed=True) for i in range(0, len(bb), 4)]
    return ints


def _unpack(ints) -> bytes:
    n = ints[0]
    raw = b"".join(int(v).to_bytes(4, "little", signed=True) for v in ints[1:])
    return raw[:n]


class Leader:
    def __init__(self, name: str, n_followers: int, ack_timeout_ms: int = 5000):
        self.log = rt().OpLog(name, True, n_followers, -1)
        self.n, self.ack_timeout_ms = n_followers, ack_timeout_ms
        self.last_beat = time.monotonic()

    def _append(self, kind: int, payload):
        seq = self.log.append(kind, payload, self.ack_timeout_ms)
        if seq == 0:
            raise FollowerLost("a follower stopped reading the op log (ring full)")
        self.last_beat = time.monotonic()
        return seq

    def message(self, msg: dict):
        """A submission / cancellation / stats request, exactly as the leader applies it."""
        raw = json.dumps(msg, separators=(",", ":")).encode()
        for off in range(0, max(len(raw), 1), _CHUNK):
            part = raw[off: off + _CHUNK]
            self._append(OP_MSG_END if off + _CHUNK >= len(raw) else OP_MSG_PART, _pack(part))

    def step(self):
        """Mark one scheduler step and wait until every follower has read the mark (they are about to run it too)."""
        seq = self._append(OP_STEP, [])
        lost = self.log.wait_acked(seq, self.ack_timeout_ms)
        if lost >= 0:
            raise FollowerLost(f"follower {lost + 1} did not pick up step {seq} within {self.ack_timeout_ms} ms")

    def heartbeat(self, period_s: float = 0.5):
        if time.monotonic() - self.last_beat >= period_s:
            self._append(OP_HEARTBEAT, [])

    def shutdown(self):
        try:
            self._append(OP_SHUTDOWN, [])
        except FollowerLost:
            pass


class Follower:
    def __init__(self, name: str, index: int, n_followers: int, deadline_ms: int = 5000, open_timeout_s: float = 60.0):
        t0 = time.monotonic()
        while True:                              # the leader creates the log; wait for it (bounded)
            try:
                self.log = rt().OpLog(name, False, n_followers, index)
                break
            except RuntimeError:
                if time.monotonic() - t0 > open_timeout_s:
                    raise LeaderLost("the leader never created the op log")
                time.sleep(0.02)
        self.seq, self.deadline_ms = 0, deadline_ms
        self._parts = []
        self.finished = {}                       # request id -> token ids this rank produced (for cross-rank checks)

    def run(self, server, max_ops: Optional[int] = None) -> int:
        """Replay the leader's ops on `server` until shutdown (or `max_ops` ops, for tests).  Returns the ops applied."""
        done = 0
        while max_ops is None or done < max_ops:
            ok, kind, payload = self.log.next(self.seq, self.deadline_ms)
            if not ok:
                raise LeaderLost(f"no op and no heartbeat from the leader for {self.deadline_ms} ms")
            self.seq += 1
            done += 1
            if kind == OP_HEARTBEAT:
                continue
            if kind == OP_SHUTDOWN:
                server.shutdown = True
                break
            if kind in (OP_MSG_PART, OP_MSG_END):
                self._parts.append(_unpack(payload))
                if kind == OP_MSG_END:
                    msg = json.loads(b"".join(self._parts).decode())
                    self._parts = []
                    server.submit(msg, replay=True)
                continue
            if kind == OP_STEP:
                server.step(replay=True)
                for m in server.out:             # replies belong to the leader's socket; keep the final ids only
                    if m.get("done"):
                        self.finished[m["id"]] = m["token_ids"]
                server.out = []
        return done
