"""Engine serving loop (rank 0 owns the socket; under TP the other ranks replay the same steps from the op log).

One iteration = one unit of work chosen by the C++ scheduler: admit a request (KV lease + prefix reuse: continue an
idle store, restore a checkpoint from the host library or the NVMe cache, or start cold), one prefill chunk, one
batched speculative round over all decoding sequences, or a cancellation.  Reference: engine-rs/src/
spec_probe.rs:2407-2708, qwen/serve.rs:158-470.
"""
from __future__ import annotations

import os
import select
import socket
import time
from typing import Dict, List, Optional

import torch

from ..cache.kv import KvManager
from ..cache.prefix import CheckpointLibrary, DiskPrefixCache
from ..config import EngineConfig, ModelConfig
from ..models.model import Model
from ..models.plan import make_plan
from ..runtime import rt
from ..spec.decoder import SeqSpec, SpecDecoder
from ..spec.lookup import LookupIndex
from ..utils.profile import Profiler
from . import protocol as proto


class _Live:
    def __init__(self, msg, now):
        self.id = msg["id"]
        self.msg = msg
        self.t_arrive = now
        self.t_admit = self.t_first = None
        self.prefill_ms = self.decode_ms = 0.0
        self.rounds = 0
        self.seq: Optional[SeqSpec] = None
        self.prefix_hit = 0
        self.sent = 0
        self.mm: list = []              # parsed media items of the request (multimodal/canvas.py)
        self.mm_rows: dict = {}         # (item index, frame) -> encoded rows, kept while the prompt is being prefilled


class EngineServer:
    def __init__(self, cfg: ModelConfig, W: dict, ecfg: Optional[EngineConfig] = None, device="cpu", tp=None,
                 leader=None, vision=None):
        """`leader`: a `serving.replica.Leader` when other ranks replay this server's inputs and steps.
        `vision`: (VisionConfig, weights) of the vision tower; requests may then carry media ("mm" items: canvas files
        and the prompt positions of their salted placeholder runs), which are encoded while their chunks are prefilled
        and written over the embedding rows of those positions.  Every rank encodes the same canvases with the same
        weights, so followers need no extra traffic."""
        self.cfg, self.ecfg = cfg, ecfg or EngineConfig()
        self.leader = leader
        self.tower = None
        if vision is not None:
            from ..multimodal.vision import VisionTower
            vcfg, vW = vision
            assert vcfg.out_hidden == cfg.hidden, "the aligner must project to the model's hidden size"
            self.tower = VisionTower(vcfg, vW, device=device, dtype=torch.float32 if str(device) == "cpu" else torch.bfloat16)
        e = self.ecfg
        dtype = torch.float32 if str(device) == "cpu" else torch.bfloat16
        per = max(256, e.kv_tokens // e.max_seqs // 256 * 256)
        backing = None
        if e.kv_backing == "vmm":
            from ..cache.kv import KvBacking
            backing = KvBacking(device)
        self.model = Model(cfg, W, device=device, dtype=dtype, n_slots=e.max_seqs, kv_tokens=per * e.max_seqs,
                           slot_tokens=per, tp=tp, kv_backing=backing)
        self.slot_tokens = per
        self.kv = KvManager(self.model, granule=256)
        self.sched = rt().Scheduler(e.max_seqs, per * e.max_seqs, per, e.prefill_chunk, e.max_seqs)
        drafter = "mtp" if (e.spec == "mtp" and self.model.mtp_layers) else (lambda s, d: ([], []))
        if e.spec == "lookup":
            drafter = "lookup"
        elif e.spec in ("feature", "stage"):
            # model-conditioned drafters beside the MTP head (randomly initialised unless the checkpoint carries them:
            # W["drafter"]); both are callables (seq, depth) -> (tokens, confidences)
            from ..spec import drafters as D
            if e.spec == "feature":
                dc = D.FeatureDrafterConfig(target_hidden=cfg.hidden, taps=(0, max(0, cfg.n_layers - 1)), vocab=cfg.vocab,
                                            sub_vocab=min(512, cfg.vocab), depth=max(1, e.spec_depth))
                drafter = D.FeatureDrafter(self.model, dc, W.get("drafter"), seed=e.seed,
                                           device=device if str(device) != "cpu" else "cpu")
            else:
                drafter = D.StageDrafter(D.StageDrafterConfig(hidden=cfg.hidden, vocab=cfg.vocab, block=max(1, e.spec_depth)),
                                         W.get("drafter"), seed=e.seed)
        self.spec = SpecDecoder(self.model, drafter, depth=e.spec_depth if e.spec != "none" else 0,
                                policy={"theta": "theta", "tau": "tau", "rate": "rate"}.get(e.spec_policy, "all"),
                                graphs=e.cuda_graphs)
        self.library = CheckpointLibrary(8)
        self.disk = DiskPrefixCache(e.pcache_dir, [cfg.name, cfg.to_json(), e.numerics], e.pcache_bytes) if e.pcache_dir else None
        self.live: Dict[int, _Live] = {}
        self.by_slot: Dict[int, _Live] = {}
        self.prof = Profiler(e.profile)
        self.totals = {"prompt_tokens": 0, "generation_tokens": 0, "requests": 0, "spec_rounds": 0, "drafted_tokens": 0,
                       "accepted_drafts": 0, "prefix_hit_tokens": 0, "disk_restores": 0, "prefill_steps": 0,
                       "prefill_shared_steps": 0}
        self.out: List[dict] = []
        self.shutdown = False
        self.watchdog = None
        # host memory guard (native watch thread): while available host memory is below the floor new requests are
        # refused, the host checkpoint library is halved and malloc arenas are trimmed, so the process sheds load
        # before the kernel's OOM killer picks it.  Reference: engine-rs/src/ds41/mem.rs:48-163, host_memory.rs:22-104.
        self.memwatch, self._mem_fired, self.mem_low_until = None, 0, 0.0
        if e.host_mem_floor_gb > 0:
            self.memwatch = rt().MemWatch(int(e.host_mem_floor_gb * (1 << 30)), 250, None, e.meminfo_path)
            self.totals["host_mem_low_events"] = 0
        if e.step_deadline_s > 0:                 # fail-stop on a stuck step: the process is aborted, never the device
            from ..parallel.faults import StepWatchdog
            self.watchdog = StepWatchdog(e.step_deadline_s)

    # ------------------------------------------------------------------------------------------ requests
    def _host_memory_low(self) -> bool:
        """Polls the guard: a new firing sheds host memory once and opens a 2 s window in which requests are refused."""
        if self.memwatch is None:
            return False
        f = self.memwatch.fired()
        if f != self._mem_fired:
            self._mem_fired = f
            self.mem_low_until = time.monotonic() + 2.0
            self.totals["host_mem_low_events"] += 1
            while len(self.library.items) > max(1, self.library.max // 2):
                self.library.items.popitem(last=False)
            rt().trim_host_memory()
        return time.monotonic() < self.mem_low_until

    def submit(self, msg: dict, replay: bool = False):
        if not replay and "prompt_ids" in msg and self._host_memory_low():
            msg = dict(msg)
            msg["_refuse"] = "host memory is low; retry later"   # the leader decides, followers replay the decision
        if self.leader is not None and not replay and not msg.get("stats"):
            msg = dict(msg)
            msg.setdefault("_t_arrive", time.time())        # followers schedule with the leader's arrival time
            self.leader.message(msg)
        now = float(msg.get("_t_arrive", time.time()))
        if "cancel" in msg:
            self.sched.cancel(int(msg["cancel"]))
            return
        if msg.get("shutdown"):
            self.shutdown = True
            return
        if msg.get("stats"):
            self.out.append({"id": msg.get("id"), "stats": self.stats()})
            return
        err = msg.get("_refuse") or proto.validate_request(msg, self.cfg.vocab, self.slot_tokens)
        if err:
            self.out.append({"id": msg.get("id"), "error": err})
            return
        items = []
        if msg.get("mm"):
            from ..multimodal import canvas as mmc
            try:
                if self.tower is None:
                    raise ValueError("this engine has no vision tower")
                tc = self.tower.c
                items = mmc.parse_items(msg["mm"], lambda it: tc.rows_for(it.height, it.width))
                mmc.validate(msg["prompt_ids"], self.cfg.vocab, items)
            except (ValueError, KeyError, TypeError, OSError) as e:
                self.out.append({"id": msg.get("id"), "error": f"media: {e}"})
                return
        R = rt().Request()
        R.id, R.prompt, R.max_new = int(msg["id"]), list(msg["prompt_ids"]), int(msg.get("max_new", 256))
        R.stop = list(msg.get("stop_token_ids", []))
        R.temperature, R.seed, R.t_arrive = float(msg.get("temperature", 0.0)), int(msg.get("seed", 0)), now
        self.live[R.id] = _Live(msg, now)
        self.live[R.id].mm = items
        self.sched.submit(R)
        self.out.append({"id": R.id, "queued": True})

    def stats(self) -> dict:
        d = dict(self.sched.stats())
        d.update(self.kv.stats())
        d.update(self.totals)
        if self.disk:
            d["pcache"] = self.disk.stats()
        d["sections_ms"] = self.prof.table()
        return d

    # ------------------------------------------------------------------------------------------ steps
    def step(self, replay: bool = False) -> bool:
        """Run one unit of work.  Returns False when idle.  With a leader attached the step is first marked in the op
        log and only runs once every follower has picked the mark up (its collectives need all ranks)."""
        K = rt().Step.Kind
        disk_tokens = 0
        if self.leader is not None and not replay:
            if not self.sched.has_work():
                return False
            self.leader.step()
        st = self.sched.next(disk_tokens)
        if st.kind == K.Idle:
            return False
        if self.watchdog is not None:
            with self.watchdog.step(str(st.kind)):
                self._run_step(st, K)
        else:
            self._run_step(st, K)
        return True

    def _run_step(self, st, K):
        if st.kind == K.Admit:
            self._admit(st.admit)
        elif st.kind == K.Prefill:
            self._prefill([(p.slot, p.begin, p.end) for p in st.parts])
        elif st.kind == K.Decode:
            self._decode(list(st.decode_slots))
        elif st.kind == K.Cancel:
            self._finish(st.slot, "cancelled")

    def _admit(self, plan):
        lv = self.live.get(plan.request_id)
        if plan.slot < 0:
            self.sched.on_admitted(plan)
            if lv:
                self.out.append({"id": lv.id, "error": "request does not fit the KV budget"})
                self.live.pop(lv.id, None)
            return
        m, msg = self.model, lv.msg
        prompt = msg["prompt_ids"]
        need = len(prompt) + int(msg.get("max_new", 256))
        reuse = 0
        RK = rt().ReuseKind
        if plan.kind == RK.ContinueStore and plan.slot in self.kv.lease and self.kv.grow(plan.slot, need):
            reuse = min(plan.reuse_tokens, m.seqs[plan.slot].length)
            self.kv.pool.pin(self.kv.lease[plan.slot], True)
        else:
            if not self.kv.assign(plan.slot, need):
                self.sched.on_admitted(plan)
                self.out.append({"id": lv.id, "error": "KV pool exhausted"})
                self.sched.on_finished(plan.slot)
                self.live.pop(lv.id, None)
                return
            m.reset_slot(plan.slot)
            hit = self.library.longest_prefix(prompt)
            if hit is not None:
                m.restore(plan.slot, hit[1])
                reuse = hit[1]["length"]
            elif self.disk is not None:
                t, key = self.disk.lookup(prompt)
                snap = self.disk.load(key) if t else None
                if snap is not None:
                    m.restore(plan.slot, snap)
                    reuse = snap["length"]
                    self.totals["disk_restores"] += 1
        # the scheduler's plan carries its own estimate; the executor reports what was really reused
        reuse = min(reuse, len(prompt) - 1)
        m.seqs[plan.slot].length = reuse
        self.sched.on_admitted(plan)
        self.sched.on_prefilled(plan.slot, reuse)
        lv.t_admit = time.time()
        lv.prefix_hit = reuse
        self.totals["prefix_hit_tokens"] += reuse
        self.by_slot[plan.slot] = lv
        lv.seq = SeqSpec(plan.slot, -1, temperature=float(msg.get("temperature", 0.0)), seed=int(msg.get("seed", 0)))
        lv.seq.lookup = LookupIndex(self.spec.lookup_n)
        lv.seq.lookup.extend([t for t in prompt[:reuse] if t < self.cfg.vocab])
        self._log("admit", id=lv.id, slot=plan.slot, kind=str(plan.kind).split(".")[-1], reuse=reuse, prompt=len(prompt),
                  queue_ms=round((lv.t_admit - lv.t_arrive) * 1e3, 2))

    def _prefill(self, parts):
        """One forward over a prefill chunk of every listed sequence: parts = [(slot, first token, end)], one segment
        each (the scheduler shares its chunk budget among the sequences that still have prompt tokens)."""
        m = self.model
        t0 = time.time()
        lives = [self.by_slot[slot] for slot, _, _ in parts]
        with self.prof.section("prefill"):
            items = [(slot, lv.msg["prompt_ids"][c0:c1], c0) for (slot, c0, c1), lv in zip(parts, lives)]
            plan = make_plan(items, device=m.device, all_logits=False)
            for (slot, c0, c1), lv, seg in zip(parts, lives, plan.segs):
                if lv.mm:
                    from ..multimodal import canvas as mmc
                    rows = mmc.chunk_rows(lv.mm, c0, c1 - c0, lambda it, f, lv=lv: self._encode_media(lv, it, f))
                    plan.mm_rows = (plan.mm_rows or []) + [(seg.r0 + r, t) for r, t in rows]
                    if c1 == len(lv.msg["prompt_ids"]):
                        lv.mm_rows.clear()
            logits = m.forward(plan)
            hid = m.hidden_out
            if m.mtp_layers:
                mtp_items, rows = [], []
                for (slot, c0, c1), lv, seg in zip(parts, lives, plan.segs):
                    nxt = lv.msg["prompt_ids"][c0 + 1: c1 + 1]
                    if nxt:
                        mtp_items.append((slot, nxt, c0))
                        rows.append(hid[seg.r0: seg.r0 + len(nxt)])
                if mtp_items:
                    mplan = make_plan(mtp_items, device=m.device, all_logits=False)
                    mplan.has_media = any(lv.mm for lv in lives)
                    m.mtp_forward(mplan, rows[0] if len(rows) == 1 else torch.cat(rows))
        dt = (time.time() - t0) * 1e3
        self._log("prefill", parts=[(slot, c0, c1) for slot, c0, c1 in parts], rows=sum(c1 - c0 for _, c0, c1 in parts),
                  ms=round(dt, 2))
        self.totals["prefill_steps"] += 1
        self.totals["prefill_shared_steps"] += len(parts) > 1
        for k, ((slot, c0, c1), lv, seg) in enumerate(zip(parts, lives, plan.segs)):
            prompt = lv.msg["prompt_ids"]
            lv.seq.lookup.extend([t for t in prompt[c0:c1] if t < self.cfg.vocab])    # media placeholders are never drafted
            lv.prefill_ms += dt / len(parts)
            self.sched.on_prefilled(slot, c1)
            if c1 == len(prompt):
                s = lv.seq
                h_last = hid[seg.r0 + seg.n - 1].clone()
                first = m.sample(logits[k], s.temperature, s.seed, len(prompt))
                s.last_token, s.hidden = first, h_last
                s.pending_mtp = [(h_last.clone(), first)]
                s.generated = [first]
                s.lookup.extend([first])
                lv.t_first = time.time()
                self.totals["prompt_tokens"] += len(prompt)
                boundary = len(prompt) // 256 * 256
                if self.disk is not None and boundary and boundary == len(prompt):
                    self.disk.save(prompt, m.snapshot(slot))
                self._emit(lv, [first])

    def _log(self, tag: str, **kv):
        """`[serve-<tag>] key=value ...` on stderr when EngineConfig.serve_log is set (reference: GLM53_SERVE_LOG lines
        `[serve-round] rows .. accepted .. round_ms`, `[serve-admit]`, spec_probe.rs:1795,1838,2570)."""
        if self.ecfg.serve_log:
            import sys
            print(f"[serve-{tag}] " + " ".join(f"{k}={v}" for k, v in kv.items()), file=sys.stderr, flush=True)

    def _trace_round(self, rec: dict):
        """One JSON line per speculative round (EngineConfig.draft_trace; reference: GLM53_DRAFT_TRACE, spec_probe.rs:1818-1827)."""
        path = self.ecfg.draft_trace
        if not path:
            return
        import json
        import sys
        line = json.dumps(rec, separators=(",", ":"))
        if path == "-":
            print(line, file=sys.stderr, flush=True)
        else:
            with open(path, "a") as f:
                f.write(line + "\n")

    def _encode_media(self, lv: _Live, item, frame: int) -> torch.Tensor:
        """Rows of one canvas frame; a segment that straddles prefill chunks is encoded once."""
        key = (id(item), frame)
        if key not in lv.mm_rows:
            from ..multimodal import canvas as mmc
            with self.prof.section("vision"):
                lv.mm_rows[key] = self.tower.encode(mmc.load_frame(item, frame))
            self.totals["media_frames"] = self.totals.get("media_frames", 0) + 1
        return lv.mm_rows[key]

    def _emit(self, lv: _Live, toks: List[int]):
        msg = lv.msg
        stop = set(msg.get("stop_token_ids", []))
        max_new = int(msg.get("max_new", 256))
        self.out.append({"id": lv.id, "delta": toks})
        lv.sent += len(toks)
        self.totals["generation_tokens"] += len(toks)
        done = lv.sent >= max_new or (toks and toks[-1] in stop)
        self.sched.on_tokens(lv.seq.slot, toks, False)
        if done:
            self._finish(lv.seq.slot, "stop" if (toks and toks[-1] in stop) else "length")

    def _decode(self, slots: List[int]):
        lvs = [self.by_slot[s] for s in slots]
        t0 = time.time()
        budgets = [int(lv.msg.get("max_new", 256)) - lv.sent for lv in lvs]
        before = [(lv.seq.drafted, lv.seq.accepted) for lv in lvs]
        stops = set()
        for lv in lvs:
            stops.update(lv.msg.get("stop_token_ids", []))
        with self.prof.section("spec.round"):
            widths = [int(x) for x in self.ecfg.spec_tree_widths.split(",") if x.strip()]
            drafter = self.spec.drafter
            if widths and hasattr(drafter, "candidates"):
                # tree verification: the drafter's top candidates per depth hang off the greedy spine as siblings
                from ..spec.drafters import to_tree
                trees = [to_tree(drafter.candidates(lv.seq), widths) for lv in lvs]
                outs = self.spec.round_tree([lv.seq for lv in lvs], trees, budgets, stop=tuple(stops))
            else:
                outs = self.spec.round([lv.seq for lv in lvs], budgets, stop=tuple(stops))
        dt = (time.time() - t0) * 1e3
        self.totals["spec_rounds"] += 1
        if self.ecfg.serve_log or self.ecfg.draft_trace:
            drafted = [lv.seq.drafted - b[0] for lv, b in zip(lvs, before)]
            accepted = [lv.seq.accepted - b[1] for lv, b in zip(lvs, before)]
            self._log("round", streams=len(lvs), rows=len(lvs) + sum(drafted), drafted=drafted, accepted=accepted,
                      emitted=[len(o) for o in outs], round_ms=round(dt, 2))
            self._trace_round({"round": self.totals["spec_rounds"], "ms": round(dt, 3),
                               "seqs": [{"id": lv.id, "slot": s, "pos": self.model.seqs[s].length, "drafted": d, "accepted": a,
                                         "emitted": list(o)} for lv, s, d, a, o in zip(lvs, slots, drafted, accepted, outs)]})
        for lv, out in zip(lvs, outs):
            lv.decode_ms += dt
            lv.rounds += 1
            own_stop = set(lv.msg.get("stop_token_ids", []))
            cut = []
            for t in out:
                cut.append(t)
                if t in own_stop:
                    break
            self._emit(lv, cut)

    def _finish(self, slot: int, reason: str):
        lv = self.by_slot.pop(slot, None)
        if lv is None:
            self.sched.on_finished(slot)
            return
        s = lv.seq
        self.totals["requests"] += 1
        self.totals["drafted_tokens"] += s.drafted
        self.totals["accepted_drafts"] += s.accepted
        gen = s.generated[: lv.sent]
        self.out.append({"id": lv.id, "done": True, "token_ids": gen, "finish_reason": reason,
                         "queue_ms": round(((lv.t_admit or time.time()) - lv.t_arrive) * 1e3, 3),
                         "prefill_ms": round(lv.prefill_ms, 3), "decode_ms": round(lv.decode_ms, 3),
                         "ttft_ms": round(((lv.t_first or time.time()) - lv.t_arrive) * 1e3, 3),
                         "prefix_hit_tokens": lv.prefix_hit, "rounds": lv.rounds, "accepted_drafts": s.accepted,
                         "drafted_tokens": s.drafted})
        # keep the finished store for prefix reuse: history = prompt + generated tokens that are in the state
        m = self.model
        L = m.seqs[slot].length
        if reason != "cancelled" and 0 < L <= 8192:
            self.library.save((lv.msg["prompt_ids"] + gen)[:L], m.snapshot(slot))
        self.kv.idle(slot)
        self.sched.on_finished(slot)
        self.live.pop(lv.id, None)

    # ------------------------------------------------------------------------------------------ socket loop
    def prewarm(self, prompt_tokens: int = 24) -> int:
        """Synthetic requests for 1 .. max_seqs concurrent streams through the normal admit / prefill / round path, so
        that the decode, verify, drafter and commit graphs of those stream counts are captured (and every scratch buffer
        sized) before the first client arrives.  Every rank calls this on its own before it serves: the requests are
        deterministic, so the ranks of a sharded model run identical steps.  Outputs and counters are discarded.
        Reference: engine-rs/src/spec_probe.rs:2215-2311 (graph prewarm, vision warm-up).  Returns the steps run."""
        saved_totals, saved_leader, saved_disk = dict(self.totals), self.leader, self.disk
        self.leader = self.disk = None          # nothing is replicated or written to the prefix cache
        steps, rid = 0, -(1 << 30)
        try:
            for n in range(1, self.ecfg.max_seqs + 1):
                for i in range(n):
                    rid += 1
                    prompt = [(17 * n + 5 * i + 3 * j + 1) % min(self.cfg.vocab, 30000) for j in range(prompt_tokens)]
                    self.submit({"id": rid, "prompt_ids": prompt, "max_new": max(4, 2 * (self.ecfg.spec_depth + 1)),
                                 "temperature": 0.0}, replay=True)
                guard = 0
                while self.sched.has_work() and guard < 10000:
                    self.step(replay=True)
                    steps += 1
                    guard += 1
                self.out = []
        finally:
            self.leader, self.disk = saved_leader, saved_disk
            self.totals = saved_totals
            self.out = []
        return steps

    def serve_forever(self, path: str, idle_sleep: float = 0.002, ready_cb=None):
        if self.ecfg.prewarm:
            t0 = time.time()
            n = self.prewarm()
            print(f"[serve] prewarm: {n} steps in {time.time() - t0:.1f} s", flush=True)
        if os.path.exists(path):
            os.unlink(path)
        srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        srv.bind(path)
        srv.listen(4)
        srv.setblocking(False)
        conns: Dict[socket.socket, proto.LineBuffer] = {}
        owner: Dict[int, socket.socket] = {}
        outbuf: Dict[socket.socket, bytearray] = {}      # bytes accepted for a connection but not yet sent
        print("[serve] rank0 ready", flush=True)
        if ready_cb:
            ready_cb()
        while not self.shutdown:
            rl, _, _ = select.select([srv] + list(conns), [], [], 0)
            for s in rl:
                if s is srv:
                    c, _ = srv.accept()
                    c.setblocking(False)
                    conns[c] = proto.LineBuffer()
                    continue
                try:
                    data = s.recv(1 << 16)
                except BlockingIOError:
                    continue
                except ConnectionError:
                    data = b""
                if not data:                          # front end gone: cancel everything it owns
                    for rid, c in list(owner.items()):
                        if c is s:
                            self.submit({"cancel": rid})      # through submit: followers replay the cancellation
                            owner.pop(rid, None)
                    conns.pop(s, None)
                    s.close()
                    continue
                for msg in conns[s].feed(data):
                    if "id" in msg and "prompt_ids" in msg:
                        owner[int(msg["id"])] = s
                    if msg.get("stats"):
                        owner[msg.get("id", -1)] = s
                    self.submit(msg)
            busy = self.step()
            for msg in self.out:
                c = owner.get(msg.get("id", -1))
                if c is None and conns:
                    c = next(iter(conns))
                if c is not None and c in conns:
                    outbuf.setdefault(c, bytearray()).extend(proto.encode(msg))
                if msg.get("done") or msg.get("error"):
                    owner.pop(msg.get("id", -1), None)
            self.out = []
            # non-blocking sockets may take only part of a line: keep the rest and send it when the socket drains, so
            # the line protocol to the front end is never cut in the middle of a message
            for c in list(outbuf):
                buf = outbuf[c]
                if c not in conns:
                    outbuf.pop(c, None)
                    continue
                try:
                    while buf:
                        n = c.send(buf)
                        if n <= 0:
                            break
                        del buf[:n]
                except BlockingIOError:
                    pass
                except (ConnectionError, OSError):
                    outbuf.pop(c, None)
                    continue
                if not buf:
                    outbuf.pop(c, None)
            if self.leader is not None:
                self.leader.heartbeat()
            if not busy and not outbuf:
                time.sleep(idle_sleep)
        if self.leader is not None:
            self.leader.shutdown()
        for c in conns:
            c.close()
        srv.close()
        if os.path.exists(path):
            os.unlink(path)
