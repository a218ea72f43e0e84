"""C++ host runtime on CPU: KV pool, NVMe prefix cache (crash safety, checksums, LRU budget, reconciliation),
scheduler admission / round planning, replicated op log with a lost leader, safetensors, memory guard."""
import pytest
import os
import threading
import time

import torch

from spark_engine_b200.runtime import rt


def test_kv_pool_first_fit_grow_and_lru():
    R = rt()
    p = R.KvPool(16 * 1024, 1024)
    a, b, c = p.acquire(1000), p.acquire(3000), p.acquire(2048)
    assert (p.get(a).base, p.get(a).cap) == (0, 1024) and p.get(b).base == 1024 and p.get(b).cap == 3072
    assert not p.grow(a, 2000)                # b sits right behind a
    p.release(b)
    assert p.grow(a, 4096) and p.get(a).cap == 4096
    d = p.acquire(20000)
    assert d == -1 and p.allocated_tokens() == 4096 + 2048          # failed acquire changed nothing
    p.pin(a, True)
    assert p.lru_victim() == c
    p.set_used(c, 100)
    try:
        p.set_used(c, 5000)
        assert False
    except IndexError:
        pass
    assert p.largest_free_run() == 16 * 1024 - 6144


def test_pcache_roundtrip_corruption_eviction_and_restart(tmp_path):
    R = rt()
    ident = R.Pcache.identity_dir(["binary-sha", "model-path", "deterministic"])
    assert ident != R.Pcache.identity_dir(["binary-sha", "model-path", "fast"])
    pc = R.Pcache(str(tmp_path), ident, 3 * (1 << 20), False)
    ids = list(range(1000))
    blob = os.urandom(1 << 20)
    k1 = R.Pcache.prefix_key(ids[:512])
    assert pc.save(k1, 512, blob)
    out = bytearray(len(blob))
    assert pc.load(k1, out) == len(blob) and bytes(out) == blob
    assert pc.longest_prefix(ids, 256) == (512, k1)
    assert pc.longest_prefix(ids[:300], 256)[0] == 0
    # LRU byte budget: two more 1 MiB entries fit, the fourth evicts the least recently used
    k2, k3, k4 = (R.Pcache.prefix_key(ids[:n]) for n in (256, 768, 1000))
    assert pc.save(k2, 256, blob) and pc.save(k3, 768, blob)
    pc.load(k1, out)
    assert pc.save(k4, 1000, blob)
    assert pc.contains(k1) and not pc.contains(k2)
    # a torn file and a leftover .tmp are dropped by reconciliation after a restart
    path = os.path.join(pc.dir(), k3 + ".pc")
    with open(path, "r+b") as f:
        f.seek(5000)
        f.write(b"\x00" * 64)
    open(os.path.join(pc.dir(), "junk.pc.tmp"), "wb").write(b"partial")
    del pc
    pc2 = R.Pcache(str(tmp_path), ident, 3 * (1 << 20), False)
    assert pc2.contains(k1) and pc2.contains(k4)
    assert pc2.load(k3, out) == -1 and not pc2.contains(k3)        # chunk checksum catches the damage
    assert not os.path.exists(os.path.join(pc2.dir(), "junk.pc.tmp"))
    pc2.keep_only([k1])
    assert [e.key for e in pc2.entries()] == [k1]


def test_scheduler_prefill_shares_are_redistributed():
    """Sequences with few prompt tokens left take what they need; the long ones split the rest of the chunk budget."""
    R = rt()
    s = R.Scheduler(4, 1 << 20, 1 << 18, 64, 4)
    for i, n in enumerate((500, 5, 300, 11)):
        r = R.Request()
        r.id, r.prompt, r.max_new = i + 1, list(range(n)), 4
        s.submit(r)
        st = s.next()
        assert st.kind == R.Step.Kind.Admit
        s.on_admitted(st.admit)
    st = s.next()
    parts = sorted((p.slot, p.begin, p.end) for p in st.parts)
    assert st.kind == R.Step.Kind.Prefill and parts == [(0, 0, 24), (1, 0, 5), (2, 0, 24), (3, 0, 11)]
    for p in st.parts:
        s.on_prefilled(p.slot, p.end)
    st = s.next()                                   # slots 1 and 3 are done prefilling: a decode round comes first
    assert st.kind == R.Step.Kind.Decode and list(st.decode_slots) == [1, 3]
    st = s.next()
    assert sorted((p.slot, p.begin, p.end) for p in st.parts) == [(0, 24, 56), (2, 24, 56)]


def test_scheduler_admission_prefix_reuse_and_round_robin():
    R = rt()
    s = R.Scheduler(2, 4096, 2048, 64, 4)

    def req(i, prompt, max_new=8):
        r = R.Request()
        r.id, r.prompt, r.max_new = i, prompt, max_new
        return r
    s.submit(req(1, list(range(100))))
    st = s.next()
    assert st.kind == R.Step.Kind.Admit and st.admit.kind == R.ReuseKind.Cold and st.admit.slot == 0
    s.on_admitted(st.admit)
    st = s.next()
    assert st.kind == R.Step.Kind.Prefill and (st.chunk_begin, st.chunk_end) == (0, 64)
    s.on_prefilled(0, 64)
    s.submit(req(2, list(range(50))))
    st = s.next()
    assert st.kind == R.Step.Kind.Admit and st.admit.slot == 1
    s.on_admitted(st.admit)
    trace = []
    for _ in range(6):              # sequences that still have prompt tokens share the chunk budget of one forward
        st = s.next()
        trace.append((st.kind, [(p.slot, p.begin, p.end) for p in st.parts], list(st.decode_slots)))
        if st.kind == R.Step.Kind.Prefill:
            assert (st.slot, st.chunk_begin, st.chunk_end) == (st.parts[0].slot, st.parts[0].begin, st.parts[0].end)
            for p in st.parts:
                s.on_prefilled(p.slot, p.end)
        if st.kind == R.Step.Kind.Decode and st.decode_slots == [0, 1]:
            break
    assert trace[0][0] == R.Step.Kind.Prefill and sorted(trace[0][1]) == [(0, 64, 96), (1, 0, 32)]
    assert trace[1][0] == R.Step.Kind.Prefill and sorted(trace[1][1]) == [(0, 96, 100), (1, 32, 50)]
    assert trace[2] == (R.Step.Kind.Decode, [], [0, 1])
    s.on_tokens(0, [7], False)
    s.on_tokens(1, [8], True)
    assert s.cancel(1)
    assert s.next().kind == R.Step.Kind.Cancel
    s.on_finished(0)
    # the finished store of request 2 (prompt 0..49 + token 8) is continued in place by a longer prompt
    s.submit(req(3, list(range(50)) + [8, 9, 10]))
    st = s.next()
    assert st.admit.kind == R.ReuseKind.ContinueStore and st.admit.slot == 1 and st.admit.reuse_tokens == 51
    s.on_admitted(st.admit)
    # a checkpoint beats a cold start; a request that can never fit is rejected (slot -1)
    s.set_checkpoint(5, list(range(500, 520)))
    s.submit(req(4, list(range(500, 540))))
    st = s.next()
    assert st.admit.kind == R.ReuseKind.Checkpoint and st.admit.source == 5 and st.admit.reuse_tokens == 20
    s.on_admitted(st.admit)
    s.submit(req(5, list(range(3000)), 100))
    st = None
    for _ in range(10):
        st = s.next()
        if st.kind == R.Step.Kind.Admit:
            break
        if st.kind == R.Step.Kind.Prefill:
            for p in st.parts:
                s.on_prefilled(p.slot, p.end)
        elif st.kind == R.Step.Kind.Decode:
            for sl in st.decode_slots:
                s.on_tokens(sl, [1], True)
    assert st.kind == R.Step.Kind.Admit and st.admit.slot == -1
    assert s.stats()["prefix_hit_tokens"] == 71


def test_oplog_replicates_and_detects_lost_leader():
    R = rt()
    name = f"/spark_oplog_test_{os.getpid()}"
    R.OpLog.unlink(name)
    leader = R.OpLog(name, True, 1)
    follower = R.OpLog(name, False, 1, 0)
    got = []

    def run():
        last = 0
        while True:
            ok, kind, payload = follower.next(last, 300)
            if not ok:
                got.append("lost")
                return
            last += 1
            got.append((kind, payload))
            if kind == 9:
                return
    t = threading.Thread(target=run)
    t.start()
    for i in range(100):
        leader.append(1, [i, i * 2])
    leader.append(9, [])
    t.join()
    assert got[-1] == (9, []) and got[5] == (1, [5, 10]) and len(got) == 101
    ok, _, _ = follower.next(leader.head(), 50)          # nothing arrives: bounded wait reports the leader as lost
    assert not ok
    for i in range(63):                                  # a follower that stopped reading: the leader notices too
        assert leader.append(1, [i], 50) > 0
    assert leader.append(1, [0], 50) == 0


def test_safetensors_roundtrip_and_memguard(tmp_path):
    from spark_engine_b200.utils.safetensors_io import load_safetensors, write_safetensors
    R = rt()
    t = {"a.weight": torch.randn(7, 5), "b.trellis": torch.randint(-30000, 30000, (3, 4, 64), dtype=torch.int16),
         "c": torch.randn(4).bfloat16()}
    p = str(tmp_path / "m.safetensors")
    write_safetensors(p, t, {"format": "pt"})
    st = R.SafeTensors(p)
    assert sorted(st.names()) == sorted(t) and st.info("b.trellis").shape == [3, 4, 64] and st.info("c").dtype == "BF16"
    back = load_safetensors(p)
    assert all(torch.equal(back[k], v) for k, v in t.items())
    fake = tmp_path / "meminfo"
    fake.write_text("MemTotal: 100 kB\nMemAvailable:     2048 kB\n")
    assert R.mem_available_bytes(str(fake)) == 2048 * 1024
    assert R.allocator_cap(1000, 500, str(fake)) == 2048 * 1024 + 500
    fired = []
    w = R.MemWatch(4 << 20, 20, lambda a: fired.append(a), str(fake))
    time.sleep(0.2)
    del w
    assert fired and fired[0] == 2048 * 1024
    assert R.sha256_hex(b"abc") == "ba7816bf8f01cfea414140de5dae2223b00361a396177a9cb410ff61f20015ad"


@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_runtime_concurrency_under_sanitizers(sanitizer, tmp_path):
    """The threaded parts of the host runtime (prefix-cache writer and evictor, op-log ring with two followers, memory
    watch thread, multi-threaded staged file load) run their stress driver under ThreadSanitizer and under
    Address/UB sanitizers: exit code 0 and no report."""
    import os
    import subprocess
    from spark_engine_b200 import build
    exe = build.build_race_stress(sanitizer)
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=1 exitcode=66", ASAN_OPTIONS="detect_leaks=1 exitcode=67",
               UBSAN_OPTIONS="halt_on_error=1 print_stacktrace=1")
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    assert "race_stress ok" in r.stdout
    assert "Sanitizer" not in r.stderr, r.stderr[-3000:]
