"""Multi-rank serving on CPU (gloo): followers replay the leader's inputs and steps from the shared-memory op log and
end up with the same tokens; a follower that stops between steps is noticed on the host before the next step runs."""
import os
import socket
import time

import pytest
import torch


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, name, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from datetime import timedelta
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=30))
    from spark_engine_b200.config import EngineConfig, tiny_hybrid
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.parallel.tp import CpuTP, shard_weights
    from spark_engine_b200.serving.replica import Follower, FollowerLost, Leader
    from spark_engine_b200.serving.worker import EngineServer
    cfg = tiny_hybrid()
    cfg.mtp_layers = 0
    W = shard_weights(init_weights(cfg, seed=0), cfg, rank, world)
    ecfg = EngineConfig(max_seqs=2, kv_tokens=1024, prefill_chunk=16, spec="none")
    leader = Leader(name, world - 1, ack_timeout_ms=1500) if rank == 0 else None
    dist.barrier()
    srv = EngineServer(cfg, W, ecfg, device="cpu", tp=CpuTP(), leader=leader)
    g = torch.Generator().manual_seed(1)
    reqs = [{"id": i, "prompt_ids": torch.randint(0, cfg.vocab, (20 + 7 * i,), generator=g).tolist(), "max_new": 6,
             "temperature": 0.0 if i == 0 else 0.8, "seed": 5} for i in range(2)]
    if rank == 0:
        done = {}
        try:
            for r in reqs:
                srv.submit(r)
            steps = 0
            while len(done) < len(reqs) and steps < 400:
                srv.step()
                steps += 1
                for m in srv.out:
                    if m.get("done"):
                        done[m["id"]] = m["token_ids"]
                srv.out = []
            leader.shutdown()
            q.put(("leader", done))
        except FollowerLost as e:
            q.put(("leader_lost_follower", str(e)))
    else:
        f = Follower(name, rank - 1, world - 1, deadline_ms=5000)
        if mode == "follower_stops":
            f.run(srv, max_ops=7)                        # leaves between steps, nothing in flight
            q.put(("follower_left", f.seq))
        else:
            f.run(srv)
            q.put(("follower", f.finished, srv.totals["generation_tokens"]))
    if mode != "follower_stops":
        dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["replay", "follower_stops"])
def test_followers_replay_the_leader(mode):
    import torch.multiprocessing as mp
    world = 2
    name = f"/spark_b200_test_oplog_{os.getpid()}_{mode}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, PORT, name, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = []
    deadline = time.time() + 120
    while len(got) < world and time.time() < deadline:
        try:
            got.append(q.get(timeout=1.0))
        except Exception:
            if all(not p.is_alive() for p in procs):
                break
    for p in procs:
        p.join(20)
        if p.is_alive():
            p.terminate()
    kinds = {g[0]: g for g in got}
    if mode == "replay":
        assert "leader" in kinds and "follower" in kinds, got
        done = kinds["leader"][1]
        assert sorted(done) == [0, 1] and all(len(v) == 6 for v in done.values())
        assert kinds["follower"][1] == done            # the follower produced the same tokens, greedy and sampled
        assert kinds["follower"][2] == 12
    else:
        assert "follower_left" in kinds and "leader_lost_follower" in kinds, got
        assert "did not pick up step" in kinds["leader_lost_follower"][1]


PORT = _free_port()
