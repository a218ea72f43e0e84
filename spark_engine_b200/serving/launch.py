"""Launcher: `python -m spark_engine_b200.serving.launch serve --model <preset> | --checkpoint DIR [--gpus N] ...`

`serve` starts one engine process per GPU and the HTTP front end.  Rank 0 owns the Unix socket and the scheduler; with
`--gpus N > 1` the model is sharded (tensor + expert parallel) and ranks 1..N-1 replay rank 0's inputs and steps from the
shared-memory op log (`serving/replica.py`).  The launcher waits for "[serve] rank0 ready" with a liveness check of every
rank and a timeout, polls /health, and tears all ranks down when any of them exits (fail-stop).  Environment profiles are
layered: built-in defaults < each `--env-file` (KEY=VALUE lines, later files win) < the caller's environment.
`status` and `stop` act on the pid file.  Reference: engine-rs/serve/start.sh, start-glm.sh:13-33 (ready wait with
liveness + 1200 s timeout), common.sh, glm-rank.sh (env layering, one process per rank) -- without ssh: all ranks live
on one box.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

_DEFAULT_ENV = {"NCCL_NVLS_ENABLE": "0", "CUDA_DEVICE_MAX_CONNECTIONS": "8", "OMP_NUM_THREADS": "8"}


def layered_env(files, base=None) -> dict:
    """defaults < env files in order < `base` (the caller's environment)."""
    env = dict(_DEFAULT_ENV)
    for path in files or []:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line or line.startswith("#") or "=" not in line:
                    continue
                k, v = line.split("=", 1)
                env[k.strip().removeprefix("export ").strip()] = v.strip().strip('"').strip("'")
    env.update(os.environ if base is None else base)
    return env


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _engine_main(a):
    """One rank.  RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT / SPARK_OPLOG come from the launcher."""
    import torch
    from ..config import EngineConfig, get_model_config
    from ..models.build import build_random_model
    from ..models.weights import init_weights, to_device
    from .worker import EngineServer
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = a.device
    if a.checkpoint:
        from ..models.checkpoint import load_config
        cfg = load_config(a.checkpoint)
    else:
        cfg = get_model_config(a.model)
    if a.layers:
        cfg.n_layers = a.layers
        cfg.layer_types = cfg.layer_types[: a.layers]
    ecfg = EngineConfig.from_env(max_seqs=a.max_seqs, kv_tokens=a.kv_tokens, prefill_chunk=a.prefill_chunk, spec=a.spec,
                                 spec_depth=a.spec_depth, pcache_dir=a.pcache_dir, socket=a.socket, profile=a.profile,
                                 tp=world, prewarm=a.prewarm)
    tp = None
    if dev != "cpu":
        torch.cuda.set_device(local)
        dev = f"cuda:{local}"
    if world > 1:
        import torch.distributed as dist
        from datetime import timedelta
        if dev == "cpu":
            from ..parallel.tp import CpuTP
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=120))
            tp = CpuTP()
        else:
            from ..parallel import symm
            from ..parallel.tp import DeviceTP
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(dev),
                                    timeout=timedelta(seconds=120))
            tp = DeviceTP(symm.Arena(1 << 30, wait_ms=ecfg.comm_wait_ms), cfg.hidden,
                          rows_cap=max(1024, min(a.prefill_chunk, 4096)))
    if a.checkpoint:
        from ..models.checkpoint import load_checkpoint
        _, W = load_checkpoint(a.checkpoint, dev, tp=(rank, world), cfg=cfg)
    elif dev == "cpu":
        W = init_weights(cfg, seed=a.seed)
        if world > 1:
            from ..parallel.tp import shard_weights
            W = shard_weights(W, cfg, rank, world)
    elif cfg.weight_format != "dense" or cfg.hidden > 1024:
        W = build_random_model(cfg, dev, seed=a.seed, tp=(rank, world))
    else:
        W = init_weights(cfg, seed=a.seed)
        if world > 1:
            from ..parallel.tp import shard_weights
            W = shard_weights(W, cfg, rank, world)
        W = to_device(W, dev)
    oplog = os.environ.get("SPARK_OPLOG", f"/spark_b200_oplog_{os.getppid()}")
    vision = _vision_tower(a, cfg)
    if world == 1:
        EngineServer(cfg, W, ecfg, device=dev, vision=vision).serve_forever(a.socket)
        return 0
    import torch.distributed as dist
    from .replica import Follower, Leader, LeaderLost
    if rank == 0:
        leader = Leader(oplog, world - 1, ack_timeout_ms=a.ack_timeout_ms)
        dist.barrier()
        EngineServer(cfg, W, ecfg, device=dev, tp=tp, leader=leader, vision=vision).serve_forever(a.socket)
        return 0
    dist.barrier()
    srv = EngineServer(cfg, W, ecfg, device=dev, tp=tp, vision=vision)
    if ecfg.prewarm:
        srv.prewarm()                          # the leader runs the same synthetic requests before it serves
    print(f"[serve] rank{rank} ready", flush=True)
    try:
        Follower(oplog, rank - 1, world - 1, deadline_ms=a.ack_timeout_ms).run(srv)
    except LeaderLost as e:
        print(f"[serve] rank{rank}: {e}", flush=True)
        return 3
    return 0


def _wait_ready(procs, log_path, timeout):
    t0 = time.time()
    while time.time() - t0 < timeout:
        for i, p in enumerate(procs):
            if p.poll() is not None:
                raise RuntimeError(f"engine rank {i} exited with {p.returncode} before the server was ready; see {log_path}")
        try:
            if "[serve] rank0 ready" in open(log_path).read():
                return
        except OSError:
            pass
        time.sleep(0.2)
    raise TimeoutError("engine did not become ready in time")


def spawn_ranks(a, env):
    """One engine process per rank; returns (processes, rank-0 log path)."""
    n = max(1, a.gpus)
    port, oplog = _free_port(), f"/spark_b200_oplog_{os.getpid()}"
    procs = []
    for r in range(n):
        e = dict(env)
        e.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(n), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                 SPARK_OPLOG=oplog)
        log = os.path.join(a.log_dir, f"spark-b200-rank{r}.log")
        procs.append(subprocess.Popen([sys.executable, "-m", "spark_engine_b200.serving.launch", "engine"] + a.passthrough,
                                      stdout=open(log, "w"), stderr=subprocess.STDOUT, env=e))
    return procs, os.path.join(a.log_dir, "spark-b200-rank0.log")


def _vision_config(a, hidden: int):
    """The vision tower the `--vision` flag names: "tiny" (tests) or "vit-l" (24 x 1024, patch 14), aligned to `hidden`."""
    from ..multimodal.vision import VisionConfig
    if not a.vision:
        return None
    if a.vision == "tiny":
        return VisionConfig(depth=2, width=64, heads=4, mlp=128, patch=4, merge=2, out_hidden=hidden, max_side=64)
    if a.vision == "vit-l":
        return VisionConfig(out_hidden=hidden)
    raise SystemExit(f"unknown --vision {a.vision!r} (tiny | vit-l)")


def _vision_tower(a, cfg):
    """(config, weights) of the vision tower: from `<checkpoint>/vision.safetensors` when the checkpoint has one, else
    random weights of the named architecture (every rank draws the same seed, so all ranks encode identical rows)."""
    vc = _vision_config(a, cfg.hidden)
    if vc is None:
        return None
    from ..multimodal.vision import init_vision_weights
    path = os.path.join(a.checkpoint, "vision.safetensors") if a.checkpoint else ""
    if path and os.path.exists(path):
        from ..utils.safetensors_io import load_safetensors
        return vc, load_safetensors(path)
    return vc, init_vision_weights(vc, seed=a.seed)


def cmd_serve(a):
    env = layered_env(a.env_file)
    procs, log = spawn_ranks(a, env)
    front = None
    try:
        _wait_ready(procs, log, a.ready_timeout)
        front_cmd = [sys.executable, "-m", "spark_engine_b200.serving.openai_server", "--socket", a.socket,
                     "--host", a.host, "--port", str(a.port), "--model-name", a.checkpoint or a.model]
        if a.vision:
            vc = _vision_config(a, 1)
            front_cmd += ["--media-canvas", str(a.canvas), "--media-rows", str(vc.rows_for(a.canvas, a.canvas))]
            if a.allow_media_fetch:
                front_cmd.append("--allow-media-fetch")
        front = subprocess.Popen(front_cmd, env=env)
        with open(a.pidfile, "w") as f:
            json.dump({**{f"engine{i}": p.pid for i, p in enumerate(procs)}, "front": front.pid}, f)
        for _ in range(100):
            try:
                if urllib.request.urlopen(f"http://{a.host}:{a.port}/health", timeout=1).status == 200:
                    break
            except Exception:
                time.sleep(0.2)
        print(f"serving {a.checkpoint or a.model} on http://{a.host}:{a.port} with {len(procs)} rank(s)", flush=True)
        while front.poll() is None and all(p.poll() is None for p in procs):   # any rank gone = the whole server stops
            time.sleep(0.5)
        return 0 if front.poll() is not None else 1
    finally:
        for p in procs + ([front] if front else []):
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)          # exact children only


def cmd_status(a):
    try:
        pids = json.load(open(a.pidfile))
    except OSError:
        print("not running")
        return 1
    alive = {k: os.path.exists(f"/proc/{v}") for k, v in pids.items()}
    print(json.dumps({"pids": pids, "alive": alive}))
    return 0 if all(alive.values()) else 1


def cmd_stop(a):
    try:
        pids = json.load(open(a.pidfile))
    except OSError:
        return 0
    for v in pids.values():
        try:
            os.kill(int(v), signal.SIGTERM)       # exact pids from the pid file only
        except ProcessLookupError:
            pass
    os.unlink(a.pidfile)
    return 0


def main():
    ap = argparse.ArgumentParser(prog="spark-b200")
    ap.add_argument("cmd", choices=["serve", "engine", "status", "stop"])
    ap.add_argument("--model", default="tiny-hybrid")
    ap.add_argument("--checkpoint", default=None, help="directory written by models.checkpoint.save_checkpoint")
    ap.add_argument("--gpus", type=int, default=1, help="ranks of one box; the model is sharded over them")
    ap.add_argument("--env-file", action="append", default=[], help="KEY=VALUE profile; repeatable, later files win")
    ap.add_argument("--log-dir", default="/tmp")
    ap.add_argument("--ack-timeout-ms", type=int, default=30000, help="op-log deadline between leader and followers")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--socket", default="/tmp/spark-b200.sock")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--max-seqs", type=int, default=4)
    ap.add_argument("--kv-tokens", type=int, default=1 << 16)
    ap.add_argument("--prefill-chunk", type=int, default=4096)
    ap.add_argument("--spec", default="mtp")
    ap.add_argument("--spec-depth", type=int, default=3)
    ap.add_argument("--pcache-dir", default=None)
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--pidfile", default="/tmp/spark-b200.pid")
    ap.add_argument("--prewarm", action="store_true", help="capture the graphs of 1..max-seqs streams before serving")
    ap.add_argument("--vision", default="", help="tiny | vit-l: serve image / video parts of chat requests through a vision tower")
    ap.add_argument("--canvas", type=int, default=448, help="side of the square canvas every frame is fitted onto (pixels)")
    ap.add_argument("--allow-media-fetch", action="store_true", help="let the front end download http(s) media URLs")
    ap.add_argument("--ready-timeout", type=float, default=1200.0)
    a = ap.parse_args()
    a.passthrough = [x for x in sys.argv[2:]]
    return {"serve": cmd_serve, "engine": _engine_main, "status": cmd_status, "stop": cmd_stop}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main() or 0)
