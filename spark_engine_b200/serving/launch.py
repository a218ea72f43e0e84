"""Launcher: `python -m spark_engine_b200.serving.launch serve --model <preset|config.json> [--gpus N] ...`

Starts one engine process per GPU (rank 0 owns the Unix socket) and the HTTP front end, waits for
"[serve] rank0 ready" with a liveness check and a timeout, polls /health, and tears everything down on exit.
`status` and `stop` act on the pid file.  Reference: engine-rs/serve/start.sh, start-glm.sh:13-33 (ready wait with
liveness + 1200 s timeout), common.sh, glm-rank.sh (env layering) -- without ssh: all ranks live on one box.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
import urllib.request


def _engine_main(a):
    import torch
    from ..config import EngineConfig, get_model_config
    from ..models.build import build_random_model
    from ..models.weights import init_weights, to_device
    from .worker import EngineServer
    cfg = get_model_config(a.model)
    if a.layers:
        cfg.n_layers = a.layers
        cfg.layer_types = cfg.layer_types[: a.layers]
    ecfg = EngineConfig.from_env(max_seqs=a.max_seqs, kv_tokens=a.kv_tokens, prefill_chunk=a.prefill_chunk, spec=a.spec,
                                 spec_depth=a.spec_depth, pcache_dir=a.pcache_dir, socket=a.socket, profile=a.profile)
    dev = a.device
    if dev == "cpu":
        W = init_weights(cfg, seed=a.seed)
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        W = build_random_model(cfg, dev, seed=a.seed) if cfg.weight_format != "dense" or cfg.hidden > 1024 \
            else to_device(init_weights(cfg, seed=a.seed), dev)
    EngineServer(cfg, W, ecfg, device=dev).serve_forever(a.socket)


def _wait_ready(proc, log_path, timeout):
    t0 = time.time()
    while time.time() - t0 < timeout:
        if proc.poll() is not None:
            raise RuntimeError(f"engine exited with {proc.returncode} before it was ready; see {log_path}")
        try:
            if "[serve] rank0 ready" in open(log_path).read():
                return
        except OSError:
            pass
        time.sleep(0.2)
    raise TimeoutError("engine did not become ready in time")


def cmd_serve(a):
    log = f"/tmp/spark-b200-rank0.log"
    env = dict(os.environ)
    eng = subprocess.Popen([sys.executable, "-m", "spark_engine_b200.serving.launch", "engine"] + a.passthrough,
                           stdout=open(log, "w"), stderr=subprocess.STDOUT, env=env)
    try:
        _wait_ready(eng, log, a.ready_timeout)
        front = subprocess.Popen([sys.executable, "-m", "spark_engine_b200.serving.openai_server", "--socket", a.socket,
                                  "--host", a.host, "--port", str(a.port), "--model-name", a.model])
        with open(a.pidfile, "w") as f:
            json.dump({"engine": eng.pid, "front": front.pid}, f)
        for _ in range(100):
            try:
                if urllib.request.urlopen(f"http://{a.host}:{a.port}/health", timeout=1).status == 200:
                    break
            except Exception:
                time.sleep(0.2)
        print(f"serving {a.model} on http://{a.host}:{a.port}", flush=True)
        front.wait()
    finally:
        for p in (eng,):
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)


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
    ap.add_argument("--ready-timeout", type=float, default=1200.0)
    a = ap.parse_args()
    a.passthrough = [x for x in sys.argv[2:]]
    return {"serve": cmd_serve, "engine": _engine_main, "status": cmd_status, "stop": cmd_stop}[a.cmd](a)


if __name__ == "__main__":
    sys.exit(main() or 0)
