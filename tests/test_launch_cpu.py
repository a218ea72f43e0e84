"""The launcher end to end on CPU: a checkpoint is written, `serve`'s rank spawner starts two gloo ranks that load their
shards of it, rank 0 answers on the Unix socket while rank 1 replays its steps, and the served tokens equal the unsharded
greedy decode.  Also: layered environment profiles, and the host-memory guard refusing requests against a fake meminfo."""
import argparse
import os
import signal
import socket
import time

import torch

from spark_engine_b200.config import EngineConfig, tiny_hybrid
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.oracle import model as oracle
from spark_engine_b200.serving import launch, protocol as proto


def test_layered_env(tmp_path):
    a, b = tmp_path / "common.env", tmp_path / "rank.env"
    a.write_text("# profile\nFOO=1\nexport BAR='x y'\nNCCL_NVLS_ENABLE=1\n")
    b.write_text("FOO=2\n")
    env = launch.layered_env([str(a), str(b)], base={"BAZ": "3", "BAR": "caller"})
    assert env["FOO"] == "2" and env["BAR"] == "caller" and env["BAZ"] == "3" and env["NCCL_NVLS_ENABLE"] == "1"
    assert launch.layered_env([], base={})["NCCL_NVLS_ENABLE"] == "0"


def test_two_rank_server_from_a_checkpoint(tmp_path):
    from spark_engine_b200.models.checkpoint import save_checkpoint
    cfg = tiny_hybrid()
    cfg.mtp_layers = 0
    W = init_weights(cfg, seed=0)
    ck = str(tmp_path / "ck")
    save_checkpoint(W, cfg, ck)
    sock = str(tmp_path / "e.sock")
    args = ["--checkpoint", ck, "--gpus", "2", "--device", "cpu", "--socket", sock, "--spec", "none", "--max-seqs", "2",
            "--kv-tokens", "2048", "--prefill-chunk", "32", "--ack-timeout-ms", "20000"]
    a = argparse.Namespace(gpus=2, log_dir=str(tmp_path), passthrough=args)
    procs, log = launch.spawn_ranks(a, launch.layered_env([]))
    try:
        launch._wait_ready(procs, log, 120)
        g = torch.Generator().manual_seed(1)
        p1 = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
        ref = oracle.greedy_generate(cfg, W, torch.tensor(p1), 8)[0].tolist()
        c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        c.connect(sock)
        buf = proto.LineBuffer()
        c.sendall(proto.encode({"id": 1, "prompt_ids": p1, "max_new": 8}))
        done, t0 = None, time.time()
        while done is None and time.time() - t0 < 120:
            for m in buf.feed(c.recv(1 << 16)):
                if m.get("done") or "error" in m:
                    done = m
        assert done is not None and done.get("token_ids") == ref, (done, open(log).read()[-2000:])
        c.sendall(proto.encode({"shutdown": True}))
        for p in procs:
            p.wait(60)
        assert [p.returncode for p in procs] == [0, 0], open(os.path.join(str(tmp_path), "spark-b200-rank1.log")).read()[-2000:]
    finally:
        for p in procs:
            if p.poll() is None:
                p.send_signal(signal.SIGTERM)


def test_memory_guard_refuses_requests_while_host_memory_is_low(tmp_path):
    from spark_engine_b200.serving.worker import EngineServer
    fake = tmp_path / "meminfo"
    fake.write_text("MemTotal: 100 kB\nMemAvailable:  900000 kB\n")
    cfg = tiny_hybrid()
    cfg.mtp_layers = 0
    es = EngineServer(cfg, init_weights(cfg, seed=0),
                      EngineConfig(max_seqs=2, kv_tokens=1024, prefill_chunk=32, spec="none", host_mem_floor_gb=0.5,
                                   meminfo_path=str(fake)))
    es.submit({"id": 1, "prompt_ids": [1, 2, 3], "max_new": 2})
    assert es.out[-1].get("queued")
    fake.write_text("MemTotal: 100 kB\nMemAvailable:  1000 kB\n")
    t0 = time.time()
    while es.memwatch.fired() == 0 and time.time() - t0 < 10:
        time.sleep(0.05)
    es.submit({"id": 2, "prompt_ids": [1, 2, 3], "max_new": 2})
    assert "host memory" in es.out[-1].get("error", "") and es.stats()["host_mem_low_events"] == 1
    fake.write_text("MemTotal: 100 kB\nMemAvailable:  900000 kB\n")
    time.sleep(0.6)
    es.mem_low_until = 0.0                               # the refusal window has passed
    es.submit({"id": 3, "prompt_ids": [1, 2, 3], "max_new": 2})
    assert es.out[-1].get("queued")
    del es.memwatch


def test_package_cli_dispatch_and_precision_flags():
    """`python -m spark_engine_b200 <command>`: version, presets, an unknown command, a launcher command; library GEMMs are
    set to fp32 accumulation without reduced-precision reductions."""
    import json
    import subprocess
    import sys
    import torch
    from spark_engine_b200.utils import precision
    run = lambda *a: subprocess.run([sys.executable, "-m", "spark_engine_b200", *a], capture_output=True, text=True, timeout=120)
    assert run("version").stdout.strip()
    cfgs = json.loads(run("configs").stdout)
    assert {"qwen3next-style", "glm-style", "ds4-style"} <= set(cfgs) and cfgs["qwen3next-style"]["n_layers"] == 48
    assert run("nope").returncode == 2
    assert "not running" in run("status", "--pidfile", "/tmp/spark-b200-no-such.pid").stdout
    flags = precision.set_fp32_accum(tf32=False)
    assert flags == {"bf16_reduced_precision_reduction": False, "fp16_reduced_precision_reduction": False, "tf32": False}
    assert torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction is False
    assert torch.backends.cuda.matmul.allow_tf32 is False
    assert precision.set_fp32_accum(tf32=True)["tf32"] and torch.backends.cuda.matmul.allow_tf32 is True
    precision.set_fp32_accum(tf32=False)
