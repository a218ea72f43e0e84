"""End-to-end serving on CPU: engine loop over a Unix socket + OpenAI-compatible HTTP front end, tiny hybrid MoE.
Checks that served tokens equal plain greedy decoding, streaming, prefix reuse, cancellation, stats and metrics."""
import json
import os
import socket
import threading
import time
import urllib.request

import torch

from spark_engine_b200.config import EngineConfig, tiny_hybrid
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.oracle import model as oracle
from spark_engine_b200.serving import protocol as proto
from spark_engine_b200.serving.openai_server import ReasoningSplit, StopStrings, parse_tool_calls, serve
from spark_engine_b200.serving.worker import EngineServer


def _start(tmp_path, spec="mtp", pcache=None, tree="", prewarm=False):
    cfg = tiny_hybrid()
    cfg.mtp_layers = 1
    W = init_weights(cfg, seed=0)
    sock = str(tmp_path / "e.sock")
    es = EngineServer(cfg, W, EngineConfig(max_seqs=2, kv_tokens=2048, prefill_chunk=32, spec=spec, spec_depth=2,
                                           spec_tree_widths=tree, pcache_dir=pcache, pcache_bytes=64 << 20, profile=True,
                                           prewarm=prewarm))
    ready = threading.Event()
    th = threading.Thread(target=es.serve_forever, args=(sock,), kwargs={"ready_cb": ready.set}, daemon=True)
    th.start()
    assert ready.wait(30)
    return cfg, W, es, sock, th


def _client(sock):
    c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    c.connect(sock)
    return c, proto.LineBuffer()


def _collect(c, buf, want_ids, timeout=120):
    done, deltas = {}, {}
    t0 = time.time()
    while len(done) < len(want_ids) and time.time() - t0 < timeout:
        for m in buf.feed(c.recv(1 << 16)):
            if "delta" in m:
                deltas.setdefault(m["id"], []).extend(m["delta"])
            if m.get("done") or "error" in m:
                done[m["id"]] = m
    return done, deltas


def test_socket_protocol_matches_greedy_and_reuses_prefix(tmp_path):
    cfg, W, es, sock, th = _start(tmp_path)
    g = torch.Generator().manual_seed(1)
    p1 = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    p2 = torch.randint(0, cfg.vocab, (25,), generator=g).tolist()
    ref1 = oracle.greedy_generate(cfg, W, torch.tensor(p1), 10)[0].tolist()
    ref2 = oracle.greedy_generate(cfg, W, torch.tensor(p2), 6)[0].tolist()
    c, buf = _client(sock)
    c.sendall(proto.encode({"id": 1, "prompt_ids": p1, "max_new": 10}) + proto.encode({"id": 2, "prompt_ids": p2, "max_new": 6}))
    done, deltas = _collect(c, buf, [1, 2])
    assert done[1]["token_ids"] == ref1 == deltas[1] and done[2]["token_ids"] == ref2
    assert done[1]["finish_reason"] == "length" and done[1]["rounds"] >= 1 and done[1]["prefill_ms"] > 0
    assert es.totals["prefill_shared_steps"] > 0        # the two prompts shared prefill forwards (one segment each)
    # follow-up turn: the finished store is continued, only the new tokens are prefilled
    p3 = p1 + ref1 + [5, 6, 7]
    ref3 = oracle.greedy_generate(cfg, W, torch.tensor(p3), 4)[0].tolist()
    c.sendall(proto.encode({"id": 3, "prompt_ids": p3, "max_new": 4}))
    done, _ = _collect(c, buf, [3])
    assert done[3]["token_ids"] == ref3 and done[3]["prefix_hit_tokens"] >= len(p1)
    # bad request, stats, cancellation
    c.sendall(proto.encode({"id": 4, "prompt_ids": [], "max_new": 4}) + proto.encode({"id": 5, "stats": True}))
    got = []
    while len(got) < 2:
        got += buf.feed(c.recv(1 << 16))
    assert any("error" in m for m in got) and any("stats" in m and m["stats"]["requests"] == 3 for m in got)
    c.sendall(proto.encode({"id": 6, "prompt_ids": p1, "max_new": 400}))
    time.sleep(0.3)
    c.sendall(proto.encode({"cancel": 6}))
    done, _ = _collect(c, buf, [6])
    assert done[6]["finish_reason"] == "cancelled" and len(done[6]["token_ids"]) < 400
    c.sendall(proto.encode({"shutdown": True}))
    th.join(10)


def test_http_front_end_streaming_and_metrics(tmp_path):
    cfg, W, es, sock, th = _start(tmp_path, spec="none")
    srv, app = serve(sock, "127.0.0.1", 0, "tiny")
    port = srv.server_address[1]
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{port}"
    assert json.load(urllib.request.urlopen(base + "/health"))["status"] == "ok"
    assert json.load(urllib.request.urlopen(base + "/v1/models"))["data"][0]["id"] == "tiny"

    def post(path, body):
        req = urllib.request.Request(base + path, json.dumps(body).encode(), {"Content-Type": "application/json"})
        return urllib.request.urlopen(req, timeout=120)
    ids = json.load(post("/tokenize", {"prompt": "hello"}))["tokens"]
    assert json.load(post("/detokenize", {"tokens": ids}))["prompt"] == "hello"
    r = json.load(post("/v1/completions", {"prompt": "abc", "max_tokens": 5}))
    assert r["usage"]["completion_tokens"] == 5 and r["choices"][0]["finish_reason"] == "length"
    want = oracle.greedy_generate(cfg, W, torch.tensor(list(b"abc")), 5)[0].tolist()
    assert r["choices"][0]["text"] == app.tok.decode(want)
    resp = post("/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "stream": True,
                                         "stream_options": {"include_usage": True}})
    events = [ln[6:] for ln in resp.read().decode().split("\n") if ln.startswith("data: ")]
    assert events[-1] == "[DONE]"
    final = json.loads(events[-2])
    assert final["usage"]["completion_tokens"] == 6 and final["choices"][0]["finish_reason"] == "length"
    text = urllib.request.urlopen(base + "/metrics").read().decode()
    assert "vllm:generation_tokens_total" in text and 'vllm:request_success_total{finished_reason="length"' in text
    srv.shutdown()
    es.shutdown = True
    th.join(10)


def test_disk_prefix_cache_restores_across_engine_restarts(tmp_path):
    pdir = str(tmp_path / "pc")
    cfg, W, es, sock, th = _start(tmp_path, pcache=pdir)
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (256,), generator=g).tolist()       # a whole granule
    c, buf = _client(sock)
    c.sendall(proto.encode({"id": 1, "prompt_ids": prompt + [3], "max_new": 3}) if False else proto.encode({"id": 1, "prompt_ids": prompt, "max_new": 3}))
    d1, _ = _collect(c, buf, [1])
    c.sendall(proto.encode({"shutdown": True}))
    th.join(10)
    cfg, W, es2, sock2, th2 = _start(tmp_path / "..", pcache=pdir) if False else _start(tmp_path, pcache=pdir)
    c2, buf2 = _client(sock2)
    c2.sendall(proto.encode({"id": 7, "prompt_ids": prompt + [9, 8], "max_new": 3}))
    d2, _ = _collect(c2, buf2, [7])
    ref = oracle.greedy_generate(cfg, W, torch.tensor(prompt + [9, 8]), 3)[0].tolist()
    assert d2[7]["token_ids"] == ref and d2[7]["prefix_hit_tokens"] == 256
    assert es2.stats()["disk_restores"] == 1
    c2.sendall(proto.encode({"shutdown": True}))
    th2.join(10)


def test_front_end_text_helpers():
    ss = StopStrings(["END"])
    out = "".join(ss.feed(x)[0] for x in ["ab", "cE", "N", "x"]) + ss.flush()
    assert out == "abcENx"
    ss = StopStrings(["END"])
    a, hit = ss.feed("abcEN")
    b, hit2 = ss.feed("Dzz")
    assert (a + b, hit2) == ("abc", True)
    rs = ReasoningSplit()
    r1, c1 = rs.feed("<thi")
    r2, c2 = rs.feed("nk>plan</think>answer")
    assert r1 + r2 == "plan" and c1 + c2 == "answer"
    txt, calls = parse_tool_calls('ok <tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>')
    assert txt == "ok" and calls[0]["function"]["name"] == "f" and json.loads(calls[0]["function"]["arguments"]) == {"x": 1}


def test_http_bench_script_against_a_live_front_end(tmp_path):
    from spark_engine_b200.serving import bench_http
    cfg, W, es, sock, th = _start(tmp_path, spec="none")
    srv, app = serve(sock, "127.0.0.1", 0, "tiny")
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{srv.server_address[1]}"
    res = bench_http.main(["--url", url, "--streams", "1", "2", "--max-tokens", "6", "--prefill", "40"])
    assert [d["streams"] for d in res["decode"]] == [1, 2]
    assert res["decode"][1]["tokens"] == 12 and res["decode"][0]["aggregate_decode_tok_s"] > 0
    assert res["prefill"][0]["prompt_tokens"] >= 30 and res["prefill"][0]["prefill_tok_s"] > 0
    srv.shutdown()
    es.shutdown = True
    th.join(10)


import pytest


@pytest.mark.parametrize("spec", ["feature", "stage", "lookup", "feature-tree"])
def test_server_with_the_other_drafters_still_serves_greedy_text(tmp_path, spec):
    """The tap-conditioned and the staged drafter (randomly initialised here) and prompt lookup as the server's drafter:
    whatever they propose, verification keeps the served text equal to plain greedy decoding."""
    cfg, W, es, sock, th = _start(tmp_path, spec=spec.split("-")[0], tree="3,2" if spec.endswith("tree") else "")
    g = torch.Generator().manual_seed(2)
    p1 = torch.randint(0, cfg.vocab, (30,), generator=g).tolist()
    ref = oracle.greedy_generate(cfg, W, torch.tensor(p1), 8)[0].tolist()
    c, buf = _client(sock)
    c.sendall(proto.encode({"id": 1, "prompt_ids": p1, "max_new": 8}))
    done, _ = _collect(c, buf, [1])
    assert done[1]["token_ids"] == ref
    assert done[1]["drafted_tokens"] >= 0
    c.sendall(proto.encode({"shutdown": True}))
    th.join(10)


def test_prewarmed_server_serves_the_same_tokens_and_starts_with_clean_counters(tmp_path):
    """Prewarm runs synthetic requests for 1..max_seqs streams before the socket opens: afterwards the counters are
    those of a fresh server, nothing was written to the prefix cache, and real requests get plain greedy text."""
    cfg, W, es, sock, th = _start(tmp_path, prewarm=True, pcache=str(tmp_path / "pc"))
    assert es.totals["requests"] == 0 and es.totals["prompt_tokens"] == 0 and es.totals["prefill_steps"] == 0
    assert es.disk is not None and es.disk.stats().get("saves", 0) == 0
    assert not es.sched.has_work() and es.out == []
    g = torch.Generator().manual_seed(3)
    p1 = torch.randint(0, cfg.vocab, (33,), generator=g).tolist()
    p2 = torch.randint(0, cfg.vocab, (21,), generator=g).tolist()
    ref1 = oracle.greedy_generate(cfg, W, torch.tensor(p1), 8)[0].tolist()
    ref2 = oracle.greedy_generate(cfg, W, torch.tensor(p2), 5)[0].tolist()
    c, buf = _client(sock)
    c.sendall(proto.encode({"id": 1, "prompt_ids": p1, "max_new": 8}) + proto.encode({"id": 2, "prompt_ids": p2, "max_new": 5}))
    done, _ = _collect(c, buf, [1, 2])
    assert done[1]["token_ids"] == ref1 and done[2]["token_ids"] == ref2
    assert es.totals["requests"] == 2
    c.sendall(proto.encode({"shutdown": True}))
    th.join(10)


def test_serve_log_lines_and_round_trace(tmp_path, capfd):
    """EngineConfig.serve_log prints one line per admission, prefill forward and round; draft_trace appends one JSON line
    per speculative round whose accepted / emitted counts add up to the served tokens."""
    import json as js
    from spark_engine_b200.serving.worker import EngineServer as ES
    cfg = tiny_hybrid()
    cfg.mtp_layers = 1
    W = init_weights(cfg, seed=0)
    trace = tmp_path / "trace.jsonl"
    es = ES(cfg, W, EngineConfig(max_seqs=2, kv_tokens=2048, prefill_chunk=32, spec="mtp", spec_depth=2, serve_log=True,
                                 draft_trace=str(trace)))
    g = torch.Generator().manual_seed(2)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    es.submit({"id": 7, "prompt_ids": prompt, "max_new": 9})
    for _ in range(200):
        if not es.step():
            break
    done = [m for m in es.out if m.get("done")]
    assert done and len(done[0]["token_ids"]) == 9
    err = capfd.readouterr().err
    assert "[serve-admit] id=7 slot=0 kind=Cold reuse=0 prompt=40" in err
    assert "[serve-prefill] parts=[(0, 0, 32)] rows=32" in err and "[serve-round] streams=1" in err
    recs = [js.loads(l) for l in trace.read_text().splitlines()]
    assert recs and all(r["seqs"][0]["id"] == 7 for r in recs)
    assert sum(len(r["seqs"][0]["emitted"]) for r in recs) >= 8               # the first token comes from the prefill
    assert sum(r["seqs"][0]["accepted"] for r in recs) == done[0]["accepted_drafts"]
    assert [r["round"] for r in recs] == list(range(1, len(recs) + 1))
