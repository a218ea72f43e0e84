"""HTTP-level decode / prefill benchmark against a running front end (the measurement the reference publishes:
aggregate tokens/s over 1-4 concurrent streams, time to first token, prefill tokens/s; bench/decode_bench.py,
bench/prefill_bench.py of the reference).

    python -m spark_engine_b200.serving.bench_http --url http://127.0.0.1:8000 --streams 1 2 3 4 --max-tokens 128
    python -m spark_engine_b200.serving.bench_http --url ... --prefill 4096 16384

Every stream is one streaming /v1/completions request; TTFT = first content event, decode rate = completion tokens
after the first one over the time after the first one, aggregate = sum over the concurrent streams.
"""
from __future__ import annotations

import argparse
import json
import statistics
import threading
import time
import urllib.request

PROSE = ("The quick brown fox jumps over the lazy dog while the engine streams tokens to every client that asked for "
         "them, one by one, and keeps a little cache of what it has already seen. ")
STRUCTURED = '{"items": [{"id": 1, "name": "alpha", "tags": ["x", "y"]}, {"id": 2, "name": "beta", "tags": []}], "next": '


def _stream_once(url: str, prompt: str, max_tokens: int, out: dict, temperature: float = 0.0):
    body = {"prompt": prompt, "max_tokens": max_tokens, "stream": True, "temperature": temperature,
            "stream_options": {"include_usage": True}}
    req = urllib.request.Request(url + "/v1/completions", json.dumps(body).encode(), {"Content-Type": "application/json"})
    t0 = time.perf_counter()
    first = None
    n = 0
    usage = None
    with urllib.request.urlopen(req, timeout=3600) as resp:
        for raw in resp:
            line = raw.decode().strip()
            if not line.startswith("data: ") or line == "data: [DONE]":
                continue
            ev = json.loads(line[6:])
            if ev.get("usage"):
                usage = ev["usage"]
            ch = ev.get("choices") or []
            if ch and ch[0].get("text"):
                n += 1
                if first is None:
                    first = time.perf_counter()
    t1 = time.perf_counter()
    tokens = usage["completion_tokens"] if usage else n
    out.update(ttft=(first or t1) - t0, total=t1 - t0, tokens=tokens,
               decode_tok_s=(tokens - 1) / max(t1 - (first or t1), 1e-9) if tokens > 1 else 0.0,
               prompt_tokens=usage["prompt_tokens"] if usage else None)


def run_streams(url: str, n_streams: int, prompt: str, max_tokens: int, temperature: float = 0.0) -> dict:
    outs = [dict() for _ in range(n_streams)]
    ths = [threading.Thread(target=_stream_once, args=(url, prompt + f" [{i}]", max_tokens, outs[i], temperature))
           for i in range(n_streams)]
    t0 = time.perf_counter()
    for t in ths:
        t.start()
    for t in ths:
        t.join()
    wall = time.perf_counter() - t0
    return {"streams": n_streams, "aggregate_decode_tok_s": round(sum(o["decode_tok_s"] for o in outs), 2),
            "ttft_ms_median": round(statistics.median(o["ttft"] for o in outs) * 1e3, 1),
            "tokens": sum(o["tokens"] for o in outs), "wall_s": round(wall, 3)}


def run_prefill(url: str, n_tokens: int) -> dict:
    words = (PROSE * (n_tokens // 20 + 1))
    ids = json.load(urllib.request.urlopen(urllib.request.Request(
        url + "/tokenize", json.dumps({"prompt": words}).encode(), {"Content-Type": "application/json"})))["tokens"][:n_tokens]
    prompt = json.load(urllib.request.urlopen(urllib.request.Request(
        url + "/detokenize", json.dumps({"tokens": ids}).encode(), {"Content-Type": "application/json"})))["prompt"]
    out = {}
    _stream_once(url, prompt, 1, out)
    n = out["prompt_tokens"] or len(ids)
    return {"prompt_tokens": n, "ttft_s": round(out["ttft"], 3), "prefill_tok_s": round(n / out["ttft"], 1)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--streams", type=int, nargs="*", default=[1, 2, 3, 4])
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--kind", default="prose", choices=["prose", "structured"])
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--prefill", type=int, nargs="*", default=[])
    a = ap.parse_args(argv)
    prompt = PROSE if a.kind == "prose" else STRUCTURED
    res = {"decode": [run_streams(a.url, s, prompt, a.max_tokens, a.temperature) for s in a.streams],
           "prefill": [run_prefill(a.url, n) for n in a.prefill]}
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
