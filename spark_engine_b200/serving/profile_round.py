"""Two eager decode rounds of a reduced-depth model between cudaProfilerStart / cudaProfilerStop, for a launch list:

    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv --log-file launches.csv \\
        python -m spark_engine_b200.serving.profile_round --layers 4 --streams 4

(one pass per launch: nothing is saved or restored).  `--prefill 1024` profiles two prefill chunks instead.  `--summary launches.csv` prints the per-kernel table of the last
round of such a capture.  Eager on purpose: every kernel of a round is its own launch with its own duration.
"""
from __future__ import annotations

import argparse
import collections
import csv
import sys


def run(a):
    import torch
    from ..config import EngineConfig, get_model_config
    from ..models.build import build_random_model
    from .engine import LLMEngine
    cfg = get_model_config(a.model, n_layers=a.layers)
    if a.hc:
        cfg.hc_kind, cfg.hc_streams, cfg.hc_rank = a.hc, 4, 32
    W = build_random_model(cfg, "cuda", 0)
    eng = LLMEngine(cfg, W, EngineConfig(cuda_graphs=False), max_seqs=a.streams, kv_tokens_per_seq=max(4096, 2 * a.prompt))
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (a.streams, a.prompt), generator=g).tolist()
    cur = [int(torch.argmax(eng.prefill(s, prompts[s]))) for s in range(a.streams)]
    slots = list(range(a.streams))
    if a.prefill:                      # one more prefill chunk of the first prompt, profiled
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStart()
        for _ in range(2):
            eng.prefill(0, prompts[0][: a.prefill], chunk=a.prefill)
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        print("done prefill")
        return
    for _ in range(3):
        cur = eng.decode_round(slots, cur)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(2):
        cur = eng.decode_round(slots, cur)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print("done", cur)


def summary(path):
    with open(path) as f:
        lines = [ln for ln in f if not ln.startswith("==")]
    rows = [(r["Kernel Name"], float(r["Metric Value"].replace(",", "")), r.get("Grid Size"))
            for r in csv.DictReader(lines)]
    half = rows[len(rows) // 2:]
    tot = sum(t for _, t, _ in half)
    agg = collections.defaultdict(lambda: [0, 0.0])
    for n, t, g in half:
        k = n.split("(")[0][:48] + " " + str(g)
        agg[k][0] += 1
        agg[k][1] += t
    print(f"{len(half)} launches per round, {tot / 1000:.1f} us under the profiler (cold, serialised)")
    print("| share | launches | avg us | kernel (grid) |\n|---|---|---|---|")
    for k, (c, t) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:24]:
        print(f"| {100 * t / tot:.1f} % | {c} | {t / c / 1000:.1f} | {k} |")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3next-style")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--streams", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--prefill", type=int, default=0, help="profile two prefill chunks of this many tokens instead of decode rounds")
    ap.add_argument("--hc", default="", help="gated | mhc: 4 hyper-connection residual streams")
    ap.add_argument("--summary", default="")
    a = ap.parse_args()
    if a.summary:
        return summary(a.summary)
    return run(a)


if __name__ == "__main__":
    sys.exit(main() or 0)
