#!/usr/bin/env python
"""Headline benchmark: aggregate decode tokens/s at 4 concurrent streams (plus 1-3 streams, prefill
tokens/s and TTFT) of the Qwen3-Next-style hybrid MoE (48 layers, hidden 2048, 512 experts top-10,
vocab 151936) with random-init EXL3 4 bpw weights and synthetic uniform-random prompts.

  python bench.py --gpus N --steps K --warmup W
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

A step is one decode round: every live stream emits one token (greedy).  Two numbers are measured:

  value  device-timed (CUDA events): K consecutive decode steps of the captured round with the sampled ids
         fed back on the device (`LLMEngine.decode_steps`): every step is a real decode step (new token ids,
         positions and KV rows advance), only the host round trip between steps is left out;
  e2e    wall clock through the public per-step API (`LLMEngine.decode_round`): every step copies its token
         ids and positions from pinned host memory to the device and reads the sampled ids back.

With N > 1 the default is ONE model sharded over the N GPUs (tensor + expert parallel, `--parallel tp`, strong
scaling); `--parallel dp` runs one replica per GPU (weak scaling, no collective).  Rank 0 prints ONE JSON line.
`--impl aten` runs the same model code through PyTorch/ATen ops instead of the kernels (a library baseline,
reported as such); `--impl reference` reports why the reference itself cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

# published aggregate decode tok/s at 4 streams (prose, greedy) of the reference, per model family:
# Qwen3.8-Flash-Next on 1x DGX Spark GB10; GLM-5.3-Flash on 2x GB10 (TP2); DeepSeek-V4.1-Flash on 3x GB10 (TP3)
BASELINE_DECODE_4STREAMS = {"qwen3next-style": 139.2, "glm-style": 82.9, "ds4-style": 124.7}
DEFAULT_FORMAT = {"qwen3next-style": "exl3", "glm-style": "exl3", "ds4-style": "mx"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference is a Rust binary + sm_121-only CUDA shim with no setup.py/pyproject.toml: "
                       "`pip install --target baseline/_ref <reference checkout>` fails (not installable), no Rust toolchain offline",
    }))
    return 0


def spec_rounds(eng, cfg, prompts, S, steps, graphs, barrier):
    """Speculative rounds on the bench model: MTP chain of 3 drafts per sequence, 4 rows per sequence verified, accepted
    rows committed.  Random weights accept next to nothing, so the cost of a round is the figure, not tokens/s."""
    import torch
    from spark_engine_b200.spec.decoder import SpecDecoder
    try:
        sd = SpecDecoder(eng.model, "mtp", depth=3, policy="all", graphs=graphs)
        seqs = [sd.start(s, prompts[s].tolist(), chunk=1024) for s in range(S)]
        for _ in range(4):
            sd.round(seqs)
        barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        emitted = 0
        ev[0].record()
        for _ in range(steps):
            emitted += sum(len(o) for o in sd.round(seqs))
        ev[1].record()
        barrier()
        out = {"rows_per_seq": 4, "sequences": S, "round_ms": round(ev[0].elapsed_time(ev[1]) / steps, 4),
               "tokens_per_round": round(emitted / steps, 3), "graphs": bool(sd.graphs),
               "accepted_drafts": sum(s.accepted for s in seqs), "drafted": sum(s.drafted for s in seqs)}
        if sd.graphs is not None:                      # the three captured pieces on their own (replays back to back)
            def timed(fn, n=32):
                torch.cuda.synchronize()
                ev[0].record()
                for _ in range(n):
                    fn()
                ev[1].record()
                torch.cuda.synchronize()
                return round(ev[0].elapsed_time(ev[1]) / n, 4)
            vg = next((g for g in sd.graphs.rounds.values() if g.k == 4 and g.graph is not None), None)
            mg = next((g for g in sd.graphs.mtp.values() if g.graph is not None), None)
            if vg is not None:
                out["verify_ms"] = timed(vg.graph.replay)
                if vg.graph_commit is not None:
                    out["commit_ms"] = timed(vg.graph_commit.replay)
                out["verify_launches"] = vg.launches
            if mg is not None:
                out["draft_chain_ms"] = timed(mg.graph.replay)
                out["draft_launches"] = mg.launches
        return out
    except Exception as e:                              # the headline must not depend on this extra
        return {"error": f"{type(e).__name__}: {e}"[:300]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", help="ours | aten (same model code on PyTorch/ATen ops) | reference")
    ap.add_argument("--model", default="qwen3next-style")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (0 = the named config; a reduced "
                                                          "count is reported in `config` and is not the headline)")
    ap.add_argument("--streams", type=int, default=4)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--format", default=None, help="dense | exl3 | mx (default: the config's)")
    ap.add_argument("--kv", default=None, help="bf16 | fp8 (default: the config's)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--chunk", type=int, default=0, help="prefill chunk in tokens (default 8192 on one GPU, 4096 under tp)")
    ap.add_argument("--hc", default=None, help="gated | mhc: run the model with 4 hyper-connection residual streams")
    ap.add_argument("--ple", action="store_true",
                    help="add hashed n-gram embedding layers (bi/tri-gram ids, 16 heads, a 4M-row table) to the model")
    ap.add_argument("--spec", default="none", help="mtp: also time speculative rounds (MTP chain of 3 drafts, 4 rows per "
                                                   "sequence verified) through the captured draft / verify / commit graphs")
    ap.add_argument("--sweep", action="store_true", help="also time 1,2,3 streams")
    ap.add_argument("--parallel", default="tp", help="N > 1: tp = one model sharded over the GPUs (tensor + expert "
                                                     "parallel, fused peer-memory all-reduce); dp = one replica per GPU")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from spark_engine_b200 import ops
    from spark_engine_b200.config import EngineConfig, get_model_config
    from spark_engine_b200.models.build import build_random_model, decode_step_bytes, weight_bytes
    from spark_engine_b200.ops import cuda as cu
    from spark_engine_b200.serving.engine import LLMEngine

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    kw = {}
    if args.layers:
        kw["n_layers"] = args.layers
    if args.format:
        kw["weight_format"] = args.format
    cfg = get_model_config(args.model, **kw)
    if args.kv:
        cfg.kv_dtype = args.kv
    if args.hc:
        cfg.hc_kind, cfg.hc_streams, cfg.hc_rank = args.hc, 4, 32
    if args.ple and not cfg.ngram_layers:
        cfg.ngram_layers, cfg.ngram_rows, cfg.ngram_dim = [1, cfg.n_layers // 2], 1 << 22, 1024
    aten = args.impl == "aten"
    if aten and cfg.weight_format != "dense":
        # the ATen path has no kernels for the packed formats: it would dequantise every matrix on the host per call
        if rank == 0:
            print(json.dumps({"impl": "aten", "unavailable": f"the ATen baseline runs bf16 weights only (--format dense, "
                              f"reduced --layers to fit): {cfg.weight_format} weights need this repo's kernels"}))
        if world > 1:
            dist.destroy_process_group()
        return 0
    t0 = time.time()
    tp = None
    use_tp = world > 1 and args.parallel == "tp"
    if use_tp:
        if aten:
            from spark_engine_b200.parallel.tp import NcclTP
            tp = NcclTP()
        else:
            from spark_engine_b200.parallel import symm
            from spark_engine_b200.parallel.tp import DeviceTP
            arena = symm.Arena(1 << 30, wait_ms=4000.0)
            tp = DeviceTP(arena, cfg.hidden, rows_cap=max(1024, args.chunk or 4096))
    W = build_random_model(cfg, dev, seed=0, tp=(rank, world) if use_tp else (0, 1))
    torch.cuda.synchronize()
    build_s = time.time() - t0
    if world > 1:
        dist.barrier()          # ranks finish building their shards at different times
    if aten:
        ops.set_fallback(True)
    S = args.streams
    eng = LLMEngine(cfg, W, EngineConfig(cuda_graphs=not (args.no_graphs or aten), prefill_chunk=args.chunk or (4096 if use_tp else 8192)),
                    device=dev, max_seqs=S, kv_tokens_per_seq=max(4096, 2 * args.prompt), tp=tp)
    g = torch.Generator().manual_seed(1234 + (0 if use_tp else rank))
    prompts = torch.randint(0, cfg.vocab, (S, args.prompt), generator=g)
    pinned_prompts = prompts.to(torch.int32).pin_memory()

    # ---- prefill (TTFT, prefill tok/s): device-timed per stream
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    cur, ttft = [], []
    for s in range(S):
        torch.cuda.synchronize()
        ev0.record()
        lg = eng.prefill(s, pinned_prompts[s].tolist())
        cur.append(int(eng.model.greedy(lg.unsqueeze(0))[0]))
        ev1.record()
        torch.cuda.synchronize()
        ttft.append(ev0.elapsed_time(ev1))
        eng.check_device_status()      # fail fast if a bounded wait gave up
    prefill_tok_s = args.prompt / (min(ttft[1:] or ttft) / 1e3)
    # the same prompts prefilled together (one segment per sequence in shared forwards): aggregate prefill rate
    batched_tok_s = None
    if S > 1:
        try:
            for rep in range(2):            # the second pass is the timed one (first: scratch growth for the larger plan)
                torch.cuda.synchronize()
                ev0.record()
                lgs = eng.prefill_many(list(range(S)), [pinned_prompts[s].tolist() for s in range(S)])
                nxt = eng.model.greedy(lgs)
                ev1.record()
                torch.cuda.synchronize()
            batched_tok_s = S * args.prompt / (ev0.elapsed_time(ev1) / 1e3)
            cur = [int(t) for t in nxt]
            eng.check_device_status()
        except Exception as e:              # the secondary figure must not take the headline measurement with it
            print(f"[bench] shared prefill skipped: {e!r}", file=sys.stderr, flush=True)
            batched_tok_s = None
            cur = []
            for s in range(S):
                lg = eng.prefill(s, pinned_prompts[s].tolist())
                cur.append(int(eng.model.greedy(lg.unsqueeze(0))[0]))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_decode(n_streams: int, steps: int, warmup: int):
        slots = list(range(n_streams))
        ids = [cur[s] for s in slots]
        for _ in range(max(warmup - 2, 1)):
            ids = eng.decode_round(slots, ids)
        ids = eng.decode_steps(slots, ids, 2)[-1]              # warms the device-fed variant of the round as well
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        n0 = cu.launch_count()
        # device-timed: K real decode steps, sampled ids fed back on the device
        ev0.record()
        toks = eng.decode_steps(slots, ids, steps)
        ev1.record()
        barrier()
        dev_ms = ev0.elapsed_time(ev1) / steps
        launches = cu.launch_count() - n0
        ids = toks[-1]
        # end to end through the public per-step API: pinned H2D of ids + positions, D2H of the result, every step
        barrier()
        t_a = time.perf_counter()
        for _ in range(steps):
            ids = eng.decode_round(slots, ids)
        barrier()
        e2e_ms = (time.perf_counter() - t_a) * 1e3 / steps
        clocks = sampler.stop()
        for s, t in zip(slots, ids):
            cur[s] = t
        return dev_ms, e2e_ms, clocks, launches

    dev_ms, e2e_ms, clocks, launches_total = timed_decode(S, args.steps, max(args.warmup, 3))
    sweep = {}
    if args.sweep:
        for n in range(1, S):
            d, e, _, _ = timed_decode(n, args.steps, 3)
            sweep[str(n)] = {"decode_tok_s": round(n * 1e3 / d, 1), "e2e_tok_s": round(n * 1e3 / e, 1), "ms_per_step": round(d, 4)}
    spec = None
    if args.spec == "mtp" and eng.model.mtp_layers and not aten:
        spec = spec_rounds(eng, cfg, pinned_prompts, S, args.steps, not args.no_graphs, barrier)
    if world > 1:
        t = torch.tensor([dev_ms, e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = t.tolist()
    st = cu.read_status(dev)
    replicas = 1 if use_tp else world
    value = replicas * S * 1e3 / dev_ms
    e2e = replicas * S * 1e3 / e2e_ms
    full = (args.layers == 0 and args.model in BASELINE_DECODE_4STREAMS and not args.hc and not args.ple
            and cfg.weight_format == DEFAULT_FORMAT[args.model])
    # what a step streams: the weights a round of S rows touches on this rank (not the whole model)
    step_bytes = decode_step_bytes(W, cfg, S)
    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    hbm_gbs = float(peaks.get("hbm_gbs", 6650.0))
    kv_t = next((mix.k if hasattr(mix, "k") else mix.lat for _, mix, _ in eng.model.layers if hasattr(mix, "k") or hasattr(mix, "lat")), None)
    kv_label = {torch.bfloat16: "bf16", torch.float8_e4m3fn: "fp8", torch.uint8: "fp8 (packed latent rows)", torch.float32: "fp32"}.get(kv_t.dtype, str(kv_t.dtype)) \
        if kv_t is not None else "none"
    out = {
        "metric": "aggregate decode tok/s at 4 streams" if S == 4 else f"aggregate decode tok/s at {S} streams",
        "value": round(value, 2), "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(dev_ms, 4), "higher_is_better": True, "scaling": "strong" if use_tp or world == 1 else "weak",
        "vs_baseline": round(value / BASELINE_DECODE_4STREAMS[args.model], 3) if full and S == 4 and not aten else None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"model": cfg.name, "layers": cfg.n_layers, "hidden": cfg.hidden, "experts": cfg.moe.n_experts,
                   "top_k": cfg.moe.top_k, "vocab": cfg.vocab, "weights": cfg.weight_format + ("-4bpw" if cfg.weight_format == "exl3" else ""),
                   "kv": kv_label, "global_batch": replicas * S, "seq_len": args.prompt, "streams_per_gpu": S,
                   "parallelism": (f"tp{world}+ep{world}" if use_tp else f"dp{world}") if world > 1 else "single", "speculation": "none (greedy)", "hyper_connections": cfg.hc_kind,
                   "ngram_layers": list(cfg.ngram_layers),
                   "cache": "inputs larger than L2: a step streams %.2f GB of weights per GPU (of %.1f GB resident)"
                            % (step_bytes / 1e9, weight_bytes(W) / 1e9),
                   "full_config": full},
        "step_weight_bytes": step_bytes,
        "hbm_fraction": round(step_bytes / (dev_ms * 1e-3) / (hbm_gbs * 1e9), 4),
        "hbm_fraction_of": "measured copy bandwidth %.0f GB/s" % hbm_gbs if peaks else "fallback 6650 GB/s",
        "clocks": clocks,
        "e2e": {"value": round(e2e, 2), "unit": "tok/s",
                "h2d_bytes_per_step": (next(iter(eng.graphs.values())).host.numel() * 4 if eng.graphs else 16 * S),
                "d2h_bytes_per_step": 4 * S, "ms_per_step": round(e2e_ms, 4)},
        "gpu_launches": launches_total,
        "prefill_tok_s": round(prefill_tok_s, 1),
        "prefill_batched_tok_s": round(batched_tok_s, 1) if batched_tok_s else None, "ttft_ms": round(statistics.median(ttft), 2),
        "streams_sweep": sweep, "weight_build_s": round(build_s, 1), "device_status": list(st),
    }
    if spec is not None:
        out["spec_mtp"] = spec
    if aten:
        out["impl"] = "aten"
        out["note"] = "library baseline: this repo's model code on PyTorch/ATen ops (+ NCCL), not the reference"
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
