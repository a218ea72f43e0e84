"""Tensor/expert-parallel sharding logic on CPU: two gloo ranks run the sharded tiny hybrid MoE and must
reproduce the unsharded logits (fp32; a rank-ordered split sum differs from the single sum only by rounding)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _config(name):
    from spark_engine_b200.config import get_model_config, scaled_down, tiny_hybrid
    if name == "tiny":
        return tiny_hybrid()
    if name in ("tiny-mhc", "tiny-gated"):
        cfg = tiny_hybrid()
        cfg.hc_kind, cfg.hc_streams, cfg.hc_rank, cfg.mtp_layers = name.split("-")[1], 4, 32, 0
        return cfg
    cfg = scaled_down(get_model_config(name))
    cfg.mtp_layers = 0
    return cfg


def _worker(rank, world, port, q, name="tiny"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.parallel.tp import CpuTP, shard_dense_weights
    torch.manual_seed(0)
    cfg = _config(name)
    W = init_weights(cfg, seed=0)
    tp = CpuTP()
    m = Model(cfg, shard_dense_weights(W, cfg, rank, world), n_slots=1, kv_tokens=128, tp=tp)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    lg = m.forward(make_plan([(0, ids[:32], 0)]))
    toks = m.greedy(lg)
    R = lg.shape[0]
    sampled = m.sample_rows(lg, [0.0 if r % 3 == 0 else 0.9 for r in range(R)], [7] * R, list(range(R)))
    prob = m.token_prob(lg[0], sampled[0])
    lg2 = m.forward(make_plan([(0, ids[32:33], 32)]))          # one decode row on top of the prefill state
    parts = [torch.empty_like(lg) for _ in range(world)]
    dist.all_gather(parts, lg)
    parts2 = [torch.empty_like(lg2) for _ in range(world)]
    dist.all_gather(parts2, lg2)
    if rank == 0:
        q.put((torch.cat(parts, 1), toks, torch.cat(parts2, 1), sampled, prob))
    dist.barrier()
    dist.destroy_process_group()


import pytest


@pytest.mark.parametrize("name", ["tiny", "glm-style", "ds4-style", "tiny-mhc", "tiny-gated"])
def test_tp2_logits_match_unsharded(name):
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, name)) for r in range(2)]
    for p in procs:
        p.start()
    logits, toks, logits2, sampled, prob = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cfg = _config(name)
    W = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    ref_m = Model(cfg, W, n_slots=1, kv_tokens=128)
    ref = ref_m.forward(make_plan([(0, ids[:32], 0)]))
    ref2 = ref_m.forward(make_plan([(0, ids[32:33], 32)]))
    assert (logits - ref).abs().max() < 1e-4
    assert (logits2 - ref2).abs().max() < 1e-4
    assert toks.tolist() == ref.argmax(-1).tolist()
    # Gumbel-max sampling keyed by the GLOBAL vocabulary id: the sharded head draws the single-GPU token
    R = ref.shape[0]
    want = ref_m.sample_rows(ref, [0.0 if r % 3 == 0 else 0.9 for r in range(R)], [7] * R, list(range(R)))
    assert sampled == want
    assert abs(prob - float(torch.softmax(ref[0], -1)[want[0]])) < 1e-5


def _worker_many(rank, world, port, q, name):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from spark_engine_b200.config import EngineConfig
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.parallel.tp import CpuTP, shard_dense_weights
    from spark_engine_b200.serving.engine import LLMEngine
    cfg = _config(name)
    W = init_weights(cfg, seed=0)
    eng = LLMEngine(cfg, shard_dense_weights(W, cfg, rank, world), EngineConfig(cuda_graphs=False, prefill_chunk=24),
                    device="cpu", max_seqs=3, kv_tokens_per_seq=128, tp=CpuTP())
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (29, 7, 40)]
    lg = eng.prefill_many([0, 1, 2], prompts)
    toks = eng.model.greedy(lg).tolist()
    nxt = eng.decode_round([0, 1, 2], toks)
    if rank == 0:
        q.put((toks, nxt))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["tiny", "glm-style"])
def test_tp2_shared_prefill_of_several_sequences_matches_unsharded(name):
    """Several ragged prompts prefilled in shared forwards on a model sharded over two ranks (one segment per sequence,
    a row budget per forward) give the tokens of per-sequence prefill on the unsharded model, and so does the next round."""
    from spark_engine_b200.config import EngineConfig
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.serving.engine import LLMEngine
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_many, args=(r, 2, port, q, name)) for r in range(2)]
    for p in procs:
        p.start()
    toks, nxt = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cfg = _config(name)
    W = init_weights(cfg, seed=0)
    ref = LLMEngine(cfg, W, EngineConfig(cuda_graphs=False, prefill_chunk=16), device="cpu", max_seqs=3, kv_tokens_per_seq=128)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (29, 7, 40)]
    want = [int(ref.prefill(s, p).argmax()) for s, p in enumerate(prompts)]
    assert toks == want
    assert nxt == ref.decode_round([0, 1, 2], want)
