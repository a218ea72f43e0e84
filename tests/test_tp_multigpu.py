"""Tensor/expert-parallel model on >= 2 GPUs: sharded tiny hybrid MoE through the fused all-reduce kernels vs the
single-GPU run; an EXL3 model through the GEMV-fused all-reduce under CUDA graphs."""
import os
import socket

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from spark_engine_b200.config import EngineConfig, qwen3next_style, tiny_hybrid
    from spark_engine_b200.models.build import build_random_model
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights, to_device
    from spark_engine_b200.parallel import symm
    from spark_engine_b200.parallel.tp import DeviceTP, shard_dense_weights
    from spark_engine_b200.serving.engine import LLMEngine
    arena = symm.Arena(512 << 20)
    # ---- dense tiny model: TP logits vs single-GPU logits
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    tp = DeviceTP(arena, cfg.hidden, rows_cap=64)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
    ref = Model(cfg, to_device(W, dev), device=dev, dtype=torch.bfloat16, n_slots=1, kv_tokens=128)
    m = Model(cfg, to_device(shard_dense_weights(W, cfg, rank, world), dev), device=dev, dtype=torch.bfloat16, n_slots=1,
              kv_tokens=128, tp=tp)
    lr = ref.forward(make_plan([(0, ids[:32], 0)], device=dev))
    lt = m.forward(make_plan([(0, ids[:32], 0)], device=dev))
    parts = [torch.empty_like(lt) for _ in range(world)]
    dist.all_gather(parts, lt.contiguous())
    full = torch.cat(parts, 1)
    err = ((full - lr).norm() / lr.norm()).item()
    assert err < 3e-2, err
    toks = m.greedy(lt)
    assert (toks.long() == full.argmax(-1)).all()
    # ---- the other families (KDA + latent attention, compressed sparse latent attention): sharded vs single GPU
    from spark_engine_b200.config import get_model_config, scaled_down
    for k, name in enumerate(("glm-style", "ds4-style")):
        cfg3 = scaled_down(get_model_config(name))
        cfg3.mtp_layers = 0
        cfg3.kv_dtype = "bf16"                       # sharding arithmetic only: e4m3 cache codes amplify last-bit differences
        W3 = init_weights(cfg3, seed=1)
        for lw in W3["layers"]:                      # wide router margins: a bf16 rounding difference must not flip an expert,
            if "gate" in lw["mlp"]:                  # so the comparison measures arithmetic, not routing luck
                lw["mlp"]["gate"] = lw["mlp"]["gate"] * 8.0
        tp3 = DeviceTP(arena, cfg3.hidden, rows_cap=64, name=f"tp3{k}")
        ref3 = Model(cfg3, to_device(W3, dev), device=dev, dtype=torch.bfloat16, n_slots=1, kv_tokens=128)
        m3 = Model(cfg3, to_device(shard_dense_weights(W3, cfg3, rank, world), dev), device=dev, dtype=torch.bfloat16,
                   n_slots=1, kv_tokens=128, tp=tp3)
        ids3 = [t % cfg3.vocab for t in ids]
        for plan_items in ([(0, ids3[:36], 0)], [(0, ids3[36:37], 36)]):
            lr3 = ref3.forward(make_plan(plan_items, device=dev))
            lt3 = m3.forward(make_plan(plan_items, device=dev))
            parts3 = [torch.empty_like(lt3) for _ in range(world)]
            dist.all_gather(parts3, lt3.contiguous())
            err3 = ((torch.cat(parts3, 1) - lr3).norm() / lr3.norm()).item()
            assert err3 < 3e-2, (name, err3)
    # ---- EXL3 model, graphs on: GEMV-fused all-reduce in the decode graph; all ranks emit the same tokens
    cfg2 = qwen3next_style(n_layers=4)
    cfg2.moe.n_experts = 32
    cfg2.vocab = 4096
    tp2 = DeviceTP(arena, cfg2.hidden, rows_cap=64, name="tp2")
    W2 = build_random_model(cfg2, dev, seed=0, tp=(rank, world))
    eng = LLMEngine(cfg2, W2, EngineConfig(cuda_graphs=True, prefill_chunk=64), device=dev, max_seqs=2, kv_tokens_per_seq=512, tp=tp2)
    prompts = torch.randint(0, cfg2.vocab, (2, 48), generator=g).tolist()
    outs = eng.generate(prompts, 10)
    t = torch.tensor(outs, device=dev)
    allt = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(allt, t)
    assert all(torch.equal(a, allt[0]) for a in allt), "ranks diverged"
    eng2 = LLMEngine(cfg2, W2, EngineConfig(cuda_graphs=False, prefill_chunk=64), device=dev, max_seqs=2, kv_tokens_per_seq=512, tp=tp2)
    assert eng2.generate(prompts, 10) == outs, "graph replay differs from eager under TP"
    # ---- the SAME quantised weights on one GPU and sharded: every rank generates the full EXL3 model from one seed, takes
    # its shard of the packed tensors (no decode / re-encode), and the sharded logits must match the unsharded ones
    from spark_engine_b200.parallel.tp import shard_weights
    cfg4 = qwen3next_style(n_layers=4)
    cfg4.moe.n_experts, cfg4.vocab, cfg4.mtp_layers = 32, 4096, 1
    Wfull = build_random_model(cfg4, dev, seed=3, tp=(0, 1))
    for lw in Wfull["layers"]:
        if "gate" in lw["mlp"]:
            lw["mlp"]["gate"] = (lw["mlp"]["gate"].float() * 8.0).to(lw["mlp"]["gate"].dtype)
    one = Model(cfg4, Wfull, device=dev, dtype=torch.bfloat16, n_slots=2, kv_tokens=1024)
    tp4 = DeviceTP(arena, cfg4.hidden, rows_cap=512, name="tp4")
    shard = Model(cfg4, shard_weights(Wfull, cfg4, rank, world), device=dev, dtype=torch.bfloat16, n_slots=2, kv_tokens=1024, tp=tp4)
    ids4 = torch.randint(0, cfg4.vocab, (2, 40), generator=g).tolist()
    # a 256-row prefill chunk takes the sequence-parallel path (reduce-scatter + owner-side norm + all-gather)
    long_ids = torch.randint(0, cfg4.vocab, (256,), generator=g).tolist()
    l_one = one.forward(make_plan([(1, long_ids, 0)], device=dev))
    h_one = one.hidden_out.clone()
    l_sp = shard.forward(make_plan([(1, long_ids, 0)], device=dev))
    assert tp4.rp is not None and not tp4.rows_sharded      # the residual was gathered back at the end of the forward
    parts_sp = [torch.empty_like(l_sp) for _ in range(world)]
    dist.all_gather(parts_sp, l_sp.contiguous())
    err_sp = ((torch.cat(parts_sp, 1) - l_one).norm() / l_one.norm()).item()
    assert err_sp < 3e-2, ("sequence-parallel prefill vs one GPU", err_sp)
    assert ((shard.hidden_out - h_one).norm() / h_one.norm()).item() < 3e-2
    one.reset_slot(1)
    shard.reset_slot(1)
    for items in ([(0, ids4[0][:32], 0), (1, ids4[1][:32], 0)], [(0, ids4[0][32:33], 32), (1, ids4[1][32:33], 32)],
                  [(0, ids4[0][33:37], 33), (1, ids4[1][33:37], 33)]):
        l1 = one.forward(make_plan(items, device=dev))
        lt4 = shard.forward(make_plan(items, device=dev))
        parts4 = [torch.empty_like(lt4) for _ in range(world)]
        dist.all_gather(parts4, lt4.contiguous())
        err4 = ((torch.cat(parts4, 1) - l1).norm() / l1.norm()).item()
        assert err4 < 3e-2, ("same EXL3 weights, sharded vs one GPU", err4)
        if lt4.shape[0] >= 32:                           # random weights give near-flat logits: judge the arg-max on many rows
            assert (shard.greedy(lt4).long() == l1.argmax(-1)).float().mean() > 0.8
    # ---- speculative rounds under tensor parallelism: captured MTP chain / verify / commit graphs == eager rounds, all ranks agree
    from spark_engine_b200.spec.decoder import SpecDecoder
    outs_sd = []
    for graphs in (False, True):
        msd = Model(cfg4, shard_weights(Wfull, cfg4, rank, world), device=dev, dtype=torch.bfloat16, n_slots=2, kv_tokens=1024,
                    tp=tp4)
        sd = SpecDecoder(msd, "mtp", depth=3, graphs=graphs)
        outs_sd.append(sd.generate([ids4[0][:24], ids4[1][:24]], 12, temperature=0.7, seed=9))
        if graphs:
            assert sd.graphs is not None and sd.graphs.rounds and sd.graphs.mtp
    assert outs_sd[0] == outs_sd[1], "speculative graphs differ from eager rounds under TP"
    t = torch.tensor(outs_sd[1], device=dev)
    allt = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(allt, t)
    assert all(torch.equal(a, allt[0]) for a in allt), "ranks diverged in sampled speculative decoding"
    torch.cuda.synchronize()
    assert arena.status()[0] == 0, arena.status()
    arena.close()
    dist.destroy_process_group()


def test_tp_model_matches_single_gpu():
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
