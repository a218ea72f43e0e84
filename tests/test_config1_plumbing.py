"""Tiny hybrid MoE decoder, fp32 on CPU: the incremental engine (chunked prefill + greedy decode
with sequence state) must reproduce the full-sequence oracle's logits to 1e-4."""
import torch

from spark_engine_b200.config import tiny_hybrid
from spark_engine_b200.models.model import Model
from spark_engine_b200.models.plan import make_plan
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.oracle import model as oracle


def _setup():
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (2, 64), generator=g)
    return cfg, W, prompts


def test_prefill_and_32_greedy_steps_match_oracle():
    cfg, W, prompts = _setup()
    m = Model(cfg, W, n_slots=2, kv_tokens=512)
    n_new = 32
    ref = [oracle.greedy_generate(cfg, W, prompts[i], n_new) for i in range(2)]
    # prefill both sequences in two chunks each (chunk boundary inside a conv window / 4-block)
    last = []
    for s in range(2):
        m.forward(make_plan([(s, prompts[s, :37].tolist(), 0)], all_logits=False))
        lg = m.forward(make_plan([(s, prompts[s, 37:].tolist(), 37)], all_logits=False))
        last.append(lg[0])
    toks = [[], []]
    logits = [[], []]
    cur = [int(torch.argmax(l)) for l in last]
    for s in range(2):
        toks[s].append(cur[s]); logits[s].append(last[s])
    for step in range(n_new - 1):
        plan = make_plan([(s, [cur[s]], 64 + step) for s in range(2)])
        lg = m.forward(plan)
        for s in range(2):
            cur[s] = int(torch.argmax(lg[s]))
            toks[s].append(cur[s]); logits[s].append(lg[s])
    for s in range(2):
        assert toks[s] == ref[s][0].tolist()
        err = (torch.stack(logits[s]) - ref[s][1]).abs().max().item()
        assert err < 1e-4, err


def test_full_prefill_logits_match_oracle():
    cfg, W, prompts = _setup()
    m = Model(cfg, W, n_slots=1, kv_tokens=128)
    lg = m.forward(make_plan([(0, prompts[0].tolist(), 0)]))
    ref = oracle.forward(cfg, W, prompts[0])
    assert (lg - ref).abs().max().item() < 1e-4
