"""Speculative decoding: acceptance walk unit tests (in the spirit of engine-rs/src/speculative.rs:40-80) and
end-to-end exactness: speculative output == plain greedy output, token for token."""
import pytest
import torch

from spark_engine_b200.config import tiny_hybrid
from spark_engine_b200.models.model import Model
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.oracle import model as oracle
from spark_engine_b200.spec import policy as P
from spark_engine_b200.spec import sampling
from spark_engine_b200.spec.decoder import SpecDecoder
from spark_engine_b200.spec.lookup import LookupIndex
from spark_engine_b200.spec.tree import Node, accept, chain


def test_rejection_at_every_depth_keeps_exact_prefix():
    truth = [5, 6, 7, 8, 9]                       # what greedy decoding emits next
    for wrong_at in range(5):                     # 4 = no wrong draft
        d = list(truth[:4])                       # draft j guesses truth[j]
        if wrong_at < 4:
            d[wrong_at] = 99
        # the target's prediction after node j is truth[j+1] as long as the whole prefix d[:j+1] is right
        preds = [truth[j + 1] if d[: j + 1] == truth[: j + 1] else 0 for j in range(4)]
        path, out, _ = accept(chain(d), truth[0], preds)
        assert len(path) == wrong_at
        assert out == truth[: wrong_at + 1]       # accepted drafts + the bonus token


def test_sibling_branches_do_not_leak_and_budget_and_stop():
    nodes = [Node(-1, 1), Node(-1, 2), Node(0, 3), Node(1, 4), Node(3, 5)]
    path, out, _ = accept(nodes, 2, [9, 4, 9, 5, 7])
    assert path == [1, 3, 4] and out == [2, 4, 5, 7]
    path, out, _ = accept(nodes, 2, [9, 4, 9, 5, 7], budget=2)
    assert out == [2, 4]
    path, out, stopped = accept(nodes, 2, [9, 4, 9, 5, 7], stop=[4])
    assert out == [2, 4] and stopped
    assert accept(nodes, 8, [0] * 5, budget=0)[1] == []


def test_policies():
    assert P.tau_depth([0.9, 0.8, 0.2, 0.9], 0.5, 8) == 2
    assert P.tau_depth([0.1, 0.9], 0.5, 8) == 1
    assert P.theta_depth([0.9, 0.9, 0.5, 0.9], 0.6, 8) == 2
    t = P.AcceptanceTable()
    for _ in range(200):
        t.observe(0, 0.95, True)
        t.observe(1, 0.15, False)
    assert t.prob(0, 0.95) > 0.9 and t.prob(1, 0.15) < 0.2
    assert P.rate_depth([0.95, 0.15, 0.15], t, P.CostModel(), 1, 0, 3) >= 1
    assert sum(P.split_rows([[0.9, 0.9], [0.2, 0.2]], 4, t, 3)) == 2
    cm = P.CostModel()
    cm.fit([(s, r, 10 + 1.0 * s + 2.0 * r) for s in (1, 2, 4) for r in (1, 4, 8)])
    assert abs(cm.per_row_ms - 2.0) < 1e-6 and abs(cm.base_ms - 10.0) < 1e-6


def test_lookup_and_gumbel_sampling():
    ix = LookupIndex(3)
    ix.extend([1, 2, 3, 4, 5, 9, 1, 2, 3])
    assert ix.propose(3) == [4, 5, 9]
    g1 = sampling.gumbel_noise_ref(7, 11, 1000)
    assert torch.equal(g1, sampling.gumbel_noise_ref(7, 11, 1000)) and not torch.equal(g1, sampling.gumbel_noise_ref(7, 12, 1000))
    u = sampling.uniform_ref(3, 5, 200000)
    assert 0.49 < float(u.mean()) < 0.51 and float(u.min()) > 0 and float(u.max()) < 1
    logits = torch.randn(1000)
    full = sampling.sample(logits, 1.0, 7, 11)
    pk = [sampling.packet(logits[o: o + 250], o, 1.0, 7, 11, 1000) for o in range(0, 1000, 250)]
    assert sampling.combine_packets(pk) == full
    assert sampling.combine_packets([(1.0, 9), (1.0, 3), (float("nan"), 0)]) == 3


def _model():
    cfg = tiny_hybrid()
    cfg.mtp_layers, cfg.mtp_depth = 1, 3
    W = init_weights(cfg, seed=0)
    return cfg, W


def test_mtp_speculation_equals_greedy():
    cfg, W = _model()
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, cfg.vocab, (2, 24), generator=g)
    ref = [oracle.greedy_generate(cfg, W, prompts[i], 14)[0].tolist() for i in range(2)]
    m = Model(cfg, W, n_slots=2, kv_tokens=256)
    sd = SpecDecoder(m, "mtp", depth=3)
    out = sd.generate([p.tolist() for p in prompts], 14)
    assert out == ref


def test_perfect_and_adversarial_drafters_equal_greedy():
    cfg, W = _model()
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=g)
    ref = oracle.greedy_generate(cfg, W, prompt, 16)[0].tolist()
    for mode in ("perfect", "half", "wrong"):
        m = Model(cfg, W, n_slots=1, kv_tokens=128)

        def drafter(seq, depth, mode=mode):
            n = len(seq.generated)
            d = ref[n: n + depth]
            if mode == "wrong":
                d = [(t + 1) % cfg.vocab for t in d]
            if mode == "half" and len(d) > 1:
                d = d[:1] + [(t + 1) % cfg.vocab for t in d[1:]]
            return d, [0.9] * len(d)
        sd = SpecDecoder(m, drafter, depth=4)
        assert sd.generate([prompt.tolist()], 16)[0] == ref, mode
        if mode == "perfect":
            assert sd.rounds <= 5


def test_sampled_speculation_is_a_function_of_the_seed():
    cfg, W = _model()
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (16,), generator=g).tolist()
    outs = []
    for drafter in ("mtp", lambda s, d: ([], [])):
        m = Model(cfg, W, n_slots=1, kv_tokens=128)
        outs.append(SpecDecoder(m, drafter, depth=3).generate([prompt], 10, temperature=1.0, seed=42)[0])
    assert outs[0] == outs[1]          # with and without drafts: same text for the same seed


@pytest.mark.parametrize("family", ["hybrid", "glm"])
def test_tree_rounds_stay_lossless_past_the_dense_context(family):
    """Tree rows read the committed context densely; once the sparse-attention layers select (context beyond top-k
    blocks x block) that is no longer what a decode row sees, so the round verifies the tree's spine as a chain: the
    text is still plain greedy decoding and the right drafts are still accepted."""
    import dataclasses
    from spark_engine_b200.config import get_model_config, scaled_down, tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.spec.decoder import SpecDecoder
    if family == "hybrid":
        cfg = tiny_hybrid()
        cfg.layer_types = ["gdn", "attn", "gdn", "attn"]
        cfg.attn = dataclasses.replace(cfg.attn, sparse_topk_blocks=4, block=4, idx_heads=2, idx_dim=32, rope_dim=32)
    else:
        cfg = scaled_down(get_model_config("glm-style"))
        cfg.mtp_layers = 0
    W = init_weights(cfg, seed=1)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab, (60,), generator=g).tolist()
    ref = SpecDecoder(Model(cfg, W, n_slots=1, kv_tokens=256), lambda s, d: ([], []), depth=0).generate([prompt], 14)[0]
    m = Model(cfg, W, n_slots=1, kv_tokens=256)
    assert m.sparse_ctx_limit() is not None and m.sparse_ctx_limit() < len(prompt)
    sd = SpecDecoder(m, lambda s, d: ([], []), depth=0)
    seq = sd.start(0, prompt)
    while len(seq.generated) < 14:
        n = len(seq.generated)
        nodes, parent = [], -1
        for tok in ref[n: n + 3]:
            first = len(nodes)
            nodes.append(Node(parent, tok))
            nodes.append(Node(parent, (tok + 1) % cfg.vocab))
            parent = first
        sd.round_tree([seq], [nodes], budgets=[14 - n])
    assert seq.generated[:14] == ref
    assert seq.accepted >= 8
