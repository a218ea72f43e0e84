"""Feature-conditioned (DFlash2-style) and staged (DSpark-style) drafters: candidate paths, trees, and exactness of
speculative decoding with them (drafts only change speed, never the tokens)."""
import pytest
import torch

from spark_engine_b200.config import tiny_hybrid
from spark_engine_b200.models.model import Model
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.spec import drafters as D
from spark_engine_b200.spec.decoder import SpecDecoder
from spark_engine_b200.spec.tree import check_topological


def test_greedy_path_and_tree():
    g = torch.Generator().manual_seed(0)
    unary = torch.randn(4, 6, generator=g)
    edges = torch.randn(3, 6, 6, generator=g)
    path = D.greedy_path(unary, edges)
    assert path[0] == int(unary[0].argmax())
    for j in range(3):
        assert path[j + 1] == int((unary[j + 1] + edges[j, path[j]]).argmax())
    ids = torch.arange(24).view(4, 6)
    c = D.Candidates(ids, unary, edges, path, [0.5] * 4)
    nodes = D.to_tree(c, [3, 2, 2, 1])
    check_topological(nodes)
    assert len(nodes) == 8
    spine = [n.token for n in nodes if n is nodes[0] or True][:1]
    assert nodes[0].token == int(ids[0, path[0]]) and nodes[0].parent == -1
    # siblings share the parent of the spine node of their depth; the spine continues from the previous spine node
    assert nodes[1].parent == -1 and nodes[2].parent == -1 and nodes[3].parent == 0 and nodes[3].token == int(ids[1, path[1]])


def _greedy(cfg, W, prompt, n):
    m = Model(cfg, W, n_slots=1, kv_tokens=256)
    return SpecDecoder(m, drafter=None, depth=0).generate([prompt], n)[0]


def test_speculation_with_feature_and_stage_drafters_is_exact():
    cfg = tiny_hybrid()
    cfg.mtp_layers = 0
    W = init_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab, (24,), generator=torch.Generator().manual_seed(3)).tolist()
    ref = _greedy(cfg, W, prompt, 20)
    m = Model(cfg, W, n_slots=1, kv_tokens=256)
    fd = D.FeatureDrafter(m, D.FeatureDrafterConfig(target_hidden=cfg.hidden, taps=(0, cfg.n_layers - 1), vocab=cfg.vocab,
                                                    sub_vocab=min(512, cfg.vocab), depth=3, cand_k=8))
    out = SpecDecoder(m, drafter=fd, depth=3).generate([prompt], 20)[0]
    assert out == ref
    assert fd.last is not None and fd.last.ids.shape == (3, 8)
    m2 = Model(cfg, W, n_slots=1, kv_tokens=256)
    sd = D.StageDrafter(D.StageDrafterConfig(hidden=cfg.hidden, vocab=cfg.vocab, threshold=0.0))
    out2 = SpecDecoder(m2, drafter=sd, depth=4).generate([prompt], 20)[0]
    assert out2 == ref


def test_stage_drafter_lengths_follow_confidence():
    sd = D.StageDrafter(D.StageDrafterConfig(threshold=0.5))
    assert sd.draft_length([0.9, 0.9, 0.5, 0.9], 5) == 2          # 0.81 ok, 0.405 < 0.5
    assert sd.draft_length([0.4], 5) == 0
    assert sd.draft_length([0.99] * 5, 3) == 3
    toks, confs = sd.propose_block(torch.randn(256, generator=torch.Generator().manual_seed(1)), 7)
    assert len(toks) == 5 and all(0.0 <= c <= 1.0 for c in confs)
    assert (toks, confs) == sd.propose_block(torch.randn(256, generator=torch.Generator().manual_seed(1)), 7)


def test_tree_verification_rounds_are_exact():
    """Rounds that verify a candidate TREE (feature drafter: spine + siblings) emit exactly the greedy tokens; the
    accepted path is committed through linear-attention replay and KV compaction."""
    cfg = tiny_hybrid()
    cfg.mtp_layers = 0
    W = init_weights(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(5)).tolist()
    ref = _greedy(cfg, W, prompt, 16)
    m = Model(cfg, W, n_slots=1, kv_tokens=256)
    fd = D.FeatureDrafter(m, D.FeatureDrafterConfig(target_hidden=cfg.hidden, taps=(0, cfg.n_layers - 1), vocab=cfg.vocab,
                                                    sub_vocab=min(512, cfg.vocab), depth=3, cand_k=8))
    dec = SpecDecoder(m, drafter=None, depth=0)
    seq = dec.start(0, prompt)
    out = list(seq.generated)
    # mix the drafter's tree with a tree that contains the true continuation, so that deep acceptances occur too
    rnd = 0
    while len(out) < 16:
        cand = fd.candidates(seq)
        nodes = D.to_tree(cand, [3, 2, 2])
        if rnd % 2 == 1:
            k = len(out)
            true_next = ref[k: k + 2]
            nodes = [D.Node(-1, (true_next[0] + 1) % cfg.vocab), D.Node(-1, true_next[0])]
            if len(true_next) > 1:
                nodes += [D.Node(1, true_next[1]), D.Node(1, (true_next[1] + 7) % cfg.vocab)]
        emitted = dec.round_tree([seq], [nodes], budgets=[16 - len(out)])[0]
        assert 1 <= len(emitted) <= len(nodes) + 1
        if rnd % 2 == 1 and len(true_next) > 1 and 16 - len(out) >= 3:
            assert len(emitted) == 3                         # root sample + both true nodes accepted
        out += emitted
        rnd += 1
    assert out == ref


@pytest.mark.gpu
def test_candidate_selection_kernels_match_the_host_selection():
    """Sorted top-K log-probabilities, pairwise edges and the greedy path on the device equal the host formulas,
    including ties (equal logits resolve to the lowest id)."""
    g = torch.Generator().manual_seed(0)
    J, V, K, d, r = 4, 512, 16, 64, 32
    logits = torch.randn(J, V, generator=g) * 2
    logits[1, 7] = logits[1, 300] = logits[1].max() + 1.0          # a tie for the best candidate
    embed, eu, ev = torch.randn(V, d, generator=g), torch.randn(r, d, generator=g), torch.randn(r, d, generator=g)
    ids, unary, edges, path, conf = D.select_candidates(logits, embed, eu, ev, K)
    gi, gu, ge, gp, gc = D.select_candidates(logits.cuda(), embed.cuda(), eu.cuda(), ev.cuda(), K)
    assert torch.equal(gi.cpu(), ids) and ids[1, 0] == 7 and ids[1, 1] == 300
    assert (gu.cpu() - unary).abs().max() < 1e-5 and (ge.cpu() - edges).abs().max() < 1e-3
    assert gp == path and max(abs(a - b) for a, b in zip(gc, conf)) < 1e-5
