"""Speculative rounds through captured CUDA graphs on the device: the drafter chain, the padded verify forward and the
commit with device-side accepted counts must emit exactly the tokens of the eager rounds and of plain greedy decoding."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from spark_engine_b200.config import tiny_hybrid
from spark_engine_b200.models.model import Model
from spark_engine_b200.models.weights import init_weights, to_device
from spark_engine_b200.spec.decoder import SpecDecoder


def _model(n_slots=2):
    cfg = tiny_hybrid()
    cfg.mtp_layers, cfg.mtp_depth = 1, 3
    W = to_device(init_weights(cfg, seed=0), "cuda")
    return cfg, W, Model(cfg, W, device="cuda", dtype=torch.bfloat16, n_slots=n_slots, kv_tokens=512 * n_slots)


def _greedy(cfg, W, prompts, n):
    m = Model(cfg, W, device="cuda", dtype=torch.bfloat16, n_slots=len(prompts), kv_tokens=512 * len(prompts))
    return SpecDecoder(m, lambda s, d: ([], []), depth=0).generate(prompts, n)


def test_mtp_chain_graphs_equal_eager_and_greedy():
    cfg, W, m = _model()
    g = torch.Generator().manual_seed(3)
    prompts = torch.randint(0, cfg.vocab, (2, 24), generator=g).tolist()
    ref = _greedy(cfg, W, prompts, 14)
    eager = SpecDecoder(m, "mtp", depth=3).generate(prompts, 14)
    cfg2, W2, m2 = _model()
    sd = SpecDecoder(m2, "mtp", depth=3, graphs=True)
    got = sd.generate(prompts, 14)
    assert sd.graphs is not None and sd.graphs.rounds and sd.graphs.mtp     # the captured path actually ran
    assert got == eager == ref


@pytest.mark.parametrize("mode", ["perfect", "half", "wrong"])
def test_verify_and_commit_graphs_with_known_drafts(mode):
    """Drafts with a known acceptance pattern: all accepted (the commit advances 4 rows), one accepted, none."""
    cfg, W, m = _model(1)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    ref = _greedy(cfg, W, [prompt], 16)[0]

    def drafter(seq, depth):
        n = len(seq.generated)
        d = ref[n: n + depth]
        if mode == "wrong":
            d = [(t + 1) % cfg.vocab for t in d]
        if mode == "half" and len(d) > 1:
            d = d[:1] + [(t + 1) % cfg.vocab for t in d[1:]]
        return d, [0.9] * len(d)
    sd = SpecDecoder(m, drafter, depth=3, graphs=True)
    assert sd.generate([prompt], 16)[0] == ref
    assert sd.graphs.rounds
    if mode == "perfect":
        assert sd.rounds <= 5


def test_sampled_graph_rounds_equal_eager_sampling():
    cfg, W, m = _model(1)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (16,), generator=g).tolist()
    eager = SpecDecoder(m, "mtp", depth=3).generate([prompt], 10, temperature=1.0, seed=42)[0]
    cfg2, W2, m2 = _model(1)
    graph = SpecDecoder(m2, "mtp", depth=3, graphs=True).generate([prompt], 10, temperature=1.0, seed=42)[0]
    assert graph == eager


def test_token_prob_kernel():
    from spark_engine_b200.ops import cuda as cu
    torch.manual_seed(1)
    lg = torch.randn(5, 3001, device="cuda") * 4
    ids = torch.tensor([0, 17, 3000, 1500, 2], dtype=torch.int32, device="cuda")
    got = cu.token_prob(lg, ids)
    want = torch.softmax(lg, -1)[torch.arange(5), ids.long()]
    assert (got - want).abs().max().item() < 1e-5


@pytest.mark.parametrize("family", ["hybrid", "glm"])
def test_tree_rounds_on_the_device_equal_greedy(family):
    """Tree verification (width 4, depth 5) through the kernels: ancestor-masked attention, one root-to-node walk per
    node for the linear-attention layers, commit of the accepted walk; the emitted text is plain greedy decoding."""
    from spark_engine_b200.spec.tree import Node
    if family == "hybrid":
        cfg, W, m = _model(1)
    else:
        from spark_engine_b200.config import get_model_config, scaled_down
        cfg = scaled_down(get_model_config("glm-style"))
        cfg.mtp_layers = 0
        W = to_device(init_weights(cfg, seed=0), "cuda")
        m = Model(cfg, W, device="cuda", dtype=torch.bfloat16, n_slots=1, kv_tokens=512)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab, (20,), generator=g).tolist()
    ref = _greedy(cfg, W, [prompt], 18)[0]
    sd = SpecDecoder(m, lambda s, d: ([], []), depth=0)
    seq = sd.start(0, prompt)
    while len(seq.generated) < 18:
        n = len(seq.generated)
        want = ref[n: n + 5]
        nodes, parent = [], -1
        for j, tok in enumerate(want):
            good = tok if j < 3 else (tok + 1) % cfg.vocab           # the spine is right for three levels
            sibs = [(tok + 2 + q) % cfg.vocab for q in range(3)]
            order = sibs[:1] + [good] + sibs[1:] if j == 1 else [good] + sibs     # level 1: the right child is not the first
            first = len(nodes)
            for t in order:
                nodes.append(Node(parent, t))
            parent = first + (1 if j == 1 else 0)
        out = sd.round_tree([seq], [nodes], budgets=[18 - n])[0]
        assert len(out) >= 1
    assert seq.generated[:18] == ref
    assert seq.accepted > 0


def test_latent_attention_tree_rows_kernel_equals_generic_path():
    """Tree rows of latent attention through the kernels (node slots, ancestor bit-masks) against the per-segment
    masked-softmax path, and the indexer pools that the accepted path completes at compaction."""
    from spark_engine_b200.config import get_model_config, scaled_down
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.ops import cuda as cu
    cfg = scaled_down(get_model_config("glm-style"))
    cfg.mtp_layers = 0
    W = to_device(init_weights(cfg, seed=0), "cuda")
    g = torch.Generator().manual_seed(8)
    prompt = torch.randint(0, cfg.vocab, (2, 70), generator=g).tolist()       # trees start at 70: the kernel's second split
    toks = torch.randint(0, cfg.vocab, (2, 9), generator=g).tolist()
    parents = [[-1, 0, 0, 1, 1, 2, 3, 3, 6], [-1, 0, 1, 2, 0, 4, 4, 5, 7]]
    outs, pools = [], []
    for kernels in (True, False):
        m = Model(cfg, W, device="cuda", dtype=torch.bfloat16, n_slots=2, kv_tokens=512)
        m.forward(make_plan([(0, prompt[0], 0), (1, prompt[1], 0)], device="cuda", all_logits=False), commit=True)
        old = cu.MLA_KERNELS
        cu.MLA_KERNELS = kernels
        try:
            plan = make_plan([(0, toks[0], 70), (1, toks[1], 70)], device="cuda", parents=parents)
            outs.append(m.forward(plan, commit=False).float())
            mla = [mix for _, mix, _ in m.layers if hasattr(mix, "lat")]
            assert mla
            for seg, rows in zip(plan.segs, ([0, 1, 3, 6, 8], [0, 4, 5, 7])):
                for mx in mla:
                    mx.compact(m.seqs, seg, rows)
            pools.append(torch.stack([mx.pool.float().clone() for mx in mla]))
        finally:
            cu.MLA_KERNELS = old
    assert torch.isfinite(outs[0]).all()
    err = (outs[0] - outs[1]).abs().max().item() / outs[1].abs().max().item()
    assert err < 3e-2, err
    assert (pools[0] - pools[1]).abs().max().item() < 3e-2 * pools[1].abs().max().item()
