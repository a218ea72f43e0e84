"""Host n-gram table: threaded gathers through the staging ring equal plain indexing; file-backed tables."""
import pytest
import torch

from spark_engine_b200.cache.engram import EngramTable


def test_prefetch_equals_index_and_ring_reuse(tmp_path):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(5000, 48, generator=g).bfloat16()
    et = EngramTable(table, ring_slots=3, max_rows=700, threads=3)
    reqs = [torch.randint(0, 5000, (n,), generator=g) for n in (1, 640, 37, 700, 255)]
    futs = []
    for ids in reqs:                       # more requests than ring slots: consume in order, like layer after layer
        futs.append((ids, et.prefetch(ids.view(-1, 1))))
        if len(futs) == 2:
            ids0, f0 = futs.pop(0)
            assert torch.equal(EngramTable.take(f0), table[ids0])
    for ids0, f0 in futs:
        assert torch.equal(EngramTable.take(f0), table[ids0])
    with pytest.raises(ValueError):
        et.prefetch(torch.zeros(701, dtype=torch.long))
    assert et.stats["requests"] == 5
    et.close()
    p = tmp_path / "t.bin"
    p.write_bytes(table.view(torch.int16).numpy().tobytes())
    ef = EngramTable.from_file(str(p), 5000, 48, max_rows=64)
    ids = torch.tensor([0, 4999, 17])
    assert torch.equal(EngramTable.take(ef.prefetch(ids)), table[ids])
    ef.close()


@pytest.mark.gpu
def test_prefetch_to_device():
    table = torch.randn(3000, 64).bfloat16()
    et = EngramTable(table, device="cuda", ring_slots=2, max_rows=512)
    for seed in range(4):
        ids = torch.randint(0, 3000, (300,), generator=torch.Generator().manual_seed(seed))
        rows = EngramTable.take(et.prefetch(ids))
        assert rows.is_cuda and torch.equal(rows.cpu(), table[ids])
    et.close()


def test_integer_chain_row_ids_equal_the_tensor_hash():
    """The decode path hashes the new positions in plain integers against the per-slot id history; same rows as
    the whole-sequence tensor hash, whatever the split into rounds."""
    from types import SimpleNamespace
    from spark_engine_b200.models.ngram import chain_row_ids
    from spark_engine_b200.oracle import layers as L
    m = SimpleNamespace(cfg=SimpleNamespace(ngram_heads=16), W={"ngram_table": torch.zeros(4096, 8)}, id_history={})
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 150000, (40,), generator=g)
    ref = L.ngram_ids(ids, 16, 256)
    got, p = [], 0
    for k in (3, 1, 1, 5, 1, 2, 27):
        got += chain_row_ids(m, 0, p, ids[p:p + k].tolist())
        p += k
    assert torch.equal(torch.tensor(got), ref)
    # a round that rewinds (rejected drafts) re-hashes from the kept prefix
    again = chain_row_ids(m, 0, 12, ids[12:15].tolist())
    assert torch.equal(torch.tensor(again), ref[12:15])
    assert m.id_history[0].tolist() == ids[:15].tolist()


@pytest.mark.gpu
def test_host_resident_table_feeds_the_model_eager_and_under_graphs():
    """DS-style model with its hashed n-gram table left on the host: rows come through the asynchronous gather ring
    (prefetched at the start of a forward, staged with the plan for captured rounds) and the tokens equal those of the
    same model with the table on the device."""
    from spark_engine_b200.config import EngineConfig, get_model_config, scaled_down
    from spark_engine_b200.models.weights import init_weights, to_device
    from spark_engine_b200.serving.engine import LLMEngine
    cfg = scaled_down(get_model_config("ds4-style"))
    cfg.mtp_layers = 0
    assert cfg.ngram_layers
    W = to_device(init_weights(cfg, seed=0), "cuda")
    Wh = dict(W)
    Wh["ngram_table"] = W["ngram_table"].cpu()
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (2, 40), generator=g).tolist()
    ref = LLMEngine(cfg, W, EngineConfig(cuda_graphs=True, prefill_chunk=16), max_seqs=2, kv_tokens_per_seq=256).generate(prompts, 8)
    for graphs in (False, True):
        eng = LLMEngine(cfg, Wh, EngineConfig(cuda_graphs=graphs, prefill_chunk=16), max_seqs=2, kv_tokens_per_seq=256)
        assert eng.model.engram is not None and eng.use_graphs == graphs
        assert eng.generate(prompts, 8) == ref, f"graphs={graphs}"
        assert eng.model.engram.stats["requests"] > 0
