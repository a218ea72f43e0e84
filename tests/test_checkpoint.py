"""Checkpoint round trip (all weight formats), loading as tensor-parallel shards without decoding, pre-split shards."""
import json
import os

import pytest
import torch

from spark_engine_b200.config import qwen3next_style, scaled_down, get_model_config
from spark_engine_b200.models.build import build_random_model
from spark_engine_b200.models.checkpoint import flatten, load_checkpoint, save_checkpoint, write_rank_shards
from spark_engine_b200.parallel.tp import shard_weights
from spark_engine_b200.quant import formats as Q


def _small(fmt):
    cfg = scaled_down(get_model_config("qwen3next-style" if fmt == "exl3" else "ds4-style"))
    cfg.weight_format = fmt
    cfg.n_layers, cfg.layer_types = 2, cfg.layer_types[:1] + cfg.layer_types[-1:]
    cfg.hidden, cfg.vocab, cfg.mtp_layers, cfg.ngram_layers = 256, 512, 0, []
    cfg.moe.n_experts, cfg.moe.top_k, cfg.moe.ffn, cfg.moe.dense_layers = 8, 2, 128, 0
    cfg.gdn.n_k_heads, cfg.gdn.n_v_heads, cfg.gdn.head_dim = 2, 4, 128
    cfg.attn.n_q_heads, cfg.attn.n_kv_heads, cfg.attn.head_dim = 4, 2, 128
    cfg.mla.n_heads, cfg.mla.head_dim, cfg.mla.q_lora, cfg.mla.kv_lora = 4, 128, 128, 128
    return cfg


def _same(a, b):
    ta, _, sa = flatten(a)
    tb, _, sb = flatten(b)
    assert sorted(ta) == sorted(tb)
    for k in ta:
        assert ta[k].dtype == tb[k].dtype and torch.equal(ta[k].cpu().view(torch.uint8), tb[k].cpu().view(torch.uint8)), k
    assert json.dumps(sa, sort_keys=True) == json.dumps(sb, sort_keys=True)


@pytest.mark.parametrize("fmt", ["exl3", "mx"])
def test_round_trip_and_shards(tmp_path, fmt):
    cfg = _small(fmt)
    W = build_random_model(cfg, "cpu", seed=3)
    d = str(tmp_path / "ckpt")
    save_checkpoint(W, cfg, d, max_shard_bytes=1 << 20)          # several shard files
    assert len([f for f in os.listdir(d) if f.endswith(".safetensors")]) > 1
    cfg2, W2 = load_checkpoint(d, "cpu")
    assert cfg2.to_json() == cfg.to_json()
    _same(W, W2)
    # the streamed load (reader threads -> staging buffers -> destination, with and without O_DIRECT) gives the same bytes
    for direct in ("0", "1"):
        os.environ["SPARK_LOAD_DIRECT"] = direct
        try:
            _, W3 = load_checkpoint(d, "cpu", stream=True)
        finally:
            os.environ.pop("SPARK_LOAD_DIRECT", None)
        _same(W, W3)
    # a rank's shard loaded from disk == the shard cut from the in-memory model
    for rank in range(2):
        _, Wr = load_checkpoint(d, "cpu", tp=(rank, 2))
        _same(Wr, shard_weights(W, cfg, rank, 2))
    # pre-split shards are complete checkpoints of each rank
    write_rank_shards(d, str(tmp_path / "split"), 2)
    _, W1 = load_checkpoint(str(tmp_path / "split" / "rank1"), "cpu")
    _same(W1, shard_weights(W, cfg, 1, 2))


def test_quantised_cuts_equal_cuts_of_the_decoded_matrix():
    """Cutting the packed tensors == cutting the decoded matrix (column-parallel rows, row-parallel columns)."""
    g = torch.Generator().manual_seed(0)
    cases = [Q.random_exl3(512, 256, 4, 0, 0.05, 1, "cpu"), Q.random_mxfp4(256, 256, 0, 0.05, 2, "cpu"),
             Q.random_mxfp8(256, 256, 0.05, 3, "cpu"), Q.random_fp8_block(256, 256, 0, 0.05, 4, "cpu")]
    for w in cases:
        full = w.dequant()
        idx = torch.cat((torch.arange(128, 256), torch.arange(0, 128))) if w.n >= 256 else torch.arange(128)
        assert torch.equal(Q.take_out(w, idx).dequant(), full[idx])
        if isinstance(w, Q.Exl3Weight):
            # a K-slice of an EXL3 matrix is the matching slice of the factorised product: x_slice @ W_slice^T sums to x @ W^T
            x = torch.randn(3, w.k, generator=g)
            parts = sum(x[:, lo:lo + 128] @ Q.take_in(w, lo, lo + 128).dequant().t() for lo in range(0, w.k, 128))
            assert torch.allclose(parts, x @ full.t(), atol=1e-4)
        else:
            assert torch.equal(Q.take_in(w, 128, 256).dequant(), full[:, 128:256])
    with pytest.raises(ValueError):
        Q.take_out(cases[0], torch.arange(64))
    ex = Q.random_exl3(128, 128, 4, 4, 0.05, 5, "cpu")
    assert torch.equal(Q.take_experts(ex, 1, 3).dequant_expert(0), ex.dequant_expert(1))
