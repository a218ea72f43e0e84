"""Host-side guards that keep bad inputs away from the device (all run on CPU)."""
import ctypes
import json
import os
import struct

import pytest
import torch

from spark_engine_b200.config import tiny_hybrid
from spark_engine_b200.models.weights import init_weights
from spark_engine_b200.runtime import rt
from spark_engine_b200.serving.engine import LLMEngine
from spark_engine_b200.spec.decoder import SeqSpec, SpecDecoder


def test_decode_round_refuses_a_row_past_the_kv_region():
    cfg = tiny_hybrid()
    eng = LLMEngine(cfg, init_weights(cfg, seed=0), device="cpu", max_seqs=2, kv_tokens_per_seq=8)
    ids = list(range(1, 8))
    first = int(eng.model.greedy(eng.prefill(0, ids).unsqueeze(0))[0])
    nxt = eng.decode_round([0], [first])          # position 7 is the last row that fits
    with pytest.raises(RuntimeError, match="KV region"):
        eng.decode_round([0], nxt)
    assert eng.model.seqs[0].length == 8           # nothing was written by the refused round
    with pytest.raises(RuntimeError, match="KV region"):
        eng.generate([list(range(1, 7))], max_new=8)


def test_ep_row_layout_is_16_byte_aligned_for_every_hidden_size():
    from spark_engine_b200.ops import cuda as cu
    if not os.path.exists(cu.LIB_PATH):
        pytest.skip("kernel library not built")
    try:
        dll = ctypes.CDLL(cu.LIB_PATH)
    except OSError:
        pytest.skip("CUDA runtime library not loadable here")
    dll.spark_ep_row_bytes.argtypes, dll.spark_ep_row_bytes.restype = [ctypes.c_int], ctypes.c_int
    for H in (128, 256, 384, 512, 1024, 2048, 4096, 5120):
        rb = dll.spark_ep_row_bytes(H)
        assert rb % 16 == 0 and rb >= H + 4 * (H // 128) + 16
        assert (rb - 16 - H) % 16 == 0            # metadata offset = H + padded scale area


def _write_st(path, header: dict, payload: bytes):
    h = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + payload)


def test_safetensors_rejects_offsets_outside_the_file(tmp_path):
    good = tmp_path / "good.safetensors"
    _write_st(good, {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 16]}}, b"\0" * 16)
    st = rt().SafeTensors(str(good))
    assert st.names() == ["a"]
    cases = {
        "past_end": {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [0, 32]}},
        "reversed": {"a": {"dtype": "F32", "shape": [2, 2], "data_offsets": [16, 0]}},
        "size_mismatch": {"a": {"dtype": "F32", "shape": [3, 2], "data_offsets": [0, 16]}},
    }
    for name, hdr in cases.items():
        p = tmp_path / f"{name}.safetensors"
        _write_st(p, hdr, b"\0" * 16)
        with pytest.raises(Exception):
            rt().SafeTensors(str(p))


def test_online_calibration_reaches_the_cells_the_rate_policy_reads():
    cfg = tiny_hybrid()
    from spark_engine_b200.models.model import Model
    m = Model(cfg, init_weights(cfg, seed=0), n_slots=1, kv_tokens=256)
    conf = 0.83

    def drafter(seq, depth):                      # always wrong, always confident
        return [(seq.last_token + 1 + j) % cfg.vocab for j in range(depth)], [conf] * depth
    dec = SpecDecoder(m, drafter=drafter, depth=3, policy="all")
    s = dec.start(0, list(range(5, 25)))
    before = [s.table.prob(j, conf) for j in range(3)]
    for _ in range(6):
        dec.round([s])
    after = [s.table.prob(j, conf) for j in range(3)]
    assert all(a < b for a, b in zip(after, before)), (before, after)


def test_index_table_check_and_poison_fill(monkeypatch):
    """Debug modes: a table with an out-of-range entry raises before anything would be launched; poison fills floats with
    NaN and integers with 0x7f bytes.  Both are no-ops unless switched on."""
    import pytest
    import torch
    from spark_engine_b200.utils import debug as dbg
    t = torch.tensor([0, 3, -1, 7], dtype=torch.int32)
    dbg.check_index("off", t, 0, 4)                                   # switched off: nothing happens
    monkeypatch.setattr(dbg, "CHECK", True)
    dbg.check_index("pairs", t, 0, 8, allow=-1)
    dbg.check_index("pairs", t, 0, 4, allow=-1, count=2)              # only the first two entries count
    with pytest.raises(dbg.IndexTableError, match=r"\[-1, 7\]"):
        dbg.check_index("pairs", t, 0, 8)
    with pytest.raises(dbg.IndexTableError, match="valid range"):
        dbg.check_index("pairs", t, 0, 7, allow=-1)
    x, i = torch.zeros(4), torch.zeros(4, dtype=torch.int32)
    assert dbg.poison(x).eq(0).all()                                  # switched off
    monkeypatch.setattr(dbg, "POISON", True)
    assert torch.isnan(dbg.poison(x)).all()
    assert dbg.poison(i).eq(0x7F7F7F7F).all()


def test_batched_prefill_equals_per_sequence_prefill():
    """Several prompts of different lengths prefilled in shared forwards (one segment each, a row budget per forward) end
    with the same last-token logits and the same cache state as one prefill per sequence."""
    import torch
    from spark_engine_b200.config import EngineConfig, tiny_hybrid
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.serving.engine import LLMEngine
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (37, 9, 64)]
    one = LLMEngine(cfg, W, EngineConfig(cuda_graphs=False, prefill_chunk=16), device="cpu", max_seqs=3, kv_tokens_per_seq=128)
    ref = torch.stack([one.prefill(s, p) for s, p in enumerate(prompts)])
    many = LLMEngine(cfg, W, EngineConfig(cuda_graphs=False, prefill_chunk=48), device="cpu", max_seqs=3, kv_tokens_per_seq=128)
    got = many.prefill_many([0, 1, 2], prompts)
    assert torch.allclose(got, ref, atol=2e-4, rtol=1e-4)
    assert [many.model.seqs[s].length for s in range(3)] == [37, 9, 64]
    nxt = ref.argmax(-1).tolist()
    assert many.decode_round([0, 1, 2], nxt) == one.decode_round([0, 1, 2], nxt)


def test_row_invariance_probe_finds_the_first_layer_that_depends_on_the_batch():
    """The probe reports nothing on the CPU runner (rows are independent) and names the layer once one layer's output is
    made to depend on the number of rows in the forward."""
    import torch
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.utils.invariance import first_divergent_layer
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g).tolist() for n in (12, 9, 15)]
    make = lambda: Model(cfg, W, n_slots=3, kv_tokens=192)
    assert first_divergent_layer(make, prompts, probe=1, rows=2, atol=1e-5) is None

    def make_bad():
        m = Model(cfg, W, n_slots=3, kv_tokens=192)
        lw, mix, mlp = m.layers[2]
        real = mlp.forward

        def leaky(h, defer=False):                      # a "kernel" whose result depends on how many rows it was given
            out = real(h, defer)
            return out + 1e-3 * (h.shape[0] > 2) if isinstance(out, torch.Tensor) else out
        mlp.forward = leaky
        return m
    hit = first_divergent_layer(make_bad, prompts, probe=1, rows=2, atol=1e-5)
    assert hit is not None and hit[0] == 2 and hit[1] > 5e-4
