"""Multimodal plumbing and the vision tower (CPU)."""
import numpy as np
import pytest
import torch

from spark_engine_b200.multimodal import canvas as C
from spark_engine_b200.multimodal.vision import VisionConfig, VisionTower, init_vision_weights, patchify


def _img(h, w, seed):
    return np.random.default_rng(seed).integers(0, 256, (h, w, 3), dtype=np.uint8)


def test_canvas_placeholders_and_validation(tmp_path):
    cfg = VisionConfig(depth=1, width=32, heads=2, mlp=64, patch=4, merge=2, out_hidden=48)
    seg = lambda it: cfg.rows_for(it["height"] if isinstance(it, dict) else it.height,
                                  it["width"] if isinstance(it, dict) else it.width)
    a = C.write_canvas([_img(30, 50, 1)], 32, 32, str(tmp_path))
    b = C.write_canvas([_img(64, 64, 2), _img(64, 64, 3)], 32, 32, str(tmp_path))      # two frames
    PH = 7
    ids = C.expand_placeholders([1, 2, PH, 3, PH, PH, 4], PH, [a, b], seg)
    n = cfg.rows_for(32, 32)
    assert len(ids) == 4 + 3 * n and a["segments"] == [[2, n, 0]] and b["segments"] == [[3 + n, n, 0], [3 + 2 * n, n, 1]]
    assert all(C.is_salted(t) for t in ids[2: 2 + n])
    # same media -> same ids (prefix reuse hits), different media -> different ids
    a2 = C.write_canvas([_img(30, 50, 1)], 32, 32, str(tmp_path))
    assert C.expand_placeholders([PH], PH, [a2], seg) == ids[2: 2 + n]
    assert ids[2: 2 + n] != ids[3 + n: 3 + 2 * n]
    items = C.parse_items([a, b], seg)
    C.validate(ids, 100, items)
    bad = list(ids)
    bad[2] = 5
    with pytest.raises(ValueError):
        C.validate(bad, 100, items)
    with pytest.raises(ValueError):
        C.validate(ids + [C.MM_BASE + 5], 100, items)
    with pytest.raises(ValueError):
        C.parse_items([dict(a, height=31)], seg)


def test_vision_tower_rows_and_injection(tmp_path):
    for rope in (True, False):
        cfg = VisionConfig(depth=2, width=32, heads=2, mlp=64, patch=4, merge=2, out_hidden=48, rope2d=rope, max_side=16)
        tower = VisionTower(cfg, init_vision_weights(cfg, 1))
        item = C.parse_items([dict(C.write_canvas([_img(40, 40, 5)], 32, 32, str(tmp_path)),
                                   segments=[[3, cfg.rows_for(32, 32), 0]])], lambda it: cfg.rows_for(it.height, it.width))[0]
        rows = tower.encode(C.load_frame(item, 0))
        assert rows.shape == (cfg.rows_for(32, 32), 48) and torch.isfinite(rows).all()
        # a different image gives different rows; the same image the same rows
        assert torch.equal(rows, tower.encode(C.load_frame(item, 0)))
    n = cfg.rows_for(32, 32)
    enc = lambda it, f: tower.encode(C.load_frame(it, f))
    ids = torch.tensor([1, 2, 3] + C.salted_ids(b"x", n) + [4, 5])
    # chunked prefill: the segment straddles two chunks of 8 positions
    emb = torch.zeros(len(ids), 48)
    for start in range(0, len(ids), 8):
        part = C.chunk_rows([item], start, 8, enc)
        C.inject_rows(emb[start: start + 8], ids[start: start + 8], part)
    assert torch.equal(emb[3: 3 + n], rows) and float(emb[:3].abs().sum()) == 0 and float(emb[3 + n:].abs().sum()) == 0


def test_patchify_layout():
    img = torch.arange(8 * 8 * 3, dtype=torch.uint8).view(8, 8, 3)
    p = patchify(img, 4)
    assert p.shape == (4, 48)
    # patch 1 = rows 0..3, columns 4..7; channel-major inside the patch
    want = (img[0:4, 4:8].float() / 127.5 - 1.0).permute(2, 0, 1).reshape(-1)
    assert torch.allclose(p[1], want)


def test_model_consumes_injected_rows():
    """A prompt with a media segment: the model's output equals a run whose embedding table holds the media rows at
    ordinary ids (so the injection is exactly 'these rows instead of embeddings')."""
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    media = torch.randn(5, cfg.hidden, generator=g) * 0.02
    ids = [3, 9] + C.salted_ids(b"img", 5) + [11, 4]
    plan = make_plan([(0, ids, 0)])
    plan.mm_rows = [(2, media)]
    out = Model(cfg, W, n_slots=1, kv_tokens=64).forward(plan)
    W2 = dict(W)
    W2["embed"] = W["embed"].clone()
    W2["embed"][100:105] = media
    ref = Model(cfg, W2, n_slots=1, kv_tokens=64).forward(make_plan([(0, [3, 9, 100, 101, 102, 103, 104, 11, 4], 0)]))
    assert torch.allclose(out, ref, atol=1e-5)
