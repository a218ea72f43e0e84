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


# ------------------------------------------------------------------------------ media pre-processing + serving
def _png_bytes(h, w, seed):
    import io
    from PIL import Image
    buf = io.BytesIO()
    Image.fromarray(_img(h, w, seed)).save(buf, format="PNG")
    return buf.getvalue()


def _data_url(raw, mime="image/png"):
    import base64
    return f"data:{mime};base64," + base64.b64encode(raw).decode()


def test_media_decode_resize_frames_and_chat_walk(tmp_path):
    import http.server
    import io
    import threading
    from PIL import Image
    from spark_engine_b200.multimodal import media as M
    raw = _png_bytes(30, 50, 1)
    (fr,) = M.decode_frames(_data_url(raw))
    assert fr.shape == (30, 50, 3) and fr.dtype == np.uint8 and np.array_equal(fr, _img(30, 50, 1))
    p = tmp_path / "a.png"
    p.write_bytes(raw)
    assert np.array_equal(M.decode_frames(str(p))[0], fr) and np.array_equal(M.decode_frames("file://" + str(p))[0], fr)
    # resize keeps the aspect ratio, pads with zeros, smooths (a constant image stays constant)
    flat = np.full((100, 200, 3), 77, np.uint8)
    c = M.fit_smooth(flat, 32, 32)
    assert c.shape == (32, 32, 3) and (c[:16] == 77).all() and (c[16:] == 0).all()
    # animated image: frames sampled evenly
    gif = io.BytesIO()
    frames = [Image.fromarray(np.full((8, 8, 3), 40 * i, np.uint8)) for i in range(6)]
    frames[0].save(gif, format="GIF", save_all=True, append_images=frames[1:], duration=50)
    got = M.decode_frames(gif.getvalue(), max_frames=3)
    assert len(got) == 3 and got[0].mean() < got[1].mean() < got[2].mean()
    # damaged / oversize / network sources are refused with ValueError
    for bad in (_data_url(raw[:40]), "data:image/png;base64,", str(tmp_path / "missing.png"), 5):
        with pytest.raises(ValueError):
            M.decode_frames(bad)
    with pytest.raises(ValueError, match="switched off"):
        M.decode_frames("http://127.0.0.1:9/x.png")

    class H(http.server.BaseHTTPRequestHandler):
        def do_GET(self):
            self.send_response(200)
            self.send_header("Content-Length", str(len(raw)))
            self.end_headers()
            self.wfile.write(raw)

        def log_message(self, *a):
            pass
    srv = http.server.HTTPServer(("127.0.0.1", 0), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    try:
        assert np.array_equal(M.decode_frames(f"http://127.0.0.1:{srv.server_port}/x.png", allow_fetch=True)[0], fr)
    finally:
        srv.shutdown()
    # the chat walk: media parts become placeholders in order, text is kept
    msgs = [{"role": "system", "content": "s"},
            {"role": "user", "content": [{"type": "text", "text": "look: "}, {"type": "image_url", "image_url": {"url": "U1"}},
                                         {"type": "text", "text": " and "}, {"type": "video_url", "video_url": {"url": "U2"}}]}]
    flat_msgs, media = M.split_chat_content(msgs, "<|image|>")
    assert flat_msgs[1]["content"] == "look: <|image|> and <|image|>" and media == [("image", "U1"), ("video", "U2")]
    with pytest.raises(ValueError):
        M.split_chat_content([{"role": "user", "content": [{"type": "audio", "audio": "x"}]}], "<|image|>")
    # canvases + prompt expansion: one run per frame, salted ids, deterministic per content
    items = M.build_items([("image", _data_url(raw)), ("video", gif.getvalue())], 16, 16, str(tmp_path), video_frames=2)
    assert [it["frames"] for it in items] == [1, 2]
    ids = M.expand_prompt([1, 258, 2, 258, 3], 258, items, lambda it: 4)
    assert len(ids) == 3 + 3 * 4 and items[0]["segments"] == [[1, 4, 0]] and items[1]["segments"] == [[6, 4, 0], [10, 4, 1]]
    with pytest.raises(ValueError):
        M.expand_prompt([1, 258], 258, M.build_items([("image", _data_url(raw))] * 2, 16, 16, str(tmp_path)), lambda it: 4)


def test_chat_request_with_an_image_is_served_through_the_vision_tower(tmp_path):
    """HTTP chat request with an image part -> decoded, fitted on a canvas, salted placeholder ids -> the engine encodes
    the canvas while it prefills (the run straddles prefill chunks) and the served tokens equal a direct greedy decode
    of the same ids with the same rows injected; the same request again reuses the prefix; a text-only server refuses."""
    import json
    import threading
    import urllib.error
    import urllib.request
    from spark_engine_b200.config import EngineConfig, tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights
    from spark_engine_b200.multimodal import media as M
    from spark_engine_b200.serving.openai_server import serve
    from spark_engine_b200.serving.tokenizer import ByteTokenizer
    from spark_engine_b200.serving.worker import EngineServer
    cfg = tiny_hybrid()
    cfg.mtp_layers = 1
    W = init_weights(cfg, seed=0)
    vcfg = VisionConfig(depth=1, width=32, heads=2, mlp=64, patch=4, merge=2, out_hidden=cfg.hidden, max_side=16)
    vW = init_vision_weights(vcfg, 3)
    sock = str(tmp_path / "e.sock")
    es = EngineServer(cfg, W, EngineConfig(max_seqs=2, kv_tokens=2048, prefill_chunk=16, spec="mtp", spec_depth=2),
                      vision=(vcfg, vW))
    ready = threading.Event()
    th = threading.Thread(target=es.serve_forever, args=(sock,), kwargs={"ready_cb": ready.set}, daemon=True)
    th.start()
    assert ready.wait(30)
    rows = vcfg.rows_for(32, 32)                                   # 16 rows per frame: straddles the 16-token chunks
    media = {"height": 32, "width": 32, "rows": rows, "dir": str(tmp_path)}
    srv, app = serve(sock, "127.0.0.1", 0, "tiny", None, media)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{srv.server_port}/v1/chat/completions"
    body = {"messages": [{"role": "user", "content": [{"type": "text", "text": "what is this? "},
                                                       {"type": "image_url", "image_url": {"url": _data_url(_png_bytes(40, 56, 9))}}]}],
            "max_tokens": 6}

    def post(u, b):
        req = urllib.request.Request(u, json.dumps(b).encode(), {"Content-Type": "application/json"})
        return json.loads(urllib.request.urlopen(req, timeout=120).read())
    try:
        r1 = post(url, body)
        # the same prompt built directly: ids, canvases, rows, plain greedy decoding with the rows injected
        ids, items = app.chat_prompt(body)
        assert sum(C.is_salted(t) for t in ids) == rows and items[0]["frames"] == 1
        tower = VisionTower(vcfg, vW)
        parsed = C.parse_items(items, lambda it: rows)
        m = Model(cfg, W, n_slots=1, kv_tokens=512)
        plan = make_plan([(0, ids, 0)], all_logits=False)
        plan.mm_rows = C.chunk_rows(parsed, 0, len(ids), lambda it, f: tower.encode(C.load_frame(it, f)))
        tok = int(m.forward(plan).argmax(-1)[0])
        want = [tok]
        for k in range(5):
            tok = int(m.forward(make_plan([(0, [tok], len(ids) + k)])).argmax(-1)[0])
            want.append(tok)
        text = ByteTokenizer().decode(want)
        assert r1["choices"][0]["message"]["content"] == text
        assert es.totals["media_frames"] == 1                      # encoded once although two chunks hold parts of the run
        # follow-up turn over the engine socket: prompt + answer + new tokens continues the finished store, so the media
        # rows are neither re-encoded nor re-prefilled
        import socket as sk
        from spark_engine_b200.serving import protocol as proto
        c = sk.socket(sk.AF_UNIX, sk.SOCK_STREAM)
        c.connect(sock)
        buf, done = proto.LineBuffer(), None
        c.sendall(proto.encode({"id": 900, "prompt_ids": ids + want + [5, 6, 7], "max_new": 3, "mm": items}))
        while done is None:
            for msg in buf.feed(c.recv(1 << 16)):
                if msg.get("done") or "error" in msg:
                    done = msg
        c.close()
        assert "error" not in done and done["prefix_hit_tokens"] >= len(ids) and es.totals["media_frames"] == 1
        # placeholders without their canvases, or canvases at the wrong positions, are refused before anything runs
        for bad_msg in ({"id": 901, "prompt_ids": ids, "max_new": 2},
                        {"id": 902, "prompt_ids": [1] + ids, "max_new": 2, "mm": items}):
            c = sk.socket(sk.AF_UNIX, sk.SOCK_STREAM)
            c.connect(sock)
            c.sendall(proto.encode(bad_msg))
            got = None
            buf = proto.LineBuffer()
            while got is None:
                for msg in buf.feed(c.recv(1 << 16)):
                    if "error" in msg or msg.get("done"):
                        got = msg
            c.close()
            assert "error" in got, got
        # a different image is a different prompt (different salted ids)
        body2 = json.loads(json.dumps(body))
        body2["messages"][0]["content"][1]["image_url"]["url"] = _data_url(_png_bytes(40, 56, 10))
        ids2, _ = app.chat_prompt(body2)
        assert ids2 != ids and [t for t in ids2 if not C.is_salted(t)] == [t for t in ids if not C.is_salted(t)]
        # malformed media is a 400, and a server without a tower refuses media parts
        bad = json.loads(json.dumps(body))
        bad["messages"][0]["content"][1]["image_url"]["url"] = "data:image/png;base64,AAAA"
        with pytest.raises(urllib.error.HTTPError) as e:
            post(url, bad)
        assert e.value.code == 400
        app.media = None
        with pytest.raises(urllib.error.HTTPError):
            post(url, body)
    finally:
        srv.shutdown()
        es.shutdown = True
        th.join(10)


@pytest.mark.gpu
def test_vision_tower_and_row_injection_on_the_device(tmp_path):
    """The tower in bf16 on the GPU (patch 4 and patch 14: widths that are not multiples of 8) against the fp32 CPU tower,
    and a prompt with injected media rows through the device model against the CPU runner."""
    from spark_engine_b200.config import tiny_hybrid
    from spark_engine_b200.models.model import Model
    from spark_engine_b200.models.plan import make_plan
    from spark_engine_b200.models.weights import init_weights, to_device
    cfg = tiny_hybrid()
    W = init_weights(cfg, seed=0)
    for vc in (VisionConfig(depth=1, width=32, heads=2, mlp=64, patch=4, merge=2, out_hidden=cfg.hidden, max_side=16),
               VisionConfig(depth=2, width=64, heads=4, mlp=128, patch=14, merge=2, out_hidden=cfg.hidden, max_side=16)):
        vW = init_vision_weights(vc, 3)
        side = vc.patch * vc.merge * 4
        item = C.parse_items([dict(C.write_canvas([_img(side, side, 1)], side, side, str(tmp_path)),
                                   segments=[[3, vc.rows_for(side, side), 0]])], lambda it: vc.rows_for(it.height, it.width))[0]
        rc = VisionTower(vc, vW).encode(C.load_frame(item, 0))
        rg = VisionTower(vc, vW, device="cuda", dtype=torch.bfloat16).encode(C.load_frame(item, 0)).float().cpu()
        assert rg.shape == rc.shape and ((rg - rc).norm() / rc.norm()).item() < 3e-2
    n = rc.shape[0]
    ids = [1, 2, 3] + C.salted_ids(b"x", n) + [4, 5]
    outs = []
    for dev in ("cpu", "cuda"):
        m = Model(cfg, W if dev == "cpu" else to_device(W, dev), device=dev,
                  dtype=torch.float32 if dev == "cpu" else torch.bfloat16, n_slots=1, kv_tokens=256)
        plan = make_plan([(0, ids, 0)], device=dev)
        plan.mm_rows = [(3, rc)]
        outs.append(m.forward(plan).float().cpu())
    assert torch.isfinite(outs[1]).all()
    assert ((outs[1] - outs[0]).norm() / outs[0].norm()).item() < 5e-2
