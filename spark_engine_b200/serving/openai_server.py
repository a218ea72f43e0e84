"""OpenAI-compatible HTTP front end.  Talks newline-JSON to the engine over a Unix socket.

Endpoints: POST /v1/chat/completions (SSE streaming, usage, stop strings, tool calls, reasoning split),
POST /v1/completions, GET /v1/models, POST /tokenize, POST /detokenize, GET /health, /ping, /version, /metrics.
Cancels the engine request when the client disconnects.  Reference: engine-rs/serve/openai_server.py:2-21,79-163,
166-272 (Engine socket client), 353-528 (TextStreamIncr, ToolCalls), 886-1073 (handlers).
"""
from __future__ import annotations

import argparse
import json
import queue
import re
import socket
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional

from . import protocol as proto
from .metrics import Metrics
from .tokenizer import IncrementalDetok, load_tokenizer

VERSION = "0.1.0"


class EngineClient:
    """Persistent connection to the engine; a reader thread routes reply lines to per-request queues."""

    def __init__(self, path: str, connect_timeout: float = 60.0):
        self.path = path
        self.lock = threading.Lock()
        self.queues: Dict[int, "queue.Queue[dict]"] = {}
        self.next_id = 1
        deadline = time.time() + connect_timeout
        while True:
            try:
                self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
                self.sock.connect(path)
                break
            except OSError:
                if time.time() > deadline:
                    raise
                time.sleep(0.1)
        self.alive = True
        threading.Thread(target=self._reader, daemon=True).start()

    def _reader(self):
        buf = proto.LineBuffer()
        while True:
            try:
                data = self.sock.recv(1 << 16)
            except OSError:
                data = b""
            if not data:
                self.alive = False
                with self.lock:
                    for q in self.queues.values():
                        q.put({"error": "engine connection lost"})
                return
            for msg in buf.feed(data):
                q = self.queues.get(msg.get("id"))
                if q is not None:
                    q.put(msg)

    def _send(self, msg: dict):
        with self.lock:
            self.sock.sendall(proto.encode(msg))

    def generate(self, prompt_ids: List[int], max_new: int, stop_ids: List[int], temperature: float, seed: int, mm=None):
        with self.lock:
            rid = self.next_id
            self.next_id += 1
            q = self.queues[rid] = queue.Queue()
        msg = {"id": rid, "prompt_ids": prompt_ids, "max_new": max_new, "stop_token_ids": stop_ids,
               "temperature": temperature, "seed": seed}
        if mm:
            msg["mm"] = mm                      # canvas files + the prompt positions of their salted placeholder runs
        self._send(msg)
        return rid, q

    def cancel(self, rid: int):
        self._send({"cancel": rid})

    def release(self, rid: int):
        with self.lock:
            self.queues.pop(rid, None)

    def stats(self, timeout: float = 5.0) -> dict:
        with self.lock:
            rid = self.next_id
            self.next_id += 1
            q = self.queues[rid] = queue.Queue()
        self._send({"id": rid, "stats": True})
        try:
            return q.get(timeout=timeout).get("stats", {})
        except queue.Empty:
            return {}
        finally:
            self.release(rid)


class StopStrings:
    """Holds back text that could be the beginning of a stop string; reports when one is hit."""

    def __init__(self, stops: List[str]):
        self.stops = [s for s in stops if s]
        self.hold = ""

    def feed(self, text: str):
        self.hold += text
        for s in self.stops:
            i = self.hold.find(s)
            if i >= 0:
                out, self.hold = self.hold[:i], ""
                return out, True
        keep = 0
        for s in self.stops:
            for k in range(min(len(s) - 1, len(self.hold)), 0, -1):
                if self.hold.endswith(s[:k]):
                    keep = max(keep, k)
                    break
        out = self.hold[: len(self.hold) - keep]
        self.hold = self.hold[len(self.hold) - keep:]
        return out, False

    def flush(self) -> str:
        out, self.hold = self.hold, ""
        return out


class ReasoningSplit:
    """Routes text between <think> ... </think> to `reasoning_content`, the rest to `content`."""

    def __init__(self, enabled: bool = True):
        self.enabled, self.in_think, self.buf = enabled, False, ""

    def feed(self, text: str):
        if not self.enabled:
            return "", text
        self.buf += text
        reasoning = content = ""
        while self.buf:
            tag = "</think>" if self.in_think else "<think>"
            i = self.buf.find(tag)
            if i >= 0:
                seg, self.buf = self.buf[:i], self.buf[i + len(tag):]
                if self.in_think:
                    reasoning += seg
                else:
                    content += seg
                self.in_think = not self.in_think
                continue
            keep = next((k for k in range(min(len(tag) - 1, len(self.buf)), 0, -1) if self.buf.endswith(tag[:k])), 0)
            seg, self.buf = self.buf[: len(self.buf) - keep], self.buf[len(self.buf) - keep:]
            if self.in_think:
                reasoning += seg
            else:
                content += seg
            break
        return reasoning, content


_TOOL_RE = re.compile(r"<tool_call>\s*(\{.*?\})\s*</tool_call>", re.S)


def parse_tool_calls(text: str):
    """(content without the tool-call blocks, [OpenAI tool_calls])."""
    calls = []
    for m in _TOOL_RE.finditer(text):
        try:
            obj = json.loads(m.group(1))
        except json.JSONDecodeError:
            continue
        calls.append({"id": "call_" + uuid.uuid4().hex[:16], "type": "function",
                      "function": {"name": obj.get("name", ""), "arguments": json.dumps(obj.get("arguments", {}))}})
    return _TOOL_RE.sub("", text).strip() if calls else text, calls


class App:
    def __init__(self, engine: EngineClient, tokenizer, model_name: str, max_new_default: int = 256, media: Optional[dict] = None):
        self.engine, self.tok, self.model_name, self.max_new_default = engine, tokenizer, model_name, max_new_default
        self.metrics = Metrics(model_name)
        # media: {"height", "width", "rows" (placeholder ids per frame), "dir", "allow_fetch", "video_frames"} when the
        # engine has a vision tower; None = text only (media parts are refused)
        self.media = media

    def chat_prompt(self, body: dict):
        """(prompt ids, mm items) of a chat request: media parts are decoded, fitted onto canvases and replaced by runs
        of salted placeholder ids (multimodal/media.py, multimodal/canvas.py)."""
        messages = body.get("messages", [])
        if not any(isinstance(m.get("content"), list) and any(isinstance(p, dict) and p.get("type", "text") != "text"
                                                              for p in m["content"]) for m in messages):
            return self.tok.apply_chat_template(messages, True, body.get("tools")), None
        from ..multimodal import media as M
        from .tokenizer import IMAGE_PLACEHOLDER
        if self.media is None:
            raise ValueError("this server has no vision tower: media parts are not accepted")
        tid = getattr(self.tok, "image_token_id", None)
        if tid is None:
            raise ValueError("the tokenizer has no media placeholder token")
        flat, sources = M.split_chat_content(messages, getattr(self.tok, "image_token", IMAGE_PLACEHOLDER))
        md = self.media
        items = M.build_items(sources, md["height"], md["width"], md.get("dir", "/dev/shm"), md.get("allow_fetch", False),
                              md.get("video_frames", 4))
        ids = self.tok.apply_chat_template(flat, True, body.get("tools"))
        return M.expand_prompt(list(ids), tid, items, lambda it: md["rows"]), items

    def run(self, prompt_ids: List[int], body: dict, chat: bool, write_event=None, disconnected=None, mm=None) -> dict:
        max_new = int(body.get("max_tokens") or body.get("max_completion_tokens") or self.max_new_default)
        stops = body.get("stop") or []
        stops = [stops] if isinstance(stops, str) else list(stops)
        eos = getattr(self.tok, "eos_token_id", None)
        t0 = time.time()
        rid, q = self.engine.generate(prompt_ids, max_new, [eos] if eos is not None else [], float(body.get("temperature", 0.0) or 0.0),
                                      int(body.get("seed", 0) or 0), mm=mm)
        detok, ss, rs = IncrementalDetok(self.tok), StopStrings(stops), ReasoningSplit(chat)
        content, reasoning, itls, last_t, done, finish = "", "", [], None, None, "length"
        try:
            while True:
                try:
                    msg = q.get(timeout=0.5)
                except queue.Empty:
                    if disconnected and disconnected():
                        self.engine.cancel(rid)
                        finish = "cancelled"
                        break
                    continue
                if "error" in msg:
                    raise RuntimeError(msg["error"])
                if "delta" in msg:
                    now = time.time()
                    if last_t is not None:
                        itls.append((now - last_t) / max(len(msg["delta"]), 1))
                    last_t = now
                    text, hit = ss.feed(detok.feed([t for t in msg["delta"] if t != eos]))
                    r, c = rs.feed(text)
                    reasoning += r
                    content += c
                    if write_event and (r or c):
                        write_event(r, c)
                    if hit:
                        self.engine.cancel(rid)
                        finish = "stop"
                if msg.get("done"):
                    done = msg
                    if finish != "stop":
                        finish = {"stop": "stop", "length": "length", "cancelled": finish}.get(msg.get("finish_reason"), "stop")
                        r, c = rs.feed(ss.flush())
                        reasoning += r
                        content += c
                        if write_event and (r or c):
                            write_event(r, c)
                    break
        finally:
            self.engine.release(rid)
        done = done or {"token_ids": [], "finish_reason": finish}
        self.metrics.finish(dict(done, finish_reason=finish), time.time() - t0, itls)
        usage = {"prompt_tokens": len(prompt_ids), "completion_tokens": len(done.get("token_ids", [])),
                 "total_tokens": len(prompt_ids) + len(done.get("token_ids", []))}
        return {"content": content, "reasoning": reasoning, "finish": finish, "usage": usage, "engine": done}


def make_handler(app: App):
    class H(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            pass

        def _json(self, code, obj):
            raw = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(raw)))
            self.end_headers()
            self.wfile.write(raw)

        def _body(self):
            n = int(self.headers.get("Content-Length", "0") or 0)
            return json.loads(self.rfile.read(n) or b"{}")

        def do_GET(self):
            if self.path in ("/health", "/ping"):
                return self._json(200 if app.engine.alive else 503, {"status": "ok" if app.engine.alive else "engine down"})
            if self.path == "/version":
                return self._json(200, {"version": VERSION})
            if self.path == "/v1/models":
                return self._json(200, {"object": "list", "data": [{"id": app.model_name, "object": "model", "owned_by": "spark_engine_b200"}]})
            if self.path == "/metrics":
                raw = app.metrics.render(app.engine.stats()).encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(raw)))
                self.end_headers()
                return self.wfile.write(raw)
            self._json(404, {"error": "not found"})

        def do_POST(self):
            try:
                body = self._body()
                if self.path == "/tokenize":
                    ids = app.tok.encode(body.get("prompt", ""))
                    return self._json(200, {"tokens": ids, "count": len(ids)})
                if self.path == "/detokenize":
                    return self._json(200, {"prompt": app.tok.decode(body.get("tokens", []))})
                if self.path == "/v1/chat/completions":
                    ids, mm = app.chat_prompt(body)
                    return self._complete(ids, body, True, mm)
                if self.path == "/v1/completions":
                    p = body.get("prompt", "")
                    ids = p if isinstance(p, list) and p and isinstance(p[0], int) else app.tok.encode(p if isinstance(p, str) else "".join(p))
                    return self._complete(list(ids), body, False)
                self._json(404, {"error": "not found"})
            except (BrokenPipeError, ConnectionResetError):
                pass
            except Exception as e:   # noqa: BLE001
                try:
                    self._json(400, {"error": {"message": str(e), "type": "invalid_request_error"}})
                except Exception:
                    pass

        def _complete(self, ids, body, chat, mm=None):
            cid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
            created = int(time.time())
            obj = "chat.completion" if chat else "text_completion"
            if not body.get("stream"):
                r = app.run(ids, body, chat, mm=mm)
                if chat:
                    text, calls = parse_tool_calls(r["content"])
                    msg = {"role": "assistant", "content": text}
                    if r["reasoning"]:
                        msg["reasoning_content"] = r["reasoning"]
                    if calls:
                        msg["tool_calls"] = calls
                    choice = {"index": 0, "message": msg, "finish_reason": "tool_calls" if calls else r["finish"]}
                else:
                    choice = {"index": 0, "text": r["content"], "finish_reason": r["finish"]}
                return self._json(200, {"id": cid, "object": obj, "created": created, "model": app.model_name,
                                        "choices": [choice], "usage": r["usage"]})
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Transfer-Encoding", "chunked")
            self.end_headers()
            gone = {"v": False}

            def chunk(data: str):
                raw = ("data: " + data + "\n\n").encode()
                try:
                    self.wfile.write(hex(len(raw))[2:].encode() + b"\r\n" + raw + b"\r\n")
                    self.wfile.flush()
                except (BrokenPipeError, ConnectionResetError, OSError):
                    gone["v"] = True

            def ev(reasoning, content):
                if chat:
                    d = {}
                    if reasoning:
                        d["reasoning_content"] = reasoning
                    if content:
                        d["content"] = content
                    choice = {"index": 0, "delta": d, "finish_reason": None}
                else:
                    choice = {"index": 0, "text": content, "finish_reason": None}
                chunk(json.dumps({"id": cid, "object": obj + ".chunk", "created": created, "model": app.model_name, "choices": [choice]}))
            if chat:
                chunk(json.dumps({"id": cid, "object": obj + ".chunk", "created": created, "model": app.model_name,
                                  "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}))
            r = app.run(ids, body, chat, ev, lambda: gone["v"], mm=mm)
            last = {"index": 0, "finish_reason": r["finish"]}
            last["delta" if chat else "text"] = {} if chat else ""
            final = {"id": cid, "object": obj + ".chunk", "created": created, "model": app.model_name, "choices": [last]}
            if (body.get("stream_options") or {}).get("include_usage"):
                final["usage"] = r["usage"]
            chunk(json.dumps(final))
            chunk("[DONE]")
            try:
                self.wfile.write(b"0\r\n\r\n")
            except OSError:
                pass
    return H


def serve(socket_path: str, host: str, port: int, model_name: str, tokenizer_path: Optional[str] = None,
          media: Optional[dict] = None):
    app = App(EngineClient(socket_path), load_tokenizer(tokenizer_path), model_name, media=media)
    srv = ThreadingHTTPServer((host, port), make_handler(app))
    srv.daemon_threads = True
    return srv, app


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--socket", default="/tmp/spark-b200.sock")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--model-name", default="spark")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--media-canvas", type=int, default=0, help="side of the canvas media frames are fitted onto (0 = text only)")
    ap.add_argument("--media-rows", type=int, default=0, help="placeholder ids per frame (rows the vision tower returns)")
    ap.add_argument("--media-dir", default="/dev/shm")
    ap.add_argument("--allow-media-fetch", action="store_true")
    a = ap.parse_args()
    media = None
    if a.media_canvas > 0 and a.media_rows > 0:
        media = {"height": a.media_canvas, "width": a.media_canvas, "rows": a.media_rows, "dir": a.media_dir,
                 "allow_fetch": a.allow_media_fetch}
    srv, _ = serve(a.socket, a.host, a.port, a.model_name, a.tokenizer, media)
    print(f"[front] listening on {a.host}:{a.port}", flush=True)
    srv.serve_forever()


if __name__ == "__main__":
    main()
