"""A small HTTP front end for inference sessions: the headless counterpart of the reference's web page
(www/index.html loads the checkpoint and pumps a few tokens per animation frame; here a client pumps
chunks over HTTP). Standard library only.

    python -m burn_dragon_b200 serve --checkpoint runs/latest --port 8080

    GET  /                                -> a prompt box (engine/www/index.html) that streams from /generate
    GET  /health                          -> {"status": "ok", "model": {...}, "device": "cuda:0"}
    GET  /metrics                         -> Prometheus text format: requests, generated tokens, busy seconds
    POST /generate  {"prompt": "ROMEO:", "max_tokens": 200, "temperature": 0.8, "top_k": 40,
                     "greedy": false, "seed": 1, "stream": true, "chunk_tokens": 4}
         stream=false -> {"text": "...", "tokens": 200}
         stream=true  -> application/x-ndjson, one {"text": "..."} line per chunk, then {"done": true, "tokens": n}
    With `--pool-slots N` concurrent single-prompt requests are decoded together (continuous batching).
    "prompt" may be a list of equally long strings: the streams are decoded together (one recurrent
    state each) and "text" becomes a list.

Requests are served one at a time (a lock around the session): the GPU decode step is already
batched over the streams of one request.
"""
from __future__ import annotations

import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

from .session import InferenceSession

MAX_BODY = 1 << 20


def make_server(session: InferenceSession, host: str = "127.0.0.1", port: int = 8080, pool_slots: int = 0,
                pool_settings=None) -> ThreadingHTTPServer:
    """`pool_slots > 0` adds continuous batching (engine/stream_pool.py): single-prompt requests whose
    sampling settings are the pool's (`pool_settings`: temperature, top_k, greedy, seed; default greedy
    off, temperature 1) share one batched decode step; anything else takes the exclusive path."""
    lock = threading.Lock()
    stats = {"requests": 0, "errors": 0, "tokens": 0, "busy_s": 0.0, "pooled": 0}
    scheduler = None
    if pool_slots > 0:
        from . import generation as GEN
        from .stream_pool import PoolScheduler, StreamPool
        ps = pool_settings or GEN.GenerationSettings(None, 1.0, None, seed=0)
        scheduler = PoolScheduler(StreamPool(session.model, pool_slots, ps, session.device), session.tokenizer, lock)

    def pool_matches(req) -> bool:
        ps = scheduler.pool.settings
        return (isinstance(req.get("prompt"), str) and not req.get("context_window")
                and float(req.get("temperature", ps.temperature)) == float(ps.temperature)
                and (req.get("top_k", ps.top_k) or None) == (ps.top_k or None)
                and bool(req.get("greedy", ps.greedy)) == bool(ps.greedy) and req.get("seed") is None)

    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):  # quiet by default; errors still reach the client
            pass

        def _json(self, code: int, obj) -> None:
            body = (json.dumps(obj) + "\n").encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path in ("/", "/index.html"):
                from pathlib import Path
                body = (Path(__file__).resolve().parent / "www" / "index.html").read_bytes()
                self.send_response(200)
                self.send_header("Content-Type", "text/html; charset=utf-8")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return
            if self.path == "/metrics":
                body = ("# TYPE bdh_requests_total counter\n"
                        f"bdh_requests_total {stats['requests']}\n"
                        "# TYPE bdh_request_errors_total counter\n"
                        f"bdh_request_errors_total {stats['errors']}\n"
                        "# TYPE bdh_generated_tokens_total counter\n"
                        f"bdh_generated_tokens_total {stats['tokens']}\n"
                        "# TYPE bdh_generate_busy_seconds_total counter\n"
                        f"bdh_generate_busy_seconds_total {stats['busy_s']:.6f}\n"
                        "# TYPE bdh_pooled_requests_total counter\n"
                        f"bdh_pooled_requests_total {stats['pooled']}\n"
                        "# TYPE bdh_pool_slots_in_use gauge\n"
                        f"bdh_pool_slots_in_use {0 if scheduler is None else scheduler.pool.slots - scheduler.pool.free_slots()}\n"
                        ).encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return
            if self.path != "/health":
                return self._json(404, {"error": "unknown path"})
            c = session.model.config
            self._json(200, {"status": "ok", "device": str(session.device), "block_size": session.block_size,
                             "model": {"n_layer": c.n_layer, "n_embd": c.n_embd, "n_head": c.n_head,
                                       "n_latent_per_head": c.latent_per_head, "vocab_size": c.vocab_size,
                                       "rotary_embedding": c.rotary_embedding}})

        def _chunk(self, data: bytes) -> None:
            self.wfile.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
            self.wfile.flush()

        def do_POST(self):
            if self.path != "/generate":
                return self._json(404, {"error": "unknown path"})
            try:
                n = int(self.headers.get("Content-Length", "0"))
                if n <= 0 or n > MAX_BODY:
                    raise ValueError("missing or oversized body")
                req = json.loads(self.rfile.read(n))
                prompt = req["prompt"]
                if not (isinstance(prompt, str) or (isinstance(prompt, list) and all(isinstance(p, str) for p in prompt))):
                    raise ValueError("prompt must be a string or a list of strings")
                kw = dict(max_tokens=int(req.get("max_tokens", 128)), temperature=float(req.get("temperature", 1.0)),
                          top_k=(int(req["top_k"]) if req.get("top_k") is not None else None),
                          greedy=bool(req.get("greedy", False)),
                          seed=(int(req["seed"]) if req.get("seed") is not None else None),
                          context_window=(int(req["context_window"]) if req.get("context_window") else None))
                chunk_tokens = max(1, int(req.get("chunk_tokens", 4)))
                stream = bool(req.get("stream", False))
            except (KeyError, ValueError, TypeError, json.JSONDecodeError) as e:
                stats["errors"] += 1
                return self._json(400, {"error": str(e)})
            many = isinstance(prompt, list)
            if scheduler is not None and pool_matches(req):
                return self._pooled(prompt, kw["max_tokens"], stream)
            with lock:
                t0 = time.perf_counter()
                stats["requests"] += 1
                try:
                    return self._generate(prompt, kw, chunk_tokens, stream, many)
                finally:
                    stats["busy_s"] += time.perf_counter() - t0
                    stats["tokens"] += session.generated * (len(prompt) if many else 1)

        def _pooled(self, prompt, max_tokens, stream):
            """The request joins the shared decode step; text arrives piece by piece from the scheduler."""
            t0 = time.perf_counter()
            stats["requests"] += 1
            stats["pooled"] += 1
            try:
                ids = session.tokenizer.encode(prompt)
                if not ids:
                    raise ValueError("prompt must contain at least one token")
                h = scheduler.submit(ids, max_tokens)
            except (ValueError, KeyError, TimeoutError) as e:
                stats["errors"] += 1
                return self._json(503 if isinstance(e, TimeoutError) else 400, {"error": str(e)})
            try:
                if not stream:
                    text = ""
                    while True:
                        piece = h.queue.get()
                        if piece is None:
                            break
                        text += piece
                    return self._json(200, {"text": text, "tokens": h.tokens})
                self.send_response(200)
                self.send_header("Content-Type", "application/x-ndjson")
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()
                try:
                    while True:
                        piece = h.queue.get()
                        if piece is None:
                            break
                        self._chunk((json.dumps({"text": piece}) + "\n").encode())
                    self._chunk((json.dumps({"done": True, "tokens": h.tokens}) + "\n").encode())
                    self.wfile.write(b"0\r\n\r\n")
                except (BrokenPipeError, ConnectionResetError):
                    h.remaining = 0          # the client went away: the stream leaves the pool at the next step
            finally:
                stats["busy_s"] += time.perf_counter() - t0
                stats["tokens"] += h.tokens

        def _generate(self, prompt, kw, chunk_tokens, stream, many):
            try:
                session.start_stream(prompt, **kw)
            except (ValueError, KeyError) as e:
                stats["errors"] += 1
                return self._json(400, {"error": str(e)})
            if not stream:
                text = ["" for _ in prompt] if many else ""
                while not session.done:
                    piece = session.next_chunk(chunk_tokens)
                    text = [a + b for a, b in zip(text, piece)] if many else text + piece
                return self._json(200, {"text": text, "tokens": session.generated})
            self.send_response(200)
            self.send_header("Content-Type", "application/x-ndjson")
            self.send_header("Transfer-Encoding", "chunked")
            self.end_headers()
            try:
                while not session.done:
                    piece = session.next_chunk(chunk_tokens)
                    if piece if not many else any(piece):
                        self._chunk((json.dumps({"text": piece}) + "\n").encode())
                self._chunk((json.dumps({"done": True, "tokens": session.generated}) + "\n").encode())
                self.wfile.write(b"0\r\n\r\n")
            except (BrokenPipeError, ConnectionResetError):
                pass        # the client went away: drop the stream, keep serving

    srv = ThreadingHTTPServer((host, port), Handler)
    srv.scheduler = scheduler
    return srv


def serve(session: InferenceSession, host: str = "127.0.0.1", port: int = 8080,
          ready: Optional[threading.Event] = None, pool_slots: int = 0, pool_settings=None) -> None:
    srv = make_server(session, host, port, pool_slots, pool_settings)
    if threading.current_thread() is threading.main_thread():
        import signal
        # SIGTERM (what a process supervisor sends) ends the accept loop; streams in flight finish
        signal.signal(signal.SIGTERM, lambda *_: threading.Thread(target=srv.shutdown, daemon=True).start())
    if ready is not None:
        ready.set()
    try:
        srv.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        if srv.scheduler is not None:
            srv.scheduler.stop()
        srv.server_close()
