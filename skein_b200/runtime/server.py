"""HTTP front end: POST /v1/completions (JSON or SSE token stream), GET /metrics, GET /healthz.

    POST /v1/completions   {"prompt": str | [int], "max_tokens": int, "stream": bool}
        stream=false -> {"id", "tokens", "text", "finish_reason"}
        stream=true  -> text/event-stream with `event: token` / data {"id", "token", "text", "is_final"}
        429 when admission rejects the request, 400 on a malformed body
    GET /metrics           Prometheus text of the engine's instruments

One driver thread owns the engine and steps it whenever work exists; request handlers talk to it
through a thread-safe inbox and receive token events on per-request asyncio queues. The same wire
protocol and driver/handler split as the reference's axum server (crates/skein_runtime/src/server/
forward.rs:57-82,237-420,437-592; lifecycle.rs:22-124), but the engine behind it is the multi-GPU one
rather than a single-process executor.
"""
from __future__ import annotations

import asyncio
import json
import queue
import threading
import time

from .engine import Engine, TokenEvent
from .tokenizer import Tokenizer


class EngineDriver:
    """Runs `engine.step()` on its own thread. Thread-safe `submit` returns an event queue."""

    def __init__(self, engine: Engine, idle_sleep_s: float = 0.001):
        self.engine = engine
        self._inbox: "queue.Queue" = queue.Queue()
        self._streams: dict[int, "queue.Queue[TokenEvent]"] = {}
        self._stop = threading.Event()
        self._idle_sleep = idle_sleep_s
        self._thread = threading.Thread(target=self._run, name="skein-engine-driver", daemon=True)
        self.draining = False

    def start(self):
        self._thread.start()
        return self

    def stop(self, timeout: float = 5.0):
        self._stop.set()
        self._thread.join(timeout)

    def submit(self, prompt_ids, max_new_tokens):
        """Returns (request_id, decision_kind, reason, event_queue or None). Blocks until the driver has decided."""
        reply: "queue.Queue" = queue.Queue(maxsize=1)
        self._inbox.put((prompt_ids, max_new_tokens, reply))
        return reply.get()

    @property
    def inflight(self) -> int:
        return len(self._streams)

    def drain(self, timeout_s: float) -> bool:
        """Stop admitting, wait for in-flight requests to finish. True if drained in time."""
        self.draining = True
        t0 = time.monotonic()
        while self._streams and time.monotonic() - t0 < timeout_s:
            time.sleep(0.005)
        ok = not self._streams
        if not ok:
            self.draining = False     # timeout: keep serving on the old state
        return ok

    def _run(self):
        eng = self.engine
        while not self._stop.is_set():
            try:
                while True:
                    prompt, max_new, reply = self._inbox.get_nowait()
                    if self.draining:
                        reply.put((0, "reject", "draining", None))
                        continue
                    try:
                        rid, d = eng.submit(prompt, max_new)
                    except ValueError as e:
                        reply.put((0, "reject", str(e), None))
                        continue
                    if d.kind == "reject":
                        reply.put((rid, "reject", d.reason, None))
                    else:
                        q: "queue.Queue[TokenEvent]" = queue.Queue()
                        self._streams[rid] = q
                        reply.put((rid, d.kind, d.reason, q))
            except queue.Empty:
                pass
            if eng.idle:
                time.sleep(self._idle_sleep)
                continue
            events = eng.step()
            if not events:
                time.sleep(self._idle_sleep)
            for ev in events:
                q = self._streams.get(ev.request_id)
                if q is not None:
                    q.put(ev)
                    if ev.is_final:
                        del self._streams[ev.request_id]


def build_app(driver: EngineDriver, tokenizer: Tokenizer):
    from aiohttp import web

    async def next_event(q):
        loop = asyncio.get_running_loop()
        return await loop.run_in_executor(None, q.get)

    async def completions(request: "web.Request"):
        try:
            body = await request.json()
            prompt = body["prompt"]
            max_tokens = int(body.get("max_tokens", 32))
            stream = bool(body.get("stream", False))
            ids = tokenizer.encode(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
            if not ids or max_tokens < 1:
                raise ValueError("empty prompt or max_tokens < 1")
        except (KeyError, ValueError, TypeError, json.JSONDecodeError) as e:
            return web.json_response({"error": {"kind": "bad_request", "message": str(e)}}, status=400)
        loop = asyncio.get_running_loop()
        rid, kind, reason, q = await loop.run_in_executor(None, driver.submit, ids, max_tokens)
        if kind == "reject":
            return web.json_response({"error": {"kind": "rejected", "message": reason}}, status=429)
        if stream:
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
            await resp.prepare(request)
            while True:
                ev = await next_event(q)
                payload = {"id": rid, "token": ev.token, "text": tokenizer.decode([ev.token]) if ev.token >= 0 else "",
                           "is_final": ev.is_final}
                if ev.error:
                    payload["error"] = ev.error
                await resp.write(f"event: token\ndata: {json.dumps(payload)}\n\n".encode())
                if ev.is_final:
                    break
            await resp.write_eof()
            return resp
        toks, err = [], None
        while True:
            ev = await next_event(q)
            if ev.error:
                err = ev.error
            elif ev.token >= 0:
                toks.append(ev.token)
            if ev.is_final:
                break
        if err:
            return web.json_response({"id": rid, "error": {"kind": "step_failed", "message": err}}, status=503)
        return web.json_response({"id": rid, "tokens": toks, "text": tokenizer.decode(toks), "finish_reason": "length"})

    async def metrics(_):
        return web.Response(text=driver.engine.metrics.render(), content_type="text/plain")

    async def healthz(_):
        return web.json_response({"ok": True, "inflight": driver.inflight, "draining": driver.draining})

    app = web.Application()
    app.router.add_post("/v1/completions", completions)
    app.router.add_get("/metrics", metrics)
    app.router.add_get("/healthz", healthz)
    return app


def serve(engine: Engine, tokenizer: Tokenizer, host: str = "0.0.0.0", port: int = 8080):
    """Blocking: start the driver and the HTTP server."""
    from aiohttp import web

    driver = EngineDriver(engine).start()
    try:
        web.run_app(build_app(driver, tokenizer), host=host, port=port, print=None)
    finally:
        driver.stop()


def serve_metrics_only(metrics, port: int = 9090):
    """Stand-alone /metrics exporter on its own port (the reference's prometheus_port, default 9090)."""
    import http.server

    class H(http.server.BaseHTTPRequestHandler):
        def do_GET(self):
            body = metrics.render().encode()
            self.send_response(200)
            self.send_header("Content-Type", "text/plain; version=0.0.4")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def log_message(self, *a):
            pass

    srv = http.server.ThreadingHTTPServer(("0.0.0.0", port), H)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv
