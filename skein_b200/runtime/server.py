"""HTTP front end: POST /v1/completions (JSON or SSE token stream), GET /metrics, GET /healthz.

    POST /v1/completions   {"prompt": str | [int], "max_tokens": int, "stream": bool,
                            "temperature": float, "top_k": int, "top_p": float, "seed": int}   (sampling optional)
        stream=false -> {"id", "tokens", "text", "finish_reason"}   ("stop": the model's end-of-sequence token, else "length")
        stream=true  -> text/event-stream with `event: token` / data {"id", "token", "text", "is_final"[, "finish_reason"]}
        429 when admission rejects the request, 400 on a malformed body
    GET /metrics           Prometheus text of the engine's instruments
    POST /admin/hotswap    {"artifact": path} (only with hot swap enabled): verify, drain, mount on every rank

One driver thread owns the engine and steps it whenever work exists; request handlers talk to it
through a thread-safe inbox and receive token events on per-request asyncio queues. The same wire
protocol and driver/handler split as the reference's axum server (crates/skein_runtime/src/server/
forward.rs:57-82,237-420,437-592; lifecycle.rs:22-124), but the engine behind it is the multi-GPU one
rather than a single-process executor.
"""
from __future__ import annotations

import asyncio
import json
import threading

from .driver import EngineDriver
from .engine import Engine, SamplingParams
from .tokenizer import IncrementalDecoder, Tokenizer

__all__ = ["EngineDriver", "build_app", "serve", "serve_metrics_only"]


def build_app(driver: EngineDriver, tokenizer: Tokenizer, hotswap=None, artifacts_root=None):
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
            vocab = driver.engine.cfg_vocab
            if any(t < 0 or t >= vocab for t in ids):
                raise ValueError(f"prompt token ids must be in [0, {vocab})")
            sampling = None
            if float(body.get("temperature", 0.0)) > 0.0:
                sampling = SamplingParams(temperature=float(body["temperature"]), top_k=int(body.get("top_k", 0)),
                                          top_p=float(body.get("top_p", 1.0)), seed=int(body.get("seed", 0)))
                if not (0.0 < sampling.top_p <= 1.0) or sampling.top_k < 0:
                    raise ValueError("top_p must be in (0, 1] and top_k >= 0")
        except (KeyError, ValueError, TypeError, json.JSONDecodeError) as e:
            return web.json_response({"error": {"kind": "bad_request", "message": str(e)}}, status=400)
        loop = asyncio.get_running_loop()
        rid, kind, reason, q = await loop.run_in_executor(None, driver.submit, ids, max_tokens, sampling)
        if kind == "reject":
            return web.json_response({"error": {"kind": "rejected", "message": reason}}, status=429)
        if stream:
            resp = web.StreamResponse(headers={"Content-Type": "text/event-stream", "Cache-Control": "no-cache"})
            await resp.prepare(request)
            pieces = IncrementalDecoder(tokenizer)
            while True:
                ev = await next_event(q)
                payload = {"id": rid, "token": ev.token, "text": pieces.push(ev.token) if ev.token >= 0 else "",
                           "is_final": ev.is_final}
                if ev.error:
                    payload["error"] = ev.error
                elif ev.is_final:
                    eos = driver.engine.cfg.eos_token
                    payload["finish_reason"] = "stop" if (eos >= 0 and ev.token == eos) else "length"
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
        eos = driver.engine.cfg.eos_token
        reason = "stop" if (eos >= 0 and toks and toks[-1] == eos) else "length"
        return web.json_response({"id": rid, "tokens": toks, "text": tokenizer.decode(toks), "finish_reason": reason})

    async def metrics(_):
        return web.Response(text=driver.engine.metrics.render(), content_type="text/plain")

    async def healthz(_):
        return web.json_response({"ok": True, "inflight": driver.inflight, "draining": driver.draining})

    async def admin_hotswap(request: "web.Request"):
        from .hotswap import HotSwapError
        try:
            path = (await request.json())["artifact"]
        except (KeyError, TypeError, json.JSONDecodeError) as e:
            return web.json_response({"error": {"kind": "bad_request", "message": str(e)}}, status=400)
        loop = asyncio.get_running_loop()
        try:
            new = await loop.run_in_executor(None, hotswap.swap, path, artifacts_root)
        except (HotSwapError, OSError, ValueError) as e:
            return web.json_response({"error": {"kind": "hotswap_failed", "message": str(e)}}, status=409)
        return web.json_response({"mounted": str(new.path)})

    app = web.Application()
    if hotswap is not None:
        app.router.add_post("/admin/hotswap", admin_hotswap)
    app.router.add_post("/v1/completions", completions)
    app.router.add_get("/metrics", metrics)
    app.router.add_get("/healthz", healthz)
    return app


def serve(engine: Engine, tokenizer: Tokenizer, host: str = "0.0.0.0", port: int = 8080, mounted=None,
          enable_hot_swap: bool = False, artifacts_root=None):
    """Blocking: start the driver and the HTTP server. With `enable_hot_swap`, POST /admin/hotswap replaces the
    weights of `mounted` (an Artifact) by those of another artifact with the same shapes."""
    from aiohttp import web

    driver = EngineDriver(engine).start()
    hs = None
    if enable_hot_swap and mounted is not None:
        from .hotswap import HotSwap
        hs = HotSwap(driver, mounted)
    try:
        web.run_app(build_app(driver, tokenizer, hs, artifacts_root), host=host, port=port, print=None)
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
