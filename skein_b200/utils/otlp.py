"""Optional OpenTelemetry trace export: request spans and step spans sent as OTLP/HTTP JSON to `SKEIN_OTLP_ENDPOINT`.

    SKEIN_OTLP_ENDPOINT=http://collector:4318     spans are POSTed to <endpoint>/v1/traces
    SKEIN_OTLP_SERVICE=skein                      resource attribute service.name (default "skein")

Nothing of this runs unless the endpoint is set. Spans are queued by the serving thread (two list appends per span) and
shipped by a background thread in batches, so a slow or absent collector never holds a step up: when the queue is full,
spans are dropped and counted. Only the standard library is used (urllib), the payload is the protobuf-JSON form of
`ExportTraceServiceRequest`.

Counterpart of the reference's optional OTLP layer (crates/skein_cli/src/output.rs:32-88) with its request and step
spans (crates/skein_runtime/src/observability/tracing_spans.rs:14,19).
"""
from __future__ import annotations

import json
import os
import queue
import random
import threading
import time
import urllib.request


def _attr(k, v):
    if isinstance(v, bool):
        return {"key": k, "value": {"boolValue": v}}
    if isinstance(v, int):
        return {"key": k, "value": {"intValue": str(v)}}
    if isinstance(v, float):
        return {"key": k, "value": {"doubleValue": v}}
    return {"key": k, "value": {"stringValue": str(v)}}


class SpanExporter:
    """Batches finished spans and POSTs them to <endpoint>/v1/traces."""

    def __init__(self, endpoint: str, service: str = "skein", rank: int = 0, max_queue: int = 4096, batch: int = 256,
                 flush_s: float = 1.0, timeout_s: float = 2.0):
        self.url = endpoint.rstrip("/") + "/v1/traces"
        self.resource = {"attributes": [_attr("service.name", service), _attr("skein.rank", rank)]}
        self.q: queue.Queue = queue.Queue(maxsize=max_queue)
        self.batch, self.flush_s, self.timeout_s = batch, flush_s, timeout_s
        self.dropped = 0
        self.sent = 0
        self.failed_posts = 0
        self._stop = threading.Event()
        self._rng = random.Random(os.getpid() ^ int(time.time()))
        self._t = threading.Thread(target=self._run, name="skein-otlp", daemon=True)
        self._t.start()

    # ---- producing side (serving thread) ----
    def new_trace_id(self) -> str:
        return "%032x" % self._rng.getrandbits(128)

    def new_span_id(self) -> str:
        return "%016x" % self._rng.getrandbits(64)

    def span(self, name: str, start_ns: int, end_ns: int, trace_id: str | None = None, parent: str | None = None,
             attrs: dict | None = None, error: str | None = None) -> str:
        """Queues one finished span; returns its span id."""
        sid = self.new_span_id()
        s = {"traceId": trace_id or self.new_trace_id(), "spanId": sid, "name": name, "kind": 1,
             "startTimeUnixNano": str(int(start_ns)), "endTimeUnixNano": str(int(end_ns)),
             "attributes": [_attr(k, v) for k, v in (attrs or {}).items()]}
        if parent:
            s["parentSpanId"] = parent
        if error:
            s["status"] = {"code": 2, "message": error}
        try:
            self.q.put_nowait(s)
        except queue.Full:
            self.dropped += 1
        return sid

    # ---- shipping side (background thread) ----
    def _post(self, spans) -> None:
        body = json.dumps({"resourceSpans": [{"resource": self.resource,
                                              "scopeSpans": [{"scope": {"name": "skein_b200"}, "spans": spans}]}]}).encode()
        req = urllib.request.Request(self.url, data=body, headers={"Content-Type": "application/json"}, method="POST")
        try:
            with urllib.request.urlopen(req, timeout=self.timeout_s) as r:
                r.read()
            self.sent += len(spans)
        except Exception:       # noqa: BLE001  (a collector that is down must not take the server with it)
            self.failed_posts += 1

    def _drain(self, block_s: float):
        spans = []
        try:
            spans.append(self.q.get(timeout=block_s))
            while len(spans) < self.batch:
                spans.append(self.q.get_nowait())
        except queue.Empty:
            pass
        return spans

    def _run(self) -> None:
        while not self._stop.is_set():
            spans = self._drain(self.flush_s)
            if spans:
                self._post(spans)

    def close(self, flush: bool = True) -> None:
        self._stop.set()
        self._t.join(timeout=self.timeout_s + self.flush_s + 1.0)
        while flush:
            spans = self._drain(0.0)
            if not spans:
                break
            self._post(spans)


_exporter = None


def exporter(rank: int = 0):
    """The process-wide exporter, or None when SKEIN_OTLP_ENDPOINT is not set."""
    global _exporter
    ep = os.environ.get("SKEIN_OTLP_ENDPOINT", "")
    if not ep:
        return None
    if _exporter is None:
        _exporter = SpanExporter(ep, os.environ.get("SKEIN_OTLP_SERVICE", "skein"), rank)
    return _exporter


def shutdown() -> None:
    global _exporter
    if _exporter is not None:
        _exporter.close()
        _exporter = None
