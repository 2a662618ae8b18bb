"""Metrics REST endpoint (stdlib only): ``/health``, ``/status``, ``/iterations``, ``/gpu``, ``/log``.

Same role as the reference's per-run monitor polled by its dashboard (scripts/gpu_monitor.py:1-17,
tools/dashboard/app.py:356-556).  The trainer publishes one record per logged iteration.
"""
from __future__ import annotations

import json
import subprocess
import threading
import time
from collections import deque
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Deque, Dict, Optional


class MetricsServer:
    def __init__(self, port: int, host: str = "127.0.0.1", history: int = 2048):
        self.port, self.host = port, host
        self.records: Deque[Dict] = deque(maxlen=history)
        self.log_lines: Deque[str] = deque(maxlen=history)
        self.started = time.time()
        self._httpd: Optional[ThreadingHTTPServer] = None
        self._thread: Optional[threading.Thread] = None
        self._lock = threading.Lock()

    def publish(self, rec: Dict) -> None:
        with self._lock:
            self.records.append(dict(rec, wall=time.time()))
            self.log_lines.append(json.dumps(rec))

    def _payload(self, path: str):
        with self._lock:
            recs = list(self.records)
            lines = list(self.log_lines)
        if path == "/health":
            return {"ok": True, "uptime_s": time.time() - self.started}
        if path == "/iterations":
            return recs
        if path == "/status":
            last = recs[-1] if recs else {}
            nan = sum(1 for r in recs if any(isinstance(v, float) and v != v for v in r.values()))
            return {"iterations": len(recs), "last": last, "nan_iterations": nan, "uptime_s": time.time() - self.started}
        if path == "/log":
            return lines[-200:]
        if path == "/gpu":
            return gpu_snapshot()
        return None

    def start(self) -> "MetricsServer":
        server = self

        class Handler(BaseHTTPRequestHandler):
            def do_GET(self):          # noqa: N802
                body = server._payload(self.path.split("?")[0])
                code = 200 if body is not None else 404
                data = json.dumps(body if body is not None else {"error": "unknown path"}).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def log_message(self, *a):
                pass

        self._httpd = ThreadingHTTPServer((self.host, self.port), Handler)
        self.port = self._httpd.server_address[1]
        self._thread = threading.Thread(target=self._httpd.serve_forever, daemon=True, name="cppmega-monitor")
        self._thread.start()
        return self

    def stop(self) -> None:
        if self._httpd is not None:
            self._httpd.shutdown()
            self._httpd.server_close()


def gpu_snapshot() -> list:
    """Read-only nvidia-smi query (clocks, power, memory, utilisation)."""
    q = "index,name,utilization.gpu,memory.used,memory.total,power.draw,clocks.sm,temperature.gpu"
    try:
        out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits"], capture_output=True,
                             text=True, timeout=5).stdout
    except Exception:
        return []
    keys = q.split(",")
    return [dict(zip(keys, [x.strip() for x in line.split(",")])) for line in out.strip().splitlines() if line.strip()]
