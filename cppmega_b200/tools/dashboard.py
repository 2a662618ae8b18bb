"""Dashboard over the per-run metrics endpoints (stdlib only).

    python -m cppmega_b200.tools.dashboard --port 8470 --scan 8471-8490 [--host 127.0.0.1]

Every training run started with ``--monitor-port P`` serves ``/health /status /iterations /gpu /log``
(:mod:`cppmega_b200.utils.monitor`).  This tool scans a port range for such endpoints and serves

* ``/``              an HTML overview: one row per run (iteration, loss, grad norm, tokens/s, TFLOP/s/GPU, skipped or
                     non-finite iterations, up time) with a loss sparkline, plus the GPUs of the machine;
* ``/run/<port>``    one run in detail: loss and throughput curves (inline SVG), analytics (median step time after
                     warm-up, loss slope over the last window), the tail of its log;
* ``/api/runs``      the same data as JSON.

Counterpart of the reference's Flask dashboard that polls its per-run REST monitors on ports 8471+
(tools/dashboard/app.py:356-556); no web framework, no login layer, read-only.
"""
from __future__ import annotations

import argparse
import html
import json
import statistics
import sys
import urllib.request
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Dict, List, Optional, Sequence


def fetch(host: str, port: int, path: str, timeout: float = 0.5):
    try:
        with urllib.request.urlopen(f"http://{host}:{port}{path}", timeout=timeout) as r:
            return json.loads(r.read().decode())
    except Exception:
        return None


def scan(host: str, ports: Sequence[int]) -> List[int]:
    return [p for p in ports if (fetch(host, p, "/health") or {}).get("ok")]


def analytics(iterations: List[Dict], warmup: int = 3, window: int = 50) -> Dict:
    """Median step time / throughput after warm-up and the loss trend over the last ``window`` records."""
    recs = [r for r in iterations if isinstance(r.get("loss"), (int, float))]
    out: Dict = {"records": len(recs)}
    body = recs[warmup:] if len(recs) > warmup else recs
    for key in ("elapsed_ms", "step_ms", "tokens_per_s", "tflops_per_gpu"):
        vals = [r[key] for r in body if isinstance(r.get(key), (int, float))]
        if vals:
            out["median_" + key] = statistics.median(vals)
    tail = recs[-window:]
    if len(tail) >= 2:
        xs = list(range(len(tail)))
        ys = [r["loss"] for r in tail]
        mx, my = sum(xs) / len(xs), sum(ys) / len(ys)
        den = sum((x - mx) ** 2 for x in xs)
        out["loss_slope_per_iteration"] = sum((x - mx) * (y - my) for x, y in zip(xs, ys)) / den if den else 0.0
    out["non_finite"] = sum(1 for r in iterations if any(isinstance(v, float) and v != v for v in r.values()))
    return out


def run_info(host: str, port: int) -> Dict:
    status = fetch(host, port, "/status") or {}
    its = fetch(host, port, "/iterations") or []
    return {"port": port, "reachable": bool(status), "status": status, "iterations": its, "analytics": analytics(its)}


def sparkline(values: Sequence[float], width: int = 220, height: int = 36, color: str = "#1f77b4") -> str:
    vals = [v for v in values if isinstance(v, (int, float)) and v == v]
    if len(vals) < 2:
        return ""
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    pts = " ".join(f"{i * (width - 2) / (len(vals) - 1) + 1:.1f},{height - 2 - (v - lo) / span * (height - 4):.1f}"
                   for i, v in enumerate(vals))
    return (f'<svg width="{width}" height="{height}" viewBox="0 0 {width} {height}">'
            f'<polyline fill="none" stroke="{color}" stroke-width="1.5" points="{pts}"/></svg>')


_CSS = ("body{font-family:system-ui,sans-serif;margin:1.5em;color:#222}table{border-collapse:collapse}"
        "td,th{border:1px solid #ccc;padding:4px 10px;text-align:right}th{background:#f2f2f2}td.l{text-align:left}"
        ".bad{color:#b00}pre{background:#f7f7f7;padding:8px;overflow:auto}")


def _fmt(v, nd=3):
    if isinstance(v, float):
        return f"{v:.{nd}f}" if abs(v) < 1e5 else f"{v:.3e}"
    return "" if v is None else html.escape(str(v))


def render_index(runs: List[Dict], gpus: List[Dict]) -> str:
    rows = []
    for r in runs:
        last = r["status"].get("last", {})
        a = r["analytics"]
        bad = r["status"].get("nan_iterations", 0)
        rows.append(
            f'<tr><td class="l"><a href="/run/{r["port"]}">{r["port"]}</a></td><td>{_fmt(last.get("iteration", last.get("step")))}</td>'
            f'<td>{_fmt(last.get("loss"))}</td><td>{_fmt(last.get("grad_norm"))}</td><td>{_fmt(a.get("median_tokens_per_s"), 0)}</td>'
            f'<td>{_fmt(a.get("median_tflops_per_gpu"), 1)}</td><td class="{"bad" if bad else ""}">{bad}</td>'
            f'<td>{_fmt(r["status"].get("uptime_s"), 0)}</td><td class="l">{sparkline([x.get("loss") for x in r["iterations"]])}</td></tr>')
    gpu_rows = "".join(
        f'<tr><td>{_fmt(g.get("index"))}</td><td class="l">{_fmt(g.get("name"))}</td><td>{_fmt(g.get("utilization.gpu"))}</td>'
        f'<td>{_fmt(g.get("memory.used"))} / {_fmt(g.get("memory.total"))}</td><td>{_fmt(g.get("power.draw"))}</td>'
        f'<td>{_fmt(g.get("clocks.sm"))}</td><td>{_fmt(g.get("temperature.gpu"))}</td></tr>' for g in gpus)
    return (f"<html><head><title>cppmega_b200 runs</title><style>{_CSS}</style><meta http-equiv='refresh' content='5'></head><body>"
            f"<h2>Training runs ({len(runs)})</h2><table><tr><th>port</th><th>iteration</th><th>loss</th><th>grad norm</th>"
            f"<th>tokens/s (median)</th><th>TFLOP/s/GPU</th><th>non-finite</th><th>up (s)</th><th>loss</th></tr>{''.join(rows)}</table>"
            f"<h2>GPUs</h2><table><tr><th>#</th><th>name</th><th>util %</th><th>memory MiB</th><th>power W</th><th>SM MHz</th>"
            f"<th>temp C</th></tr>{gpu_rows}</table></body></html>")


def render_run(r: Dict, log_tail: List[str]) -> str:
    its = r["iterations"]
    a = "".join(f"<tr><td class='l'>{html.escape(k)}</td><td>{_fmt(v, 4)}</td></tr>" for k, v in r["analytics"].items())
    return (f"<html><head><title>run {r['port']}</title><style>{_CSS}</style></head><body><p><a href='/'>all runs</a></p>"
            f"<h2>Run on port {r['port']}</h2><h3>loss</h3>{sparkline([x.get('loss') for x in its], 720, 160)}"
            f"<h3>tokens/s</h3>{sparkline([x.get('tokens_per_s') for x in its], 720, 120, '#2ca02c')}"
            f"<h3>analytics</h3><table>{a}</table><h3>log (tail)</h3><pre>{html.escape(chr(10).join(log_tail[-40:]))}</pre></body></html>")


class Dashboard:
    def __init__(self, host: str, ports: Sequence[int], listen_port: int, listen_host: str = "127.0.0.1"):
        self.host, self.ports = host, list(ports)
        self.listen = (listen_host, listen_port)
        self._httpd: Optional[ThreadingHTTPServer] = None

    def runs(self) -> List[Dict]:
        return [run_info(self.host, p) for p in scan(self.host, self.ports)]

    def handle(self, path: str):
        """(status, content type, body) for a GET of ``path``."""
        path = path.split("?")[0]
        if path == "/api/runs":
            return 200, "application/json", json.dumps(self.runs())
        if path == "/":
            runs = self.runs()
            gpus = (fetch(self.host, runs[0]["port"], "/gpu") if runs else None) or []
            return 200, "text/html", render_index(runs, gpus)
        if path.startswith("/run/"):
            try:
                port = int(path[len("/run/"):])
            except ValueError:
                return 404, "text/plain", "bad port"
            if port not in self.ports:
                return 404, "text/plain", "port outside the scanned range"
            return 200, "text/html", render_run(run_info(self.host, port), fetch(self.host, port, "/log") or [])
        return 404, "text/plain", "unknown path"

    def serve(self, block: bool = True):
        dash = self

        class Handler(BaseHTTPRequestHandler):
            def do_GET(self):          # noqa: N802
                code, ctype, body = dash.handle(self.path)
                data = body.encode()
                self.send_response(code)
                self.send_header("Content-Type", ctype + "; charset=utf-8")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def log_message(self, *a):
                pass

        self._httpd = ThreadingHTTPServer(self.listen, Handler)
        self.listen = self._httpd.server_address
        if block:
            self._httpd.serve_forever()
        return self

    def stop(self):
        if self._httpd is not None:
            self._httpd.shutdown()
            self._httpd.server_close()


def _parse_ports(spec: str) -> List[int]:
    out: List[int] = []
    for part in spec.split(","):
        if "-" in part:
            a, b = part.split("-", 1)
            out.extend(range(int(a), int(b) + 1))
        elif part:
            out.append(int(part))
    return out


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--port", type=int, default=8470, help="port this dashboard listens on")
    ap.add_argument("--listen-host", default="127.0.0.1")
    ap.add_argument("--host", default="127.0.0.1", help="host whose monitor ports are scanned")
    ap.add_argument("--scan", default="8471-8490", help="monitor ports: a-b and/or comma-separated")
    ap.add_argument("--once", action="store_true", help="print /api/runs as JSON and exit")
    ns = ap.parse_args(argv)
    dash = Dashboard(ns.host, _parse_ports(ns.scan), ns.port, ns.listen_host)
    if ns.once:
        print(json.dumps(dash.runs()))
        return 0
    print(f"dashboard on http://{ns.listen_host}:{ns.port}/ scanning {ns.host}:{ns.scan}", flush=True)
    dash.serve()
    return 0


if __name__ == "__main__":
    sys.exit(main())
