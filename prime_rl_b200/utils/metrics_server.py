"""Prometheus text endpoint of the trainer: ``GET /metrics`` with the latest step's gauges
(step, loss, throughput, MFU, grad norm, peak memory, last-step timestamp) and ``GET /health``
(reference: src/prime_rl/utils/metrics_server.py). Runs in a daemon thread on the master rank."""

from __future__ import annotations

import http.server
import threading
import time


class MetricsServer:
    def __init__(self, port: int, host: str = "0.0.0.0", prefix: str = "trainer"):
        self.host, self.port, self.prefix = host, port, prefix
        self.values: dict[str, float] = {}
        self.lock = threading.Lock()
        self.httpd: http.server.ThreadingHTTPServer | None = None

    def update(self, metrics: dict, step: int | None = None) -> None:
        with self.lock:
            for k, v in metrics.items():
                if isinstance(v, (int, float)):
                    self.values[k] = float(v)
            if step is not None:
                self.values["step"] = float(step)
            self.values["last_step_timestamp_seconds"] = time.time()

    def render(self) -> str:
        lines = []
        with self.lock:
            for k, v in sorted(self.values.items()):
                name = f"{self.prefix}_{k}".replace("/", "_").replace(".", "_").replace("-", "_")
                lines.append(f"# TYPE {name} gauge")
                lines.append(f"{name} {v}")
        return "\n".join(lines) + "\n"

    def start(self) -> "MetricsServer":
        outer = self

        class Handler(http.server.BaseHTTPRequestHandler):
            def do_GET(self):
                if self.path.startswith("/metrics"):
                    body, ctype = outer.render().encode(), "text/plain; version=0.0.4"
                elif self.path.startswith("/health"):
                    body, ctype = b'{"status": "ok"}', "application/json"
                else:
                    self.send_error(404)
                    return
                self.send_response(200)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def log_message(self, *a):
                pass

        self.httpd = http.server.ThreadingHTTPServer((self.host, self.port), Handler)
        self.port = self.httpd.server_address[1]
        threading.Thread(target=self.httpd.serve_forever, daemon=True, name="metrics-server").start()
        return self

    def stop(self) -> None:
        if self.httpd is not None:
            self.httpd.shutdown()
            self.httpd.server_close()
            self.httpd = None
