"""Liveness heartbeat: one HTTP GET per finished step to a monitoring URL (for example a
BetterStack heartbeat); failures are logged and never raised
(reference: src/prime_rl/utils/heartbeat.py)."""

from __future__ import annotations

import threading
import urllib.request

from .logger import get_logger


class Heartbeat:
    def __init__(self, url: str, timeout: float = 5.0):
        self.url, self.timeout = url, timeout

    def _send(self) -> None:
        try:
            urllib.request.urlopen(self.url, timeout=self.timeout).read()
        except Exception as e:
            get_logger().warning(f"heartbeat to {self.url} failed: {e}")

    def beat(self, blocking: bool = False) -> None:
        if blocking:
            self._send()
        else:
            threading.Thread(target=self._send, daemon=True).start()
