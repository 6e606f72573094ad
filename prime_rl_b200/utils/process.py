"""Child-process supervision for the launchers: start, monitor, and tear down whole process
trees (reference: src/prime_rl/utils/process.py:28-105, entrypoints/rl.py:373-398)."""

from __future__ import annotations

import os
import queue
import signal
import subprocess
import threading
import time
from pathlib import Path


def popen(cmd: list[str], env: dict[str, str], log_file: Path | None = None) -> subprocess.Popen:
    out = open(log_file, "w") if log_file is not None else None
    return subprocess.Popen(cmd, env=env, stdout=out, stderr=subprocess.STDOUT if out else None,
                            start_new_session=True)


def kill_tree(proc: subprocess.Popen, grace: float = 10.0) -> None:
    """SIGTERM then SIGKILL to the process group that ``popen`` created for this child."""
    if proc.poll() is not None:
        return
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        return
    t0 = time.monotonic()
    while proc.poll() is None and time.monotonic() - t0 < grace:
        time.sleep(0.1)
    if proc.poll() is None:
        try:
            os.killpg(proc.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass


class Supervisor:
    """Watches named children; the first non-zero exit is reported through ``errors``."""

    def __init__(self):
        self.children: dict[str, subprocess.Popen] = {}
        self.errors: queue.Queue = queue.Queue()
        self._threads: list[threading.Thread] = []

    def add(self, name: str, proc: subprocess.Popen) -> None:
        self.children[name] = proc
        t = threading.Thread(target=self._watch, args=(name, proc), daemon=True)
        t.start()
        self._threads.append(t)

    def _watch(self, name: str, proc: subprocess.Popen) -> None:
        rc = proc.wait()
        if rc != 0:
            self.errors.put((name, rc))

    def wait(self, required: list[str], poll: float = 0.5) -> tuple[str, int] | None:
        """Returns None when every ``required`` child exited with 0, or (name, rc) of the first failure."""
        while True:
            try:
                return self.errors.get(timeout=poll)
            except queue.Empty:
                pass
            if all(self.children[n].poll() == 0 for n in required):
                return None

    def shutdown(self) -> None:
        for proc in self.children.values():
            kill_tree(proc)
