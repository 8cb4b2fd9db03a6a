"""Host-side step watchdog (fail-stop + auto-resume model of the reference's launcher:
`modal_train.py:115` restarts the whole job, `--auto_resume` picks the newest checkpoint).

A daemon thread watches the time since the last `beat()`.  When a step takes longer than
`factor` x the median of recent steps (and at least `min_seconds`), it dumps every Python thread's
stack to stderr, calls `on_timeout` and, unless told otherwise, exits the process with a non-zero
code so that the launcher restarts the job.  Nothing here touches a GPU.
"""
from __future__ import annotations

import faulthandler
import os
import statistics
import sys
import threading
import time


class StepWatchdog:
    def __init__(self, factor: float = 20.0, min_seconds: float = 120.0, window: int = 50, on_timeout=None,
                 exit_code: int | None = 75, poll_seconds: float = 1.0):
        self.factor, self.min_seconds, self.window = factor, min_seconds, window
        self.on_timeout, self.exit_code, self.poll = on_timeout, exit_code, poll_seconds
        self._durations: list[float] = []
        self._last = None
        self._stop = threading.Event()
        self._thread = None
        self.fired = False
        self._lock = threading.Lock()

    def start(self) -> "StepWatchdog":
        self._last = time.monotonic()
        self._thread = threading.Thread(target=self._run, name="step-watchdog", daemon=True)
        self._thread.start()
        return self

    def beat(self) -> None:
        now = time.monotonic()
        with self._lock:
            if self._last is not None:
                self._durations.append(now - self._last)
                del self._durations[:-self.window]
            self._last = now

    def limit(self) -> float:
        with self._lock:
            if len(self._durations) < 3:
                return float("inf") if self.min_seconds <= 0 else max(self.min_seconds, 10 * self.min_seconds)
            return max(self.min_seconds, self.factor * statistics.median(self._durations))

    def _run(self) -> None:
        while not self._stop.wait(self.poll):
            with self._lock:
                last = self._last
            if last is None:
                continue
            if time.monotonic() - last > self.limit():
                self.fired = True
                print(f"[watchdog] step exceeded {self.limit():.1f}s; dumping stacks", file=sys.stderr, flush=True)
                try:
                    faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
                except Exception:
                    pass
                if self.on_timeout is not None:
                    try:
                        self.on_timeout()
                    except Exception:
                        pass
                if self.exit_code is not None:
                    os._exit(self.exit_code)
                return

    def stop(self) -> None:
        self._stop.set()
