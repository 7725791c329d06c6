"""One metric logger behind a queue for all roles (parity: torchtune/dev/rl/workers/metric_logger.py:12-30)."""
from __future__ import annotations

import queue
from typing import Any, Dict


class MetricLoggerWorker:
    def __init__(self, logger, inbox=None):
        self.logger = logger
        self.inbox = inbox if inbox is not None else queue.Queue()

    def log_dict(self, payload: Dict[str, Any], step: int) -> None:
        """Called by any role (any thread / process): enqueue, never block on the backend."""
        self.inbox.put((dict(payload), int(step)))

    def drain(self) -> int:
        n = 0
        while True:
            try:
                payload, step = self.inbox.get_nowait()
            except queue.Empty:
                return n
            self.logger.log_dict(payload, step=step)
            n += 1

    def run(self, stop_event) -> None:
        while not stop_event.is_set():
            if not self.drain():
                stop_event.wait(0.1)
        self.drain()

    def close(self) -> None:
        self.drain()
        if hasattr(self.logger, "close"):
            self.logger.close()
