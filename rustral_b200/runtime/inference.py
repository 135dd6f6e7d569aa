"""InferencePool: a bounded queue in front of worker threads (crates/runtime/src/inference.rs:22-76).
`infer` blocks for the reply; a full queue applies back-pressure to callers."""
from __future__ import annotations

import queue
import threading


class PoolClosed(RuntimeError):
    pass


class InferencePool:
    def __init__(self, workers: int, queue_bound: int, handler):
        self._q: queue.Queue = queue.Queue(maxsize=max(1, queue_bound))
        self._handler = handler
        self._closed = False
        self._threads = [threading.Thread(target=self._run, daemon=True) for _ in range(max(1, workers))]
        for t in self._threads:
            t.start()

    def _run(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            inp, box, ev = item
            try:
                box.append((True, self._handler(inp)))
            except BaseException as e:   # noqa: BLE001 - delivered to the caller
                box.append((False, e))
            ev.set()

    def infer(self, inp, timeout: float | None = None):
        if self._closed:
            raise PoolClosed("pool is shut down")
        box, ev = [], threading.Event()
        self._q.put((inp, box, ev), timeout=timeout)
        if not ev.wait(timeout):
            raise TimeoutError("inference timed out")
        ok, val = box[0]
        if not ok:
            raise val
        return val

    def shutdown(self):
        if self._closed:
            return
        self._closed = True
        for _ in self._threads:
            self._q.put(None)
        for t in self._threads:
            t.join(timeout=5)
